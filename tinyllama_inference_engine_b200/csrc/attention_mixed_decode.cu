// Attention with mixed heads for steps of few rows (decoded tokens) on the tensor cores, bfloat16: the mathematics of
// attention_mixed.cu, with the two products of a key tile as MMAs and the mix between them in 32-bit.
//
// A CTA owns one query token and a run of its key tiles (32 keys each; gridDim.y CTAs share a row's tiles, as in the general
// kernel, and merge_mixed_decode_kernel puts their parts together).  The heads of one key/value head are the 16 rows of an MMA
// (a group of fewer heads leaves rows empty), so per tile and key/value head
//   raw  [16 heads x 32 keys] = Q_c [16 x KEY_DIM] . K_c^T          (mma.sync m16n8k16, 32-bit accumulators)
// goes to shared memory with scale and distance bias applied; the heads' scores are mixed there in 32-bit (a warp per head, a
// lane per key) with the running maximum and sum of the softmax; the weights go back as bfloat16 and
//   out  [16 heads x VALUE_DIM] += P_c [16 x 32] . V_c [32 x VALUE_DIM]
// accumulates in registers across the tiles.  Nothing of the scores is rounded before the softmax.
//
// Compile-time: KEY_DIM, VALUE_DIM (multiples of 16), KV_HEADS.  Heads per key/value head: at most 16.
#include "common.cuh"
#include "mma_utils.cuh"

#ifndef KEY_DIM
#define KEY_DIM 64
#endif
#ifndef VALUE_DIM
#define VALUE_DIM 64
#endif
#ifndef KV_HEADS
#define KV_HEADS 4
#endif

namespace tlie {

constexpr int kD = KEY_DIM, kVD = VALUE_DIM, kG = KV_HEADS;
constexpr int kKeys = 32;
constexpr int kWarps = 4, kThreads = kWarps * 32;
constexpr int kGroupsPerWarp = (kG + kWarps - 1) / kWarps;
constexpr int kQRow = kD + 8, kKRow = kD + 8, kVRow = kVD + 8, kPRow = kKeys + 8;   // padded shared-memory rows (elements)

struct DecodeSmem {
  // byte offsets of the sections for ``heads`` query heads
  size_t q, k, v, p, raw, mix, stats, rows, total;
  __host__ __device__ explicit DecodeSmem(int heads, bool mixed) {
    size_t at = 0;
    rows = at;  at += 2 * kKeys * sizeof(long long);                          // where a key's row starts in its plane, keys and values
    q = at;     at += (size_t)kG * 16 * kQRow * sizeof(__nv_bfloat16);         // [kv head][16 heads][kQRow]
    k = at;     at += (size_t)kG * kKeys * kKRow * sizeof(__nv_bfloat16);      // [kv head][32 keys][kKRow]
    v = at;     at += (size_t)kG * kKeys * kVRow * sizeof(__nv_bfloat16);      // [kv head][32 keys][kVRow]
    p = at;     at += (size_t)kG * 16 * kPRow * sizeof(__nv_bfloat16);         // [kv head][16 heads][kPRow]
    raw = at;   at += (size_t)heads * kKeys * sizeof(float);                   // [head][32 keys]
    mix = at;   at += mixed ? (size_t)heads * heads * sizeof(float) : 0;
    stats = at; at += 3 * (size_t)heads * sizeof(float);                       // running maximum, running sum, this tile's shrink
    total = (at + 15) / 16 * 16;
  }
};

__global__ void __launch_bounds__(kThreads)
    mixed_decode_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, int gate_offset, const __nv_bfloat16* __restrict__ k_pages,
                        long long k_page_stride, const __nv_bfloat16* __restrict__ v_pages, long long v_page_stride, const int* __restrict__ positions,
                        const int* __restrict__ token_seq, const int* __restrict__ block_table, int table_stride, const float* __restrict__ slopes,
                        const float* __restrict__ mix, __nv_bfloat16* __restrict__ out, int heads, int page_size, int window, float scale,
                        float* __restrict__ partial, int keep_first, int gate_per_head) {
  extern __shared__ __align__(16) unsigned char smem[];
  const DecodeSmem at(heads, mix != nullptr);
  long long* k_at = reinterpret_cast<long long*>(smem + at.rows);
  long long* v_at = k_at + kKeys;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem + at.q);
  __nv_bfloat16* k_t = reinterpret_cast<__nv_bfloat16*>(smem + at.k);
  __nv_bfloat16* v_t = reinterpret_cast<__nv_bfloat16*>(smem + at.v);
  __nv_bfloat16* p_s = reinterpret_cast<__nv_bfloat16*>(smem + at.p);
  float* raw_s = reinterpret_cast<float*>(smem + at.raw);
  float* mix_s = reinterpret_cast<float*>(smem + at.mix);
  float* max_s = reinterpret_cast<float*>(smem + at.stats);
  float* sum_s = max_s + heads;
  float* shrink_s = sum_s + heads;

  const int t = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int group = heads / kG;
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_seq[t] * table_stride;
  const __nv_bfloat16* row = rows + (size_t)t * row_stride;

  // queries: the heads of key/value head c are rows 0 .. group - 1 of its 16-row block, the rest zero
  constexpr int kQChunks = kD / 8;
  for (int i = tid; i < kG * 16 * kQChunks; i += kThreads) {
    const int chunk = i % kQChunks, r = i / kQChunks;
    const int c = r >> 4, in_group = r & 15;
    uint4 value = make_uint4(0u, 0u, 0u, 0u);
    if (in_group < group) value = *reinterpret_cast<const uint4*>(row + (size_t)(c * group + in_group) * kD + chunk * 8);
    *reinterpret_cast<uint4*>(q_s + (size_t)r * kQRow + chunk * 8) = value;
  }
  for (int i = tid; i < kG * 16 * kPRow / 2; i += kThreads) reinterpret_cast<unsigned*>(p_s)[i] = 0u;   // rows of no head stay zero
  if (mix)
    for (int i = tid; i < heads * heads; i += kThreads) mix_s[i] = mix[i];
  for (int i = tid; i < heads; i += kThreads) {
    max_s[i] = -INFINITY;
    sum_s[i] = 0.0f;
  }

  float o[kGroupsPerWarp][kVD / 8][4];
#pragma unroll
  for (int u = 0; u < kGroupsPerWarp; ++u)
#pragma unroll
    for (int i = 0; i < kVD / 8; ++i) o[u][i][0] = o[u][i][1] = o[u][i][2] = o[u][i][3] = 0.0f;

  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // The visible keys are numbered 0, 1, ...: first the ``kept`` keys that stay visible behind the window, then the window's.
  const int kept = min(keep_first, lo);
  const int visible = kept + (pos - lo + 1);
  const int splits = gridDim.y;
  const int tiles = (visible + kKeys - 1) / kKeys;
  const int tiles_each = (tiles + splits - 1) / splits;
  const int first_key = blockIdx.y * tiles_each * kKeys;
  const int last_key = min(visible - 1, first_key + tiles_each * kKeys - 1);

  for (int base = first_key; base <= last_key; base += kKeys) {
    const int count = min(kKeys, last_key - base + 1);
    __syncthreads();   // the tile before is done with its rows, keys and values (and, the first time, the queries are in place)
    if (tid < count) {
      const int key = base + tid < kept ? base + tid : lo + (base + tid - kept);
      const long long page = table[key / page_size];
      const int slot = key % page_size;
      k_at[tid] = page * k_page_stride + (long long)slot * kD;
      v_at[tid] = page * v_page_stride + (long long)slot * kVD;
    }
    __syncthreads();
    // the tile's keys and values of every key/value head; keys past the run's end are zero (their weights are zero too)
    constexpr int kKChunks = kD / 8, kVChunks = kVD / 8;
    // asynchronous copies: all of a thread's rows are in flight together (a load into a register followed by its store would wait
    // for the row before it, since the compiler cannot tell the store from the next row's address in shared memory)
    for (int i = tid; i < kG * kKeys * kKChunks; i += kThreads) {
      const int chunk = i % kKChunks, j = (i / kKChunks) % kKeys, c = i / (kKChunks * kKeys);
      const bool valid = j < count;
      cp_async_16(k_t + ((size_t)c * kKeys + j) * kKRow + chunk * 8, valid ? k_pages + k_at[j] + (size_t)c * page_size * kD + chunk * 8 : k_pages, valid);
    }
    for (int i = tid; i < kG * kKeys * kVChunks; i += kThreads) {
      const int chunk = i % kVChunks, j = (i / kVChunks) % kKeys, c = i / (kVChunks * kKeys);
      const bool valid = j < count;
      cp_async_16(v_t + ((size_t)c * kKeys + j) * kVRow + chunk * 8, valid ? v_pages + v_at[j] + (size_t)c * page_size * kVD + chunk * 8 : v_pages, valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    // raw scores of every key/value head's heads: a warp per key/value head
#pragma unroll
    for (int u = 0; u < kGroupsPerWarp; ++u) {
      const int c = warp + u * kWarps;
      if (c < kG) {
        float s[kKeys / 8][4];
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
          unsigned qa[4];
          ldmatrix_x4(qa, q_s + (size_t)(c * 16 + (lane & 15)) * kQRow + ks * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int jp = 0; jp < kKeys / 16; ++jp) {
            unsigned b[4];
            const int r = (jp * 2 + (lane >> 4)) * 8 + (lane & 7);
            ldmatrix_x4(b, k_t + ((size_t)c * kKeys + r) * kKRow + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[jp * 2], qa, b[0], b[1]);
            mma_bf16(s[jp * 2 + 1], qa, b[2], b[3]);
          }
        }
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int in_group = g + (e >> 1) * 8, key = j * 8 + 2 * tq + (e & 1);
            if (in_group < group) {
              const int h = c * group + in_group;
              float raw = s[j][e] * scale;
              if (slopes) raw -= slopes[h] * (float)(pos - (base + key < kept ? base + key : lo + (base + key - kept)));
              raw_s[h * kKeys + key] = raw;
            }
          }
      }
    }
    __syncthreads();
    // the heads' scores mixed, the softmax's running maximum and sum, and the weights as bfloat16: a warp per head, a lane per key
    for (int h = warp; h < heads; h += kWarps) {
      float score;
      if (mix) {
        // four sums side by side: one chain of dependent adds would wait for every load in turn
        float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float* weights = mix_s + h * heads;
        int q = 0;
#pragma unroll 2
        for (; q + 4 <= heads; q += 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) part[i] += weights[q + i] * raw_s[(q + i) * kKeys + lane];
        }
        for (; q < heads; ++q) part[0] += weights[q] * raw_s[q * kKeys + lane];
        score = (part[0] + part[1]) + (part[2] + part[3]);
      } else {
        score = raw_s[h * kKeys + lane];
      }
      if (lane >= count) score = -INFINITY;
      const float before = max_s[h];
      const float now = fmaxf(before, warp_max(score));
      const float shrink = expf(before - now);   // exp(-inf) = 0 on the first tile
      const float p = lane < count ? expf(score - now) : 0.0f;
      const float total = warp_sum(p);
      p_s[(size_t)((h / group) * 16 + h % group) * kPRow + lane] = __float2bfloat16_rn(p);
      __syncwarp();
      if (lane == 0) {
        max_s[h] = now;
        sum_s[h] = sum_s[h] * shrink + total;
        shrink_s[h] = shrink;
      }
    }
    __syncthreads();
    // weights times values: the warp of a key/value head adds the tile into its heads' outputs
#pragma unroll
    for (int u = 0; u < kGroupsPerWarp; ++u) {
      const int c = warp + u * kWarps;
      if (c < kG) {
        const float shrink_lo = g < group ? shrink_s[c * group + g] : 0.0f, shrink_hi = g + 8 < group ? shrink_s[c * group + g + 8] : 0.0f;
#pragma unroll
        for (int i = 0; i < kVD / 8; ++i) {
          o[u][i][0] *= shrink_lo;
          o[u][i][1] *= shrink_lo;
          o[u][i][2] *= shrink_hi;
          o[u][i][3] *= shrink_hi;
        }
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk) {
          unsigned pa[4];
          ldmatrix_x4(pa, p_s + (size_t)(c * 16 + (lane & 15)) * kPRow + kk * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int np = 0; np < kVD / 16; ++np) {
            unsigned b[4];
            const int r = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
            ldmatrix_x4_trans(b, v_t + ((size_t)c * kKeys + r) * kVRow + np * 16 + (lane >> 4) * 8);
            mma_bf16(o[u][np * 2], pa, b[0], b[1]);
            mma_bf16(o[u][np * 2 + 1], pa, b[2], b[3]);
          }
        }
      }
    }
  }
  __syncthreads();
  const int outputs = heads * kVD;
  float* mine = splits > 1 ? partial + ((size_t)t * splits + blockIdx.y) * (outputs + 2 * heads) : nullptr;
  if (mine != nullptr)
    for (int i = tid; i < heads; i += kThreads) {
      mine[outputs + i] = max_s[i];
      mine[outputs + heads + i] = sum_s[i];
    }
#pragma unroll
  for (int u = 0; u < kGroupsPerWarp; ++u) {
    const int c = warp + u * kWarps;
    if (c >= kG) continue;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int in_group = g + half * 8;
      if (in_group >= group) continue;
      const int h = c * group + in_group;
      const float inv = mine != nullptr ? 1.0f : 1.0f / sum_s[h];
#pragma unroll
      for (int i = 0; i < kVD / 8; ++i) {
        const int d = i * 8 + 2 * tq;
        float a = o[u][i][half * 2] * inv, b = o[u][i][half * 2 + 1] * inv;
        if (mine != nullptr) {
          mine[h * kVD + d] = a;
          mine[h * kVD + d + 1] = b;
        } else {
          if (gate_offset >= 0 && gate_per_head) {
            const float gate = 1.0f / (1.0f + expf(-__bfloat162float(row[gate_offset + h])));
            a *= gate;
            b *= gate;
          } else if (gate_offset >= 0) {
            const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(row + gate_offset + h * kVD + d);
            a *= 1.0f / (1.0f + expf(-__bfloat162float(gv.x)));
            b *= 1.0f / (1.0f + expf(-__bfloat162float(gv.y)));
          }
          *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * outputs + h * kVD + d) = __floats2bfloat162_rn(a, b);
        }
      }
    }
  }
}

// The parts of a row put together (see merge_mixed_kernel of the general kernel): a CTA per (row, head), a thread per output.
__global__ void merge_mixed_decode_kernel(const float* __restrict__ partial, const __nv_bfloat16* __restrict__ rows, int row_stride, int gate_offset,
                                          __nv_bfloat16* __restrict__ out, int heads, int splits, int gate_per_head) {
  __shared__ float weight_s[64];   // at most 64 parts: each part's e^(max - highest)
  __shared__ float scratch[2];
  const int t = blockIdx.x, h = blockIdx.y;
  const int outputs = heads * kVD;
  const size_t part_size = (size_t)outputs + 2 * heads;
  const float* mine = partial + (size_t)t * splits * part_size;
  if (threadIdx.x < 32) {   // one warp: a lane per part (two at most), all loads in one round trip
    const int lane = threadIdx.x;
    float top[2], sum[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int s = lane + 32 * i;
      top[i] = s < splits ? mine[s * part_size + outputs + h] : -INFINITY;
      sum[i] = s < splits ? mine[s * part_size + outputs + heads + h] : 0.0f;
    }
    const float highest = warp_max(fmaxf(top[0], top[1]));
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float weight = expf(top[i] - highest);   // a part that saw no key has maximum -inf: weight 0
      if (lane + 32 * i < splits) weight_s[lane + 32 * i] = weight;
      total += sum[i] * weight;
    }
    total = warp_sum(total);
    if (lane == 0) scratch[0] = 1.0f / total;
  }
  __syncthreads();
  const float inv = scratch[0];
  for (int d = threadIdx.x; d < kVD; d += blockDim.x) {
    const int o = h * kVD + d;
    float value[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) value[i] += mine[(s + i) * part_size + o] * weight_s[s + i];
    }
    for (; s < splits; ++s) value[0] += mine[s * part_size + o] * weight_s[s];
    float v = ((value[0] + value[1]) + (value[2] + value[3])) * inv;
    if (gate_offset >= 0) v *= 1.0f / (1.0f + expf(-__bfloat162float(rows[(size_t)t * row_stride + gate_offset + (gate_per_head ? h : o)])));
    out[(size_t)t * outputs + o] = __float2bfloat16_rn(v);
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT long long tlie_mixed_decode_smem_bytes(int heads, int mixed) { return (long long)DecodeSmem(heads, mixed != 0).total; }

// ``splits`` > 1: ``partial`` holds tokens * splits * (heads * VALUE_DIM + 2 * heads) floats.
TLIE_EXPORT int tlie_mixed_decode(const void* rows, int row_stride, int gate_offset, const void* k_pages, long long k_page_stride, const void* v_pages,
                                  long long v_page_stride, const int* positions, const int* token_seq, const int* block_table, int table_stride,
                                  const float* slopes, const float* mix, void* out, int tokens, int heads, int page_size, int window, float scale, int splits,
                                  float* partial, int keep_first, int gate_per_head, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (keep_first < 0) return (int)cudaErrorInvalidValue;
  if (heads <= 0 || heads % kG != 0 || heads / kG > 16 || row_stride % 8 != 0 || (gate_offset >= 0 && !gate_per_head && gate_offset % 2 != 0) || splits < 1 || splits > 64 ||
      (splits > 1 && partial == nullptr))
    return (int)cudaErrorInvalidValue;
  const size_t smem = DecodeSmem(heads, mix != nullptr).total;
  if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    const cudaError_t set = cudaFuncSetAttribute(mixed_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (set != cudaSuccess) return (int)set;
  }
  mixed_decode_kernel<<<dim3(tokens, splits), kThreads, smem, stream>>>((const __nv_bfloat16*)rows, row_stride, gate_offset, (const __nv_bfloat16*)k_pages,
                                                                       k_page_stride, (const __nv_bfloat16*)v_pages, v_page_stride, positions, token_seq,
                                                                       block_table, table_stride, slopes, mix, (__nv_bfloat16*)out, heads, page_size, window,
                                                                       scale, partial, window > 0 ? keep_first : 0, gate_per_head);
  if (splits > 1)
    merge_mixed_decode_kernel<<<dim3(tokens, heads), kVD >= 128 ? 128 : (kVD > 32 ? 64 : 32), 0, stream>>>(partial, (const __nv_bfloat16*)rows, row_stride,
                                                                                                        gate_offset, (__nv_bfloat16*)out, heads, splits, gate_per_head);
  return (int)cudaGetLastError();
}
