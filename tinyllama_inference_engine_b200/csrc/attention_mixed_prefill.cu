// Attention with mixed heads for prompt portions on the tensor cores, bfloat16 (the mathematics of attention_mixed.cu).
//
// The mix is linear in the raw scores, so it can be applied to the queries instead of the scores:
//   mixed_h(i, j) = sum_g M[h, g] ((q_g . k_{c(g)}) * scale - slope_g (i - j))
//                 = sum_c Q'_{h, c} . k_c(j)  -  slope'_h (i - j)
// with Q'_{h, c} = scale * sum_{g in group c} M[h, g] q_g (one folded query per head and key/value head, made by
// fold_queries_kernel in 32-bit and rounded to bfloat16 once) and slope'_h = sum_g M[h, g] slope_g (made on the host).  Head h
// is then ordinary flash attention whose query is the concatenation of its PARTS folded queries and whose key is the
// concatenation of the token's PARTS key heads: nothing of the scores is ever mixed outside the tensor cores.  Without a mix
// PARTS is 1 and the query is the head's own.
//
// One CTA per (tile of rows of one request, head), one warp per 16 rows; keys and values stream through shared memory in
// 64-key tiles (cp.async, a ring of chunks); Q'.K^T and P.V on mma.sync m16n8k16 with 32-bit accumulators, the
// distance bias, the mask, the running maximum and sum in 32-bit; the output gate in the epilogue.
//
// Compile-time: KEY_DIM, VALUE_DIM (multiples of 16), PARTS (key heads per folded query).
#include "common.cuh"
#include "mma_utils.cuh"

#ifndef KEY_DIM
#define KEY_DIM 64
#endif
#ifndef VALUE_DIM
#define VALUE_DIM 64
#endif
#ifndef PARTS
#define PARTS 1
#endif

namespace tlie {

constexpr int kD = KEY_DIM, kVD = VALUE_DIM, kParts = PARTS;
constexpr int kKeys = 64;
constexpr int kKRow = kD + 8, kVRow = kVD + 8, kQRow = kParts * kD + 8;   // padded shared-memory rows (elements)
constexpr size_t kSmemLimit = 227 * 1024;
// Keys pass through shared memory in chunks of a 64-key tile: all PARTS key heads at once with the next tile's chunk in flight (a ring
// of two) where that fits beside 128 rows of folded queries, else one key head at a time with two chunks in flight (a ring of three).
// Values pass one tile at a time: two buffers, or as many as the ring where a tile is a single chunk, so that a tile issued ahead
// never lands in a buffer still being read.  The folded queries of the CTA's rows stay resident.
constexpr size_t smem_for(int rows, int parts_per_chunk) {
  const int ring = parts_per_chunk == kParts ? 2 : 3;
  const int v_buffers = parts_per_chunk == kParts ? ring : 2;
  return ((size_t)rows * kQRow + (size_t)ring * parts_per_chunk * kKeys * kKRow + (size_t)v_buffers * kKeys * kVRow) * sizeof(__nv_bfloat16);
}
constexpr bool fits(int rows, int parts_per_chunk) { return smem_for(rows, parts_per_chunk) <= kSmemLimit; }
// rows per CTA: the most that fit shared memory, whole tiles before single key heads; 0 if nothing fits (the host then uses the general kernel)
constexpr int kRows = (fits(128, kParts) || fits(128, 1)) ? 128 : (fits(64, kParts) || fits(64, 1)) ? 64 : (fits(32, kParts) || fits(32, 1)) ? 32 : fits(16, 1) ? 16 : 0;
constexpr int kPartsPerChunk = fits(kRows > 0 ? kRows : 16, kParts) ? kParts : 1;
constexpr int kChunksPerTile = kParts / kPartsPerChunk;
constexpr int kRing = kPartsPerChunk == kParts ? 2 : 3;
constexpr int kVBuffers = kChunksPerTile == 1 ? kRing : 2;
constexpr size_t kChunkElements = (size_t)kPartsPerChunk * kKeys * kKRow;
constexpr int kWarps = kRows > 0 ? kRows / 16 : 1;
constexpr int kThreads = kWarps * 32;
constexpr float kLog2e = 1.4426950408889634f;

// folded[t, h, p, :] = scale * sum over the query heads g of key/value head c(p) of M[h, g] q[t, g, :]   (no mix: scale * q[t, h, :])
// A CTA per token: its queries and the mixing matrix wait in shared memory, a thread takes outputs of one (head, part) at
// neighbouring elements, so a warp reads one mixing weight (broadcast) and 32 neighbouring query elements per step.
__global__ void __launch_bounds__(256) fold_queries_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, const float* __restrict__ mix, float scale,
                                                           __nv_bfloat16* __restrict__ folded, int heads, int group) {
  extern __shared__ float fold_smem[];
  float* q_s = fold_smem;                 // [heads][kD]
  float* mix_s = q_s + heads * kD;        // [heads][heads]
  const int t = blockIdx.x;
  const __nv_bfloat16* q = rows + (size_t)t * row_stride;
  __nv_bfloat16* dst = folded + (size_t)t * heads * kParts * kD;
  for (int i = threadIdx.x; i < heads * kD / 2; i += blockDim.x) {
    const float2 pair = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(q)[i]);
    q_s[2 * i] = pair.x;
    q_s[2 * i + 1] = pair.y;
  }
  if (mix != nullptr)
    for (int i = threadIdx.x; i < heads * heads; i += blockDim.x) mix_s[i] = mix[i];
  __syncthreads();
  for (int i = threadIdx.x; i < heads * kParts * kD; i += blockDim.x) {
    const int d = i % kD, p = (i / kD) % kParts, h = i / (kD * kParts);
    float sum;
    if (mix == nullptr) {
      sum = q_s[h * kD + d];
    } else {
      float part[2] = {0.0f, 0.0f};
      const float* weights = mix_s + h * heads + p * group;
      const float* column = q_s + (size_t)p * group * kD + d;
      int g = 0;
      for (; g + 2 <= group; g += 2) {
        part[0] += weights[g] * column[g * kD];
        part[1] += weights[g + 1] * column[(g + 1) * kD];
      }
      if (g < group) part[0] += weights[g] * column[g * kD];
      sum = part[0] + part[1];
    }
    dst[i] = __float2bfloat16_rn(sum * scale);
  }
}

// where the four 16-key quarters of a tile lie: a page holds a multiple of 16 keys, so each quarter lies in one page
struct TileRows {
  long long page[kKeys / 16];
  int slot[kKeys / 16];
};

__device__ __forceinline__ TileRows tile_rows(const int* table, int key0, int lo, int n_keys, int page_size, int keep) {
  TileRows rows;
#pragma unroll
  for (int h = 0; h < kKeys / 16; ++h) {
    const int k = key0 + 16 * h;
    const bool any = k < n_keys && (k + 16 > lo || k < keep);
    rows.page[h] = any ? table[k / page_size] : 0;
    rows.slot[h] = k % page_size;
  }
  return rows;
}

// one plane's rows of a tile for one head: [64][row] in shared memory, ``width`` elements each
template <int WIDTH, int ROW>
__device__ __forceinline__ void load_plane(__nv_bfloat16* smem, const __nv_bfloat16* pages, long long page_stride, const TileRows& rows, int key0, int lo,
                                           int n_keys, int head, int page_size, int keep) {
  constexpr int kChunks = WIDTH / 8;
  for (int idx = threadIdx.x; idx < kKeys * kChunks; idx += kThreads) {
    const int chunk = idx % kChunks, row = idx / kChunks;
    const int key = key0 + row, quarter = row >> 4;
    const bool valid = (key >= lo || key < keep) && key < n_keys;
    const long long page = quarter == 0 ? rows.page[0] : quarter == 1 ? rows.page[1] : quarter == 2 ? rows.page[2] : rows.page[3];
    const int slot = (quarter == 0 ? rows.slot[0] : quarter == 1 ? rows.slot[1] : quarter == 2 ? rows.slot[2] : rows.slot[3]) + (row & 15);
    const __nv_bfloat16* src = pages + page * page_stride + ((size_t)head * page_size + slot) * WIDTH + chunk * 8;
    cp_async_16(smem + (size_t)row * ROW + chunk * 8, valid ? src : pages, valid);
  }
}

// two CTAs on an SM where shared memory has room for both and the output accumulators leave the registers for it
constexpr int kMinBlocks = (kRows > 0 && 2 * smem_for(kRows > 0 ? kRows : 16, kPartsPerChunk) <= kSmemLimit && kVD <= 64) ? 2 : 1;

__global__ void __launch_bounds__(kThreads, kMinBlocks)
    mixed_prefill_kernel(const __nv_bfloat16* __restrict__ folded, const __nv_bfloat16* __restrict__ rows, int row_stride, int gate_offset,
                         const __nv_bfloat16* __restrict__ k_pages, long long k_page_stride, const __nv_bfloat16* __restrict__ v_pages,
                         long long v_page_stride, const int* __restrict__ seq_starts, const int* __restrict__ first_positions,
                         const int* __restrict__ block_table, int table_stride, const float* __restrict__ slopes, __nv_bfloat16* __restrict__ out,
                         int heads, int kv_heads, int page_size, int window, int mixed, int keep_first, int gate_per_head) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [kRows][kQRow]
  __nv_bfloat16* k_ring = q_smem + (size_t)kRows * kQRow;                        // [kRing][kPartsPerChunk][64][kKRow]
  __nv_bfloat16* v_ring = k_ring + (size_t)kRing * kChunkElements;               // [kVBuffers][64][kVRow]
  const int seq = blockIdx.y, head = blockIdx.z;
  const int seq_start = seq_starts[seq];
  const int q_len = seq_starts[seq + 1] - seq_start;
  const int row_in_seq = (gridDim.x - 1 - blockIdx.x) * kRows;   // later tiles see more keys: they start first
  if (row_in_seq >= q_len) return;
  const int row0 = seq_start + row_in_seq;
  const int kvh = head / (heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rows_here = min(kRows, q_len - row_in_seq);
  const int pos0 = first_positions[seq] + row_in_seq;
  const int last_pos = pos0 + rows_here - 1;
  const int n_keys = last_pos + 1;
  const int lo_tile = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int* table = block_table + (size_t)seq * table_stride;
  const float slope = slopes ? slopes[head] * kLog2e : 0.0f;

  constexpr int kQChunks = kParts * kD / 8;
  for (int idx = threadIdx.x; idx < kRows * kQChunks; idx += kThreads) {
    const int row = idx / kQChunks, chunk = idx - row * kQChunks;
    const bool valid = row < rows_here;
    const __nv_bfloat16* src = folded + ((size_t)(row0 + (valid ? row : 0)) * heads + head) * (kParts * kD) + chunk * 8;
    cp_async_16(q_smem + (size_t)row * kQRow + chunk * 8, src, valid);
  }

  const int first_tile = lo_tile / kKeys;
  const int end_tile = (n_keys + kKeys - 1) / kKeys;
  // With a window, the keys below ``keep`` stay visible behind it: the tiles that hold them and lie before the window's first tile
  // come first (those from the window's first tile on are loaded anyway; a key is masked per row).
  const int keep = window > 0 ? keep_first : 0;
  const int kept_tiles = min((keep + kKeys - 1) / kKeys, first_tile);
  const int chunks = (kept_tiles + end_tile - first_tile) * kChunksPerTile;   // chunk c: key heads [c % per tile * kPartsPerChunk, ...) of the (c / per tile)-th tile
  auto tile_of = [&](int c) { const int n = c / kChunksPerTile; return n < kept_tiles ? n : first_tile + (n - kept_tiles); };
  auto issue = [&](int c) {
    if (c < chunks) {
      const int tile = tile_of(c), first_part = (c % kChunksPerTile) * kPartsPerChunk;
      const TileRows rows_of = tile_rows(table, tile * kKeys, lo_tile, n_keys, page_size, keep);
#pragma unroll
      for (int i = 0; i < kPartsPerChunk; ++i)
        load_plane<kD, kKRow>(k_ring + (size_t)(c % kRing) * kChunkElements + (size_t)i * kKeys * kKRow, k_pages, k_page_stride, rows_of, tile * kKeys, lo_tile, n_keys,
                              mixed ? first_part + i : kvh, page_size, keep);
      if (first_part == 0)
        load_plane<kVD, kVRow>(v_ring + (size_t)((c / kChunksPerTile) % kVBuffers) * kKeys * kVRow, v_pages, v_page_stride, rows_of, tile * kKeys, lo_tile, n_keys, kvh,
                               page_size, keep);
    }
    cp_async_commit();   // a group per chunk, empty past the end, so that the count of groups in flight is the same at every step
  };
  issue(0);   // in one group with the folded queries
  if (kRing == 3) issue(1);

  const int my_row[2] = {warp * 16 + g, warp * 16 + g + 8};
  int my_pos[2], my_lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    my_pos[r] = pos0 + min(my_row[r], rows_here - 1);   // rows past the end behave like the last row; never stored
    my_lo[r] = (window > 0 && my_pos[r] - window + 1 > 0) ? my_pos[r] - window + 1 : 0;
  }
  float o[kVD / 8][4];
#pragma unroll
  for (int i = 0; i < kVD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.0f, 0.0f};

  float s_frag[kKeys / 8][4];
  for (int c = 0; c < chunks; ++c) {
    issue(c + kRing - 1);
    cp_async_wait<kRing - 1>();   // everything but the chunks issued ahead has landed: chunk c, and its tile's values
    __syncthreads();
    const int tile = tile_of(c), first_part = (c % kChunksPerTile) * kPartsPerChunk;
    const __nv_bfloat16* k_smem = k_ring + (size_t)(c % kRing) * kChunkElements;
    const __nv_bfloat16* v_smem = v_ring + (size_t)((c / kChunksPerTile) % kVBuffers) * kKeys * kVRow;
    const int key0 = tile * kKeys;
    const int warp_last_pos = pos0 + min(warp * 16 + 15, rows_here - 1);
    const int warp_first_pos = pos0 + min(warp * 16, rows_here - 1);
    const int warp_lo = (window > 0 && warp_first_pos - window + 1 > 0) ? warp_first_pos - window + 1 : 0;
    const bool tile_seen = key0 <= warp_last_pos && (key0 + kKeys > warp_lo || key0 < keep);   // some row of this warp sees some key of this tile
    if (tile_seen) {
      if (first_part == 0) {
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) s_frag[j][0] = s_frag[j][1] = s_frag[j][2] = s_frag[j][3] = 0.0f;
      }
#pragma unroll 1
      for (int i = 0; i < kPartsPerChunk; ++i) {
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
          unsigned qa[4];
          ldmatrix_x4(qa, q_smem + (size_t)(warp * 16 + (lane & 15)) * kQRow + (first_part + i) * kD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int jp = 0; jp < kKeys / 16; ++jp) {
            unsigned b[4];
            const int row = (jp * 2 + (lane >> 4)) * 8 + (lane & 7);
            const int col = ks * 16 + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(b, k_smem + ((size_t)i * kKeys + row) * kKRow + col);
            mma_bf16(s_frag[jp * 2], qa, b[0], b[1]);
            mma_bf16(s_frag[jp * 2 + 1], qa, b[2], b[3]);
          }
        }
      }
    }
    if (first_part + kPartsPerChunk == kParts && tile_seen) {
      // scores in units of log2: (dot - slope (i - j)) log2 e; keys outside a row's window or after it are masked
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < kKeys / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + j * 8 + 2 * t + (e & 1);
          const int r = e >> 1;
          const float v = ((key >= my_lo[r] || key < keep) && key <= my_pos[r]) ? fmaf(s_frag[j][e], kLog2e, -slope * (float)(my_pos[r] - key)) : -INFINITY;
          s_frag[j][e] = v;
          tile_max[r] = fmaxf(tile_max[r], v);
        }
      }
      float rescale[2], base[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float new_max = fmaxf(row_max[r], tile_max[r]);
        base[r] = (new_max == -INFINITY) ? 0.0f : new_max;   // a row may see no key of an early tile
        rescale[r] = exp2f(row_max[r] - base[r]);
        row_max[r] = new_max;
        row_sum[r] *= rescale[r];
      }
      unsigned pa[kKeys / 16][4];
#pragma unroll
      for (int j = 0; j < kKeys / 8; ++j) {
        const float p0 = exp2_approx(s_frag[j][0] - base[0]);
        const float p1 = exp2_approx(s_frag[j][1] - base[0]);
        const float p2 = exp2_approx(s_frag[j][2] - base[1]);
        const float p3 = exp2_approx(s_frag[j][3] - base[1]);
        row_sum[0] += p0 + p1;
        row_sum[1] += p2 + p3;
        pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
        pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int i = 0; i < kVD / 8; ++i) {
        o[i][0] *= rescale[0];
        o[i][1] *= rescale[0];
        o[i][2] *= rescale[1];
        o[i][3] *= rescale[1];
      }
#pragma unroll
      for (int kk = 0; kk < kKeys / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < kVD / 16; ++np) {
          unsigned b[4];
          const int row = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int col = np * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(b, v_smem + (size_t)row * kVRow + col);
          mma_bf16(o[np * 2], pa[kk], b[0], b[1]);
          mma_bf16(o[np * 2 + 1], pa[kk], b[2], b[3]);
        }
      }
    }
    __syncthreads();   // everyone is done with this chunk before the ring comes round to its buffer
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (my_row[r] >= rows_here) continue;
    const float inv = 1.0f / row_sum[r];
    const size_t row = (size_t)(row0 + my_row[r]);
    __nv_bfloat16* dst = out + (row * heads + head) * kVD + 2 * t;
    const __nv_bfloat16* gate = (gate_offset >= 0 && !gate_per_head) ? rows + row * row_stride + gate_offset + (size_t)head * kVD + 2 * t : nullptr;
    const float head_gate = (gate_offset >= 0 && gate_per_head) ? 1.0f / (1.0f + __expf(-__bfloat162float(rows[row * row_stride + gate_offset + head]))) : 1.0f;
#pragma unroll
    for (int i = 0; i < kVD / 8; ++i) {
      float a = o[i][r * 2] * inv * head_gate, b = o[i][r * 2 + 1] * inv * head_gate;
      if (gate != nullptr) {
        const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(gate + i * 8);
        a *= 1.0f / (1.0f + __expf(-__bfloat162float(gv.x)));
        b *= 1.0f / (1.0f + __expf(-__bfloat162float(gv.y)));
      }
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(a, b);
    }
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_mixed_prefill_tile_rows() { return kRows; }
TLIE_EXPORT int tlie_mixed_prefill_folded_width() { return kParts * kD; }

// ``folded``: scratch for the folded queries, bfloat16 [tokens, heads, PARTS * KEY_DIM].  ``slopes``: the folded slopes (or null).
// ``mix`` null: PARTS must be 1.  ``longest``: the most rows any entry of the step has.
TLIE_EXPORT int tlie_mixed_prefill(const void* rows, int row_stride, int gate_offset, const float* mix, float scale, void* folded, const void* k_pages,
                                   long long k_page_stride, const void* v_pages, long long v_page_stride, const int* seq_starts,
                                   const int* first_positions, const int* block_table, int table_stride, const float* slopes, void* out, int tokens,
                                   int entries, int longest, int heads, int kv_heads, int page_size, int window, int keep_first, int gate_per_head,
                                   cudaStream_t stream) {
  if (tokens <= 0 || entries <= 0) return 0;
  if (keep_first < 0) return (int)cudaErrorInvalidValue;
  if (kRows == 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size % 16 != 0 || heads > 65535 || entries > 65535 ||
      (mix != nullptr ? kParts != kv_heads : kParts != 1) || row_stride % 8 != 0 || (gate_offset >= 0 && !gate_per_head && gate_offset % 2 != 0))
    return (int)cudaErrorInvalidValue;
  const size_t fold_smem = ((size_t)heads * kD + (mix != nullptr ? (size_t)heads * heads : 0)) * sizeof(float);
  if (fold_smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  if (fold_smem > 48 * 1024) {
    e = cudaFuncSetAttribute(fold_queries_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fold_smem);
    if (e != cudaSuccess) return (int)e;
  }
  fold_queries_kernel<<<tokens, 256, fold_smem, stream>>>((const __nv_bfloat16*)rows, row_stride, mix, scale, (__nv_bfloat16*)folded, heads, heads / kv_heads);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  constexpr size_t smem = smem_for(kRows > 0 ? kRows : 16, kPartsPerChunk);
  static bool configured = false;
  if (!configured) {
    e = cudaFuncSetAttribute(mixed_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tile_rows = kRows > 0 ? kRows : 16;
  const dim3 grid((longest + tile_rows - 1) / tile_rows, entries, heads);
  mixed_prefill_kernel<<<grid, kThreads, smem, stream>>>((const __nv_bfloat16*)folded, (const __nv_bfloat16*)rows, row_stride, gate_offset,
                                                         (const __nv_bfloat16*)k_pages, k_page_stride, (const __nv_bfloat16*)v_pages, v_page_stride,
                                                         seq_starts, first_positions, block_table, table_stride, slopes, (__nv_bfloat16*)out, heads,
                                                         kv_heads, page_size, window, mix != nullptr ? 1 : 0, keep_first, gate_per_head);
  return (int)cudaGetLastError();
}
