// Attention of many heads over ONE cached vector per token whose leading columns are also the values (latent attention with the
// keys' and values' expansions moved across it), for prompt portions on the tensor cores, bfloat16.
//
// Every head of a token reads the same cached rows, so the (token, head) pairs of a request's portion are simply the rows of
// one tall query matrix [tokens * heads, KEY_DIM] (which is how the queries lie in memory) against the request's cached rows
// [keys, KEY_DIM]; the values are the first VALUE_DIM columns of the same rows, so a key tile in shared memory serves both
// products and is fetched once.  Causal; softmax in 32-bit with an optional sink per head in the denominator.
//
// One CTA per 64 consecutive (token, head) rows of one request: 8 warps = 4 row tiles of 16 x 2 halves of the value columns.  The
// two warps of a row tile both work out its 16 x 32 scores (Q.K^T on mma.sync m16n8k16, 32-bit accumulators) and keep the running
// maximum and sum; each multiplies the weights with its half of the value columns, the accumulators (16 x VALUE_DIM / 2 per warp)
// staying in registers.  Keys stream through a ring of 32-key tiles (cp.async).
//
// Steps of few rows (decoded tokens): gridDim.z CTAs share a row tile's key tiles; each leaves its unnormalised sums, maxima and
// totals in ``partial`` ([token][part][heads * VALUE_DIM + 2 heads], as the general kernel's parts) and a merge kernel puts them
// together and adds the sink.
//
// Compile-time: KEY_DIM (a multiple of 16), VALUE_DIM (a multiple of 32, at most KEY_DIM).
#include "common.cuh"
#include "mma_utils.cuh"

#ifndef KEY_DIM
#define KEY_DIM 576
#endif
#ifndef VALUE_DIM
#define VALUE_DIM 512
#endif

namespace tlie {

constexpr int kD = KEY_DIM, kVD = VALUE_DIM, kHalf = VALUE_DIM / 2;
constexpr int kRows = 64, kKeys = 32, kThreads = 256;
constexpr int kRow = kD + 8;   // padded shared-memory row (elements)
constexpr size_t kSmemLimit = 227 * 1024;
constexpr size_t smem_with(int stages) { return ((size_t)kRows + (size_t)stages * kKeys) * kRow * sizeof(__nv_bfloat16); }
constexpr int kStages = smem_with(3) <= kSmemLimit ? 3 : 2;
constexpr bool kFits = smem_with(2) <= kSmemLimit && kD % 16 == 0 && kVD % 32 == 0 && kVD <= kD;
constexpr float kLog2e = 1.4426950408889634f;

__global__ void __launch_bounds__(kThreads, 1)
    latent_prefill_kernel(const __nv_bfloat16* __restrict__ queries, const __nv_bfloat16* __restrict__ pages, long long page_stride, const int* __restrict__ seq_starts,
                          const int* __restrict__ first_positions, const int* __restrict__ block_table, int table_stride, const float* __restrict__ sinks,
                          __nv_bfloat16* __restrict__ out, int heads, int page_size, float scale, float* __restrict__ partial) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [64][kRow]
  __nv_bfloat16* k_ring = q_smem + (size_t)kRows * kRow;                // [kStages][32][kRow]
  const int seq = blockIdx.y;
  const int seq_start = seq_starts[seq];
  const int total_rows = (seq_starts[seq + 1] - seq_start) * heads;     // (token, head) pairs of this request's portion
  const int row_in_seq = (gridDim.x - 1 - blockIdx.x) * kRows;          // later tiles see more keys: they start first
  if (row_in_seq >= total_rows) return;
  const int rows_here = min(kRows, total_rows - row_in_seq);
  const size_t row0 = (size_t)seq_start * heads + row_in_seq;           // first row of the tile in the query and output matrices
  const int first_pos = first_positions[seq];
  const int n_keys = first_pos + (row_in_seq + rows_here - 1) / heads + 1;   // the last row's position + 1
  const int* table = block_table + (size_t)seq * table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_m = warp >> 1, half = warp & 1;
  const int g = lane >> 2, t = lane & 3;

  constexpr int kChunks = kD / 8;
  for (int idx = threadIdx.x; idx < kRows * kChunks; idx += kThreads) {
    const int row = idx / kChunks, chunk = idx - row * kChunks;
    const bool valid = row < rows_here;
    cp_async_16(q_smem + (size_t)row * kRow + chunk * 8, queries + (row0 + (valid ? row : 0)) * kD + chunk * 8, valid);
  }
  const int all_tiles = (n_keys + kKeys - 1) / kKeys;
  const int tiles_each = (all_tiles + (int)gridDim.z - 1) / (int)gridDim.z;
  const int tile0 = blockIdx.z * tiles_each, tiles = min(all_tiles, tile0 + tiles_each);   // this CTA's tiles: [tile0, tiles)
  auto issue = [&](int tile) {
    if (tile < tiles) {
      __nv_bfloat16* dst = k_ring + (size_t)((tile - tile0) % kStages) * kKeys * kRow;
      for (int idx = threadIdx.x; idx < kKeys * kChunks; idx += kThreads) {
        const int row = idx / kChunks, chunk = idx - row * kChunks;
        const int key = tile * kKeys + row;
        const bool valid = key < n_keys;
        const long long page = valid ? table[key / page_size] : 0;
        cp_async_16(dst + (size_t)row * kRow + chunk * 8, pages + page * page_stride + (size_t)(key % page_size) * kD + chunk * 8, valid);
      }
    }
    cp_async_commit();   // a group per tile, empty past the end
  };
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(tile0 + s);   // the first group also holds the queries

  const int my_row[2] = {tile_m * 16 + g, tile_m * 16 + g + 8};
  int my_pos[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) my_pos[r] = first_pos + (row_in_seq + min(my_row[r], rows_here - 1)) / heads;   // rows past the end behave like the last row; never stored
  const int warp_last_pos = first_pos + (row_in_seq + min(tile_m * 16 + 15, rows_here - 1)) / heads;
  const float to_log2 = scale * kLog2e;

  float o[kHalf / 8][4];
#pragma unroll
  for (int i = 0; i < kHalf / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.0f, 0.0f};

  for (int tile = tile0; tile < tiles; ++tile) {
    cp_async_wait<kStages - 2>();   // this thread's copies of this tile have landed ...
    __syncthreads();                // ... and everyone's; and everyone is done with the tile before, whose buffer is written next
    issue(tile + kStages - 1);
    const __nv_bfloat16* k_smem = k_ring + (size_t)((tile - tile0) % kStages) * kKeys * kRow;
    const int key0 = tile * kKeys;
    if (key0 > warp_last_pos) continue;   // no row of this warp sees a key of this tile (nor of any later one)
    float s_frag[kKeys / 8][4];
#pragma unroll
    for (int j = 0; j < kKeys / 8; ++j) s_frag[j][0] = s_frag[j][1] = s_frag[j][2] = s_frag[j][3] = 0.0f;
#pragma unroll 4
    for (int ks = 0; ks < kD / 16; ++ks) {
      unsigned qa[4];
      ldmatrix_x4(qa, q_smem + (size_t)(tile_m * 16 + (lane & 15)) * kRow + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int jp = 0; jp < kKeys / 16; ++jp) {
        unsigned b[4];
        const int row = (jp * 2 + (lane >> 4)) * 8 + (lane & 7);
        const int col = ks * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(b, k_smem + (size_t)row * kRow + col);
        mma_bf16(s_frag[jp * 2], qa, b[0], b[1]);
        mma_bf16(s_frag[jp * 2 + 1], qa, b[2], b[3]);
      }
    }
    // scores in units of log2; keys after a row's own position are masked
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kKeys / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + j * 8 + 2 * t + (e & 1);
        const int r = e >> 1;
        const float v = key <= my_pos[r] ? s_frag[j][e] * to_log2 : -INFINITY;
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
      base[r] = (new_max == -INFINITY) ? 0.0f : new_max;
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
    for (int i = 0; i < kHalf / 8; ++i) {
      o[i][0] *= rescale[0];
      o[i][1] *= rescale[0];
      o[i][2] *= rescale[1];
      o[i][3] *= rescale[1];
    }
    // weights times values: the values are the first VALUE_DIM columns of the key rows; this warp takes its half of them
#pragma unroll
    for (int kk = 0; kk < kKeys / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < kHalf / 16; ++np) {
        unsigned b[4];
        const int row = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int col = half * kHalf + np * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(b, k_smem + (size_t)row * kRow + col);
        mma_bf16(o[np * 2], pa[kk], b[0], b[1]);
        mma_bf16(o[np * 2 + 1], pa[kk], b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
#pragma unroll
  if (partial != nullptr) {
    const int outputs = heads * kVD;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (my_row[r] >= rows_here) continue;
      const size_t row = row0 + my_row[r];
      const int h = (int)(row % heads);
      float* mine = partial + ((row / heads) * gridDim.z + blockIdx.z) * ((size_t)outputs + 2 * heads);
#pragma unroll
      for (int i = 0; i < kHalf / 8; ++i) {
        mine[h * kVD + half * kHalf + i * 8 + 2 * t] = o[i][r * 2];
        mine[h * kVD + half * kHalf + i * 8 + 2 * t + 1] = o[i][r * 2 + 1];
      }
      if (half == 0 && t == 0) {
        mine[outputs + h] = row_max[r] * 0.6931471805599453f;   // the parts' maxima are kept in natural units
        mine[outputs + heads + h] = row_sum[r];
      }
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (my_row[r] >= rows_here) continue;
    const size_t row = row0 + my_row[r];
    float total = row_sum[r];
    if (sinks != nullptr) total += exp2f(sinks[row % heads] * kLog2e - row_max[r]);   // the sink: a weight without a key, not scaled
    const float inv = 1.0f / total;
    __nv_bfloat16* dst = out + row * kVD + half * kHalf + 2 * t;
#pragma unroll
    for (int i = 0; i < kHalf / 8; ++i)
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][r * 2] * inv, o[i][r * 2 + 1] * inv);
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_latent_prefill_fits() { return kFits ? 1 : 0; }

// ``queries`` bfloat16 [tokens * heads, KEY_DIM]; ``pages`` [page][slot][KEY_DIM] with ``page_stride`` elements between pages; ``out``
// bfloat16 [tokens * heads, VALUE_DIM]; ``sinks`` 32-bit [heads] or null; ``longest``: the most rows any entry of the step has.
// ``splits`` > 1: that many CTAs share a row tile's keys and write ``partial`` (tokens * splits * (heads * VALUE_DIM + 2 * heads) floats)
// instead of ``out``; the caller merges the parts (and adds the sinks there).
TLIE_EXPORT int tlie_latent_prefill(const void* queries, const void* pages, long long page_stride, const int* seq_starts, const int* first_positions,
                                    const int* block_table, int table_stride, const float* sinks, void* out, int tokens, int entries, int longest, int heads,
                                    int page_size, float scale, int splits, float* partial, cudaStream_t stream) {
  if (tokens <= 0 || entries <= 0) return 0;
  if (!kFits || heads <= 0 || entries > 65535 || page_size <= 0 || splits < 1 || splits > 64 || (splits > 1 && partial == nullptr)) return (int)cudaErrorInvalidValue;
  constexpr size_t smem = smem_with(kStages);
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(latent_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const dim3 grid(((size_t)longest * heads + kRows - 1) / kRows, entries, splits);
  latent_prefill_kernel<<<grid, kThreads, smem, stream>>>((const __nv_bfloat16*)queries, (const __nv_bfloat16*)pages, page_stride, seq_starts, first_positions,
                                                          block_table, table_stride, sinks, (__nv_bfloat16*)out, heads, page_size, scale, splits > 1 ? partial : nullptr);
  return (int)cudaGetLastError();
}
