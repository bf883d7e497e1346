// Small row-wise kernels around the residual stream and the feed-forward, and a product per head.
//
//   add_row_vector      residual[t] += delta[t] (optional) + vector                    a learned vector added to every row
//   complete_and_round  residual[t] += delta[t] (optional); out[t] = T(residual[t])    the finished stream as a product's operand
//   clamped_gate_mul    g = min(gate, limit), u = clamp(up, -limit, limit); out = g * sigmoid(alpha g) * (u + shift)
//   scale_rows          x *= factor (32-bit, in place)
//   gather_gated        out[t, d] = act(z[t, d]) * table[ids[t], offset + d]           a slice of a second token table, gated
//   unit_norm_add       residual[t] += y[t] / sqrt(mean(y[t]^2) + eps) * weight        a normalised branch joins the stream
//   head_linear         out[t, h, :] = W[h] . x[t, h, :]  per head, operands with strides of their own, 32-bit sums in a fixed order
// Storage float or bfloat16, arithmetic 32-bit.
#include "common.cuh"

namespace tlie {

template <typename T>
__global__ void add_row_vector_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ vector, int hidden, size_t total) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float v = residual[i];
    if (delta) v += to_float(delta[i]);
    residual[i] = v + vector[i % hidden];
  }
}

template <typename T>
__global__ void complete_and_round_kernel(float* __restrict__ residual, const T* __restrict__ delta, T* __restrict__ out, size_t total) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float v = residual[i];
    if (delta) {
      v += to_float(delta[i]);
      residual[i] = v;
    }
    out[i] = from_float<T>(v);
  }
}

template <typename T>
__global__ void clamped_gate_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total, float limit, float alpha, float shift) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / inter, col = i - row * inter;
    const float g = fminf(to_float(gate_up[row * 2 * inter + col]), limit);
    const float u = fminf(fmaxf(to_float(gate_up[row * 2 * inter + inter + col]), -limit), limit);
    out[i] = from_float<T>(g * (1.0f / (1.0f + expf(-alpha * g))) * (u + shift));
  }
}

// the same, eight bfloat16 elements per thread (inter a multiple of 8): 16-byte loads and stores
__global__ void clamped_gate_mul_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter, size_t total8, float limit, float alpha,
                                            float shift) {
  const int per_row = inter / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / per_row, col = (i - row * per_row) * 8;
    const uint4 graw = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + col);
    const uint4 uraw = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + inter + col);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 result;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const float2 g2 = __bfloat1622float2(gp[n]), u2 = __bfloat1622float2(up[n]);
      const float g0 = fminf(g2.x, limit), g1 = fminf(g2.y, limit);
      const float u0 = fminf(fmaxf(u2.x, -limit), limit), u1 = fminf(fmaxf(u2.y, -limit), limit);
      rp[n] = __floats2bfloat162_rn(g0 * (1.0f / (1.0f + expf(-alpha * g0))) * (u0 + shift), g1 * (1.0f / (1.0f + expf(-alpha * g1))) * (u1 + shift));
    }
    *reinterpret_cast<uint4*>(out + row * inter + col) = result;
  }
}

__global__ void scale_rows_kernel(float* __restrict__ x, float factor, size_t total) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] *= factor;
}

__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

template <typename T>
__global__ void gather_gated_kernel(const T* __restrict__ z, const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out, int dim,
                                    int table_width, int offset, int table_rows, size_t total) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / dim;
    const int d = (int)(i - row * dim);
    int id = ids[row];
    if (id < 0 || id >= table_rows) id = 0;   // the embedding kernel has already reported it
    out[i] = from_float<T>(gelu_tanh_f(to_float(z[i])) * to_float(table[(size_t)id * table_width + offset + d]));
  }
}

// one CTA per row; a thread keeps its (up to 16) elements of y in registers between the sum of squares and the add
template <typename T>
__global__ void unit_norm_add_kernel(float* __restrict__ residual, const T* __restrict__ y, const float* __restrict__ weight, float eps, int hidden) {
  __shared__ float scratch[32];
  constexpr int kKept = 16;
  const size_t row = blockIdx.x;
  float kept[kKept];
  float squares = 0.0f;
#pragma unroll
  for (int n = 0; n < kKept; ++n) {
    const int i = threadIdx.x + n * blockDim.x;
    kept[n] = i < hidden ? to_float(y[row * hidden + i]) : 0.0f;
    squares += kept[n] * kept[n];
  }
  for (int i = threadIdx.x + kKept * blockDim.x; i < hidden; i += blockDim.x) {
    const float v = to_float(y[row * hidden + i]);
    squares += v * v;
  }
  const float inv = rsqrtf(block_sum(squares, scratch) / (float)hidden + eps);
#pragma unroll
  for (int n = 0; n < kKept; ++n) {
    const int i = threadIdx.x + n * blockDim.x;
    if (i < hidden) residual[row * hidden + i] += kept[n] * inv * weight[i];
  }
  for (int i = threadIdx.x + kKept * blockDim.x; i < hidden; i += blockDim.x) residual[row * hidden + i] += to_float(y[row * hidden + i]) * inv * weight[i];
}

// out[t, h, n] = sum_k x[t, h, k] * w[h, n, k]: a warp per output, the lanes taking k in turns (neighbouring lanes read neighbouring
// elements) and adding up in a fixed order, so a row's bits depend on the row alone.
template <typename T>
__global__ void head_linear_kernel(const T* __restrict__ x, long long x_row, long long x_head, const T* __restrict__ w, T* __restrict__ out, long long out_row,
                                   long long out_head, int heads, int n_out, int k_in, size_t total) {
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < total; i += warps) {
    const int n = (int)(i % n_out);
    const int h = (int)((i / n_out) % heads);
    const size_t t = i / ((size_t)n_out * heads);
    const T* xr = x + t * x_row + h * x_head;
    const T* wr = w + ((size_t)h * n_out + n) * k_in;
    float sum = 0.0f;
    for (int k = lane; k < k_in; k += 32) sum += to_float(xr[k]) * to_float(wr[k]);
    sum = warp_sum(sum);
    if (lane == 0) out[t * out_row + h * out_head + n] = from_float<T>(sum);
  }
}

static inline int blocks_for(size_t total, int threads) {
  const size_t wanted = (total + threads - 1) / threads;
  const size_t most = (size_t)device_sm_count() * 16;
  return (int)(wanted < most ? (wanted ? wanted : 1) : most);
}

}  // namespace tlie

using namespace tlie;

#define TLIE_BY_TYPE(dtype, CALL)        \
  if (dtype == TLIE_F32) {               \
    using T = float;                     \
    CALL;                                \
  } else {                               \
    using T = __nv_bfloat16;             \
    CALL;                                \
  }

TLIE_EXPORT int tlie_add_row_vector(int dtype, float* residual, const void* delta, const float* vector, int rows, int hidden, cudaStream_t stream) {
  const size_t total = (size_t)rows * hidden;
  if (total == 0) return 0;
  TLIE_BY_TYPE(dtype, (add_row_vector_kernel<T><<<blocks_for(total, 256), 256, 0, stream>>>(residual, (const T*)delta, vector, hidden, total)));
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_complete_and_round(int dtype, float* residual, const void* delta, void* out, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  TLIE_BY_TYPE(dtype, (complete_and_round_kernel<T><<<blocks_for((size_t)count, 256), 256, 0, stream>>>(residual, (const T*)delta, (T*)out, (size_t)count)));
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_clamped_gate_mul(int dtype, const void* gate_up, void* out, int rows, int inter, float limit, float alpha, float shift, cudaStream_t stream) {
  const size_t total = (size_t)rows * inter;
  if (total == 0) return 0;
  if (dtype == TLIE_BF16 && inter % 8 == 0) {
    clamped_gate_mul_vec_kernel<<<blocks_for(total / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total / 8, limit, alpha, shift);
    return (int)cudaGetLastError();
  }
  TLIE_BY_TYPE(dtype, (clamped_gate_mul_kernel<T><<<blocks_for(total, 256), 256, 0, stream>>>((const T*)gate_up, (T*)out, inter, total, limit, alpha, shift)));
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_scale_rows(float* x, float factor, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  scale_rows_kernel<<<blocks_for((size_t)count, 256), 256, 0, stream>>>(x, factor, (size_t)count);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_gather_gated(int dtype, const void* z, const void* table, const int* ids, void* out, int rows, int dim, int table_width, int offset,
                                  int table_rows, cudaStream_t stream) {
  const size_t total = (size_t)rows * dim;
  if (total == 0) return 0;
  if (offset < 0 || offset + dim > table_width || table_rows <= 0) return (int)cudaErrorInvalidValue;
  TLIE_BY_TYPE(dtype, (gather_gated_kernel<T><<<blocks_for(total, 256), 256, 0, stream>>>((const T*)z, (const T*)table, ids, (T*)out, dim, table_width, offset,
                                                                                        table_rows, total)));
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_unit_norm_add(int dtype, float* residual, const void* y, const float* weight, float eps, int rows, int hidden, cudaStream_t stream) {
  if (rows <= 0 || hidden <= 0) return 0;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 1024 ? 256 : 128);
  TLIE_BY_TYPE(dtype, (unit_norm_add_kernel<T><<<rows, threads, 0, stream>>>(residual, (const T*)y, weight, eps, hidden)));
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_head_linear(int dtype, const void* x, long long x_row, long long x_head, const void* w, void* out, long long out_row, long long out_head,
                                 int rows, int heads, int n_out, int k_in, cudaStream_t stream) {
  const size_t total = (size_t)rows * heads * n_out;
  if (total == 0) return 0;
  TLIE_BY_TYPE(dtype, (head_linear_kernel<T><<<blocks_for(total * 32, 256), 256, 0, stream>>>((const T*)x, x_row, x_head, (const T*)w, (T*)out, out_row, out_head, heads,
                                                                                       n_out, k_in, total)));
  return (int)cudaGetLastError();
}
