// Gated linear recurrences over the rows of a step, with the state every request carries between steps.
//
// minGRU (a gated recurrence whose gates read the current token only): for every channel c of a request,
//   z_t = sigmoid(a_t + bias_z),  u_t = x_t + bias_x,  cand_t = u_t >= 0 ? u_t + 1/2 : sigmoid(u_t)
//   S_t = (1 - z_t) S_{t-1} + z_t cand_t,             out_t = S_t * silu(g_t)
// where a, x and g are the three thirds of a row of one stacked product [T, 3 W] (bfloat16 or 32-bit) and S lives in 32-bit
// in the request's state slot [slots, W].  Everything after the product is 32-bit.
//
// The recurrence is linear in S, S_t = p_t S_{t-1} + r_t, so a run of rows composes to S_end = P S_in + R.  A prompt portion
// is cut into up to 64 runs per request: a thread per (run, channel) first finds its run's (P, R), one warp carries the state
// through the runs, and every thread walks its run again from the state it starts in, writing the outputs.  A single decoded
// token is one run: read the state, one update, write it back.  How a request's rows were cut into steps and runs changes a
// state only by rounding.
#include "common.cuh"

namespace tlie {

constexpr int kScanChannels = 32;   // channels per CTA at most: one warp's width, consecutive in memory (16 where that fills more SMs)
constexpr int kScanThreads = 1024;  // channels x runs of a CTA at most

struct GateStep {
  float keep, drive;   // S <- keep * S + drive
};

__device__ __forceinline__ float sigmoidf(float v) { return 1.0f / (1.0f + expf(-v)); }

constexpr int kScanBatch = 8;   // rows whose loads a thread has in flight together

// one token's update from its two pre-activations: z = sigmoid(a + bias_z), candidate from x + bias_x
__device__ __forceinline__ GateStep mingru_step(float a, float x, float bias_z, float bias_x) {
  const float z = sigmoidf(a + bias_z);
  const float u = x + bias_x;
  const float cand = u >= 0.0f ? u + 0.5f : sigmoidf(u);
  return {1.0f - z, z * cand};
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads) mingru_scan_kernel(const T* __restrict__ zxg, const float* __restrict__ bias_z,
                                                                                  const float* __restrict__ bias_x, float* __restrict__ state,
                                                                                  const int* __restrict__ seq_starts, const int* __restrict__ state_slots,
                                                                                  T* __restrict__ out, int width) {
  __shared__ float keep_of[kScanThreads], drive_of[kScanThreads], start_of[kScanThreads];   // [run][channel of the CTA]
  const int channels = blockDim.x;
  const int c = blockIdx.x * channels + threadIdx.x;
  const int entry = blockIdx.y;
  const int runs = blockDim.y, run = threadIdx.y;
  const int first = seq_starts[entry], rows = seq_starts[entry + 1] - first;
  const bool live = c < width;
  const int per_run = (rows + runs - 1) / runs;
  const int lo = min(rows, run * per_run), hi = min(rows, lo + per_run);
  const float bz = live ? bias_z[c] : 0.0f, bx = live ? bias_x[c] : 0.0f;
  float* slot = state + (size_t)state_slots[entry] * width;
  const size_t stride = (size_t)3 * width;

  if (runs > 1) {
    float keep = 1.0f, drive = 0.0f;
    if (live)
      for (int t0 = lo; t0 < hi; t0 += kScanBatch) {
        // a batch of rows' loads are issued together; the updates then run in order
        float a[kScanBatch], u[kScanBatch];
#pragma unroll
        for (int k = 0; k < kScanBatch; ++k) {
          const T* row = zxg + (size_t)(first + min(t0 + k, hi - 1)) * stride;
          a[k] = to_float(row[c]);
          u[k] = to_float(row[width + c]);
        }
#pragma unroll
        for (int k = 0; k < kScanBatch; ++k) {
          if (t0 + k >= hi) break;
          const GateStep g = mingru_step(a[k], u[k], bz, bx);
          keep *= g.keep;
          drive = g.keep * drive + g.drive;
        }
      }
    keep_of[run * channels + threadIdx.x] = keep;
    drive_of[run * channels + threadIdx.x] = drive;
    __syncthreads();
    if (run == 0 && live) {
      float s = slot[c];
      for (int r = 0; r < runs; ++r) {
        start_of[r * channels + threadIdx.x] = s;
        s = keep_of[r * channels + threadIdx.x] * s + drive_of[r * channels + threadIdx.x];
      }
      slot[c] = s;
    }
    __syncthreads();
  }
  if (!live) return;
  float s = runs > 1 ? start_of[run * channels + threadIdx.x] : slot[c];
  for (int t0 = lo; t0 < hi; t0 += kScanBatch) {
    float a[kScanBatch], u[kScanBatch], gate[kScanBatch];
#pragma unroll
    for (int k = 0; k < kScanBatch; ++k) {
      const T* row = zxg + (size_t)(first + min(t0 + k, hi - 1)) * stride;
      a[k] = to_float(row[c]);
      u[k] = to_float(row[width + c]);
      gate[k] = to_float(row[2 * width + c]);
    }
#pragma unroll
    for (int k = 0; k < kScanBatch; ++k) {
      if (t0 + k >= hi) break;
      const GateStep g = mingru_step(a[k], u[k], bz, bx);
      s = g.keep * s + g.drive;
      out[(size_t)(first + t0 + k) * width + c] = from_float<T>(s * (gate[k] * sigmoidf(gate[k])));
    }
  }
  if (runs == 1) slot[c] = s;
}

}  // namespace tlie

using namespace tlie;

// ``runs``: how many runs a request's rows are cut into (1 to 64); the host picks it from the longest entry of the step.  A CTA takes
// 32 channels, or 16 (and then up to 64 runs) where 32 would leave SMs without a CTA.
TLIE_EXPORT int tlie_mingru_scan(int dtype, const void* zxg, const float* bias_z, const float* bias_x, float* state, const int* seq_starts,
                                 const int* state_slots, void* out, int entries, int width, int runs, cudaStream_t stream) {
  if (entries <= 0 || width <= 0) return 0;
  if (runs < 1 || runs > 64) return (int)cudaErrorInvalidValue;
  int channels = kScanChannels;
  if (runs > 1 && (long long)((width + 31) / 32) * entries < device_sm_count()) channels = 16;
  if (runs * channels > kScanThreads) runs = kScanThreads / channels;
  const dim3 grid((width + channels - 1) / channels, entries), block(channels, runs);
  if (dtype == TLIE_F32)
    mingru_scan_kernel<float><<<grid, block, 0, stream>>>((const float*)zxg, bias_z, bias_x, state, seq_starts, state_slots, (float*)out, width);
  else
    mingru_scan_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((const __nv_bfloat16*)zxg, bias_z, bias_x, state, seq_starts, state_slots,
                                                                 (__nv_bfloat16*)out, width);
  return (int)cudaGetLastError();
}
