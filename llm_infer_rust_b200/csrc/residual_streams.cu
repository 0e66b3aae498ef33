// A residual that is S parallel float32 streams ("hyper-connections"), read through an RMS norm.
//
// A sublayer q reads u = sum_s in_q[s] X_s, and its output y is written back to all streams at once from the old
// ones:  X_t <- sum_s mix_q[s][t] X_s + out_q[t] y   (mix is indexed [from][to]).  One kernel does the write-back of
// the sublayer BEFORE (whose y arrives now) and the read of the sublayer AFTER, a block a token:
//
//     X' = mix^T X + out y        (skipped when there is nothing to write back; or X' = (e, ..., e) at the start)
//     u  = sum_t in[t] X'_t
//     out = u / sqrt(mean(u^2) + eps) * (w + offset)         (offset 1: a weight stored around zero)
//
// S = 1 with mix = out = in = 1 is the ordinary pre-norm residual sum.  Everything is float; only `out` is rounded
// (once) to the consumer's dtype.  `rows` picks tokens (the rows whose logits are wanted) and `store` 0 leaves the
// streams as they are: the model's last norm reads the sum of the streams (in = 1) that way.
// streams: [tokens, S, width] float32.  coefficients of a sublayer: in[S], out[S], mix[S][S], packed in that order.
// Sums over s run in index order and the sum of squares in a fixed order, so a token's result does not depend on
// the batch around it.
#include "common.cuh"

template <int S, typename TY, typename TO>
__global__ void __launch_bounds__(256)
stream_step_kernel(float* __restrict__ streams, const float* __restrict__ start, const TY* __restrict__ y,
                   const float* __restrict__ before, const float* __restrict__ read_in,
                   const float* __restrict__ norm_w, float offset, float eps, const int* __restrict__ rows,
                   TO* __restrict__ out, int width, int store) {
  extern __shared__ float u_row[];                    // [width]
  __shared__ float scratch[33];
  __shared__ float c_mix[S * S], c_out[S], c_in[S];
  const int t = rows ? rows[blockIdx.x] : blockIdx.x;
  if (threadIdx.x < S) {
    c_in[threadIdx.x] = read_in ? read_in[threadIdx.x] : 1.0f;
    c_out[threadIdx.x] = before ? before[S + threadIdx.x] : 0.0f;
  }
  if (threadIdx.x < S * S) c_mix[threadIdx.x] = before ? before[2 * S + threadIdx.x] : 0.0f;
  __syncthreads();
  float* X = streams + static_cast<size_t>(t) * S * width;
  const size_t row = static_cast<size_t>(t) * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float nx[S];
    if (start != nullptr) {
      const float e = start[row + c];
#pragma unroll
      for (int s = 0; s < S; ++s) nx[s] = e;
    } else {
      float x[S];
#pragma unroll
      for (int s = 0; s < S; ++s) x[s] = X[static_cast<size_t>(s) * width + c];
      if (before != nullptr) {
        const float yv = to_f32<TY>(y[row + c]);
#pragma unroll
        for (int to = 0; to < S; ++to) {
          float a = 0.0f;
#pragma unroll
          for (int s = 0; s < S; ++s) a = fmaf(c_mix[s * S + to], x[s], a);
          nx[to] = fmaf(c_out[to], yv, a);
        }
      } else {
#pragma unroll
        for (int s = 0; s < S; ++s) nx[s] = x[s];
      }
    }
    if (store && (start != nullptr || before != nullptr)) {
#pragma unroll
      for (int s = 0; s < S; ++s) X[static_cast<size_t>(s) * width + c] = nx[s];
    }
    float u = 0.0f;
#pragma unroll
    for (int s = 0; s < S; ++s) u = fmaf(c_in[s], nx[s], u);
    u_row[c] = u;
    ss = fmaf(u, u, ss);
  }
  ss = block_sum(ss, scratch);
  if (out == nullptr) return;
  const float r = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  TO* dst = out + static_cast<size_t>(blockIdx.x) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = from_f32<TO>(u_row[c] * r * (norm_w[c] + offset));
}

template <int S, typename TY, typename TO>
static int launch_step(float* streams, const float* start, const void* y, const float* before, const float* read_in,
                       const float* norm_w, float offset, float eps, const int* rows, void* out, int n, int width,
                       int store, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
  if (smem > 200 * 1024) return B200_BAD_SIZE;
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(stream_step_kernel<S, TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = smem;
  }
  stream_step_kernel<S, TY, TO><<<n, 256, smem, stream>>>(streams, start, static_cast<const TY*>(y), before, read_in,
                                                          norm_w, offset, eps, rows, static_cast<TO*>(out), width,
                                                          store);
  return b200_check_launch();
}

template <int S>
static int dispatch_types(float* streams, const float* start, const void* y, int y_dtype, const float* before,
                          const float* read_in, const float* norm_w, float offset, float eps, const int* rows,
                          void* out, int out_dtype, int n, int width, int store, cudaStream_t stream) {
#define STEP(TY, TO) launch_step<S, TY, TO>(streams, start, y, before, read_in, norm_w, offset, eps, rows, out, n, \
                                             width, store, stream)
  const bool y32 = y == nullptr || y_dtype == B200_F32;
  if (!y32 && y_dtype != B200_BF16) return B200_BAD_DTYPE;
  if (out_dtype == B200_F32) return y32 ? STEP(float, float) : STEP(__nv_bfloat16, float);
  if (out_dtype == B200_BF16) return y32 ? STEP(float, __nv_bfloat16) : STEP(__nv_bfloat16, __nv_bfloat16);
#undef STEP
  return B200_BAD_DTYPE;
}

constexpr int MAX_STREAMS = 8;

// One write-back and read.  `start` (float32 [tokens, width]): the streams begin as copies of it; else, with
// `before` (the coefficients of the sublayer whose output `y` is), the streams are updated; with neither they
// are read as they are.  `read_in`: in[S] of the reading sublayer (null: ones).  `rows` null: every token.
B200_EXPORT int b200_stream_step(float* streams, int num_streams, const float* start, const void* y, int y_dtype,
                                 const float* before, const float* read_in, const float* norm_w, float offset,
                                 float eps, const int* rows, void* out, int out_dtype, int n, int width, int store,
                                 cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0 || num_streams < 1 || num_streams > MAX_STREAMS) return B200_BAD_SIZE;
  if (before != nullptr && y == nullptr) return B200_BAD_SIZE;
  switch (num_streams) {
#define CASE(S)                                                                                                       \
  case S:                                                                                                             \
    return dispatch_types<S>(streams, start, y, y_dtype, before, read_in, norm_w, offset, eps, rows, out, out_dtype, \
                             n, width, store, stream)
    CASE(1); CASE(2); CASE(3); CASE(4); CASE(5); CASE(6); CASE(7); CASE(8);
#undef CASE
  }
  return B200_BAD_SIZE;
}
