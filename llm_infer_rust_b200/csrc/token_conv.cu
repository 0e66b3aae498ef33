// A float32 residual stream with one-gain RMS norms, and short causal convolutions over time whose last
// inputs are per-request state.
//
//   residual_scale   x[t] += y[t] (optional, the sum in float), s[t] = gain / sqrt(mean(x[t]^2) + eps)
//   scaled_rows      out[r] = x[rows[r]] * s[rows[r]]                       (the norm itself, for chosen rows)
//   causal_taps      y[t][c] = (identity ? u[t][c] : 0) + sum_j w[c][j] * u[t - taps + 1 + j][c],
//                    u[t][c] = in[t][c] * (s ? s[t] : 1)
//   taps_state_update   the last taps - 1 inputs u of every row become the row's state
//   add_norm_taps_single   the first, the third and the fourth in one kernel, for steps whose rows have one token
//
// Inputs before a row's first token of this step come from the request's state slot,
// state[slot][taps - 1][C] in float32, oldest first; a row that starts at position 0 reads zeros, and positions
// before the sequence's start are stored as zeros, so the state of a sequence shorter than taps - 1 is right
// too.  The state of a row with several tokens in the step is read by causal_taps and written by taps_state_update,
// a kernel of its own behind it in the stream: in one kernel the block of a row's last token could overwrite what
// the block of its first token has yet to read.  A row of ONE token has one reader per channel, which writes the
// state itself.  Slot 0 belongs to padding rows and may hold anything.
//
// A row's result depends on its own tokens only; sums over a token's vector are taken in a fixed order.
#include "token_conv.cuh"

// ------------------------------------------------------------------ residual sum and the norm's scale
template <typename TY>
__global__ void __launch_bounds__(256)
residual_scale_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ gain, float eps,
                      float* __restrict__ scale, int width) {
  __shared__ float scratch[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = x[base + c];
    if (y != nullptr) {
      v += to_f32<TY>(y[base + c]);
      x[base + c] = v;
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0 && scale != nullptr) scale[blockIdx.x] = gain[0] / sqrtf(ss / static_cast<float>(width) + eps);
}

template <typename TO>
__global__ void __launch_bounds__(256)
scaled_rows_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ scale,
                   const int* __restrict__ rows, int width) {
  const int t = rows ? rows[blockIdx.x] : blockIdx.x;
  const float s = scale[t];
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[static_cast<size_t>(blockIdx.x) * width + c] = from_f32<TO>(x[static_cast<size_t>(t) * width + c] * s);
}

// ------------------------------------------------------------------ the convolution
// grid (tokens, channel tiles of 256)
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
causal_taps_kernel(TapsInput<TI> in, TO* __restrict__ out, int out_stride, int identity) {
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= in.channels) return;
  const TapsRow row = taps_row(in, t);
  const float y = taps_value(in, row, t, c, identity != 0);
  out[static_cast<size_t>(t) * out_stride + c] = from_f32<TO>(y);
}

// grid (tokens, tiles of 128 x 8 channels): the same, eight channels a thread; a token that is alone in its row
// also brings the row's state up to date (see taps_value8)
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
causal_taps_vec_kernel(TapsInput<TI> in, TO* __restrict__ out, int out_stride, int identity) {
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= in.channels) return;
  const TapsRow row = taps_row(in, t);
  float y[8];
  taps_value8(in, row, t, c, identity != 0, taps_single(in, t), y);
  store8<TO>(out + static_cast<size_t>(t) * out_stride + c, y);
}

// ------------------------------------------------------------------ a step whose rows all have one token
// x[t] += y[t], the norm's scale, the convolution and the row's new state in one kernel, a block a token: no token
// of the step is another token's past, so nothing that one block writes is read by another.
template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
add_norm_taps_single_kernel(float* x /* also read through `in` */, const TY* __restrict__ y, const float* __restrict__ gain, float eps,
                            float* __restrict__ scale, TapsInput<float> in, TO* __restrict__ out, int out_stride,
                            int identity) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int width = in.channels;
  const size_t base = static_cast<size_t>(t) * width;
  float ss = 0.0f;
  for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
    float v[8];
    load_floats<float, 8>(x + base + c, v);
    if (y != nullptr) {
      float a[8];
      load_floats<TY, 8>(y + base + c, a);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += a[i];
      store8<float>(x + base + c, v);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale[t] = gain[0] / sqrtf(ss / static_cast<float>(width) + eps);
  __syncthreads();                                   // the scale, and every thread's own x, are read back below
  const TapsRow row = taps_row(in, t);
  for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
    float r[8];
    taps_value8(in, row, t, c, identity != 0, true, r);
    store8<TO>(out + static_cast<size_t>(t) * out_stride + c, r);
  }
}

// ------------------------------------------------------------------ C interface
B200_EXPORT int b200_residual_scale(float* x, const void* y, int y_dtype, const float* gain, float eps, float* scale,
                                    int tokens, int width, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0) return B200_BAD_SIZE;
  if (y == nullptr || y_dtype == B200_F32)
    residual_scale_kernel<float><<<tokens, 256, 0, stream>>>(x, static_cast<const float*>(y), gain, eps, scale, width);
  else if (y_dtype == B200_BF16)
    residual_scale_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(x, static_cast<const __nv_bfloat16*>(y), gain,
                                                                      eps, scale, width);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}

B200_EXPORT int b200_scaled_rows(void* out, int out_dtype, const float* x, const float* scale, const int* rows,
                                 int n, int width, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0) return B200_BAD_SIZE;
  if (out_dtype == B200_F32)
    scaled_rows_kernel<float><<<n, 256, 0, stream>>>(static_cast<float*>(out), x, scale, rows, width);
  else if (out_dtype == B200_BF16)
    scaled_rows_kernel<__nv_bfloat16><<<n, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(out), x, scale, rows, width);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}

template <typename TI>
static int launch_taps(const TapsInput<TI>& in, void* out, int out_dtype, int out_stride, int identity, int tokens,
                       int num_rows, int update_state, int all_single, cudaStream_t stream) {
  const dim3 grid(tokens, (in.channels + 255) / 256);
  const bool vec = update_state && in.channels % 8 == 0 && in.in_stride % 8 == 0 && out_stride % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(in.x) | reinterpret_cast<uintptr_t>(out) |
                    reinterpret_cast<uintptr_t>(in.state)) % 16 == 0;
  if (vec) {
    const dim3 vgrid(tokens, (in.channels / 8 + 127) / 128);
    if (out_dtype == B200_F32)
      causal_taps_vec_kernel<TI, float><<<vgrid, 128, 0, stream>>>(in, static_cast<float*>(out), out_stride, identity);
    else if (out_dtype == B200_BF16)
      causal_taps_vec_kernel<TI, __nv_bfloat16><<<vgrid, 128, 0, stream>>>(in, static_cast<__nv_bfloat16*>(out),
                                                                          out_stride, identity);
    else
      return B200_BAD_DTYPE;
    int rc = b200_check_launch();
    if (rc != 0 || in.taps <= 1 || all_single) return rc;
    const dim3 sgrid(num_rows, (in.channels + 255) / 256);
    taps_state_update_kernel<TI><<<sgrid, 256, 0, stream>>>(in, num_rows, 1);
    return b200_check_launch();
  }
  if (out_dtype == B200_F32)
    causal_taps_kernel<TI, float><<<grid, 256, 0, stream>>>(in, static_cast<float*>(out), out_stride, identity);
  else if (out_dtype == B200_BF16)
    causal_taps_kernel<TI, __nv_bfloat16><<<grid, 256, 0, stream>>>(in, static_cast<__nv_bfloat16*>(out), out_stride,
                                                                    identity);
  else
    return B200_BAD_DTYPE;
  int rc = b200_check_launch();
  if (rc != 0 || !update_state || in.taps <= 1) return rc;
  const dim3 sgrid(num_rows, (in.channels + 255) / 256);
  taps_state_update_kernel<TI><<<sgrid, 256, 0, stream>>>(in, num_rows, 0);
  return b200_check_launch();
}

template <typename TI>
static TapsInput<TI> taps_input(const void* x, int in_stride, const float* scale, const float* w, int taps,
                                int channels, float* state, const int* row_of_token, const int* cu_q,
                                const int* prefix_len, const int* state_slots) {
  TapsInput<TI> in;
  in.x = static_cast<const TI*>(x); in.in_stride = in_stride; in.scale = scale; in.w = w; in.taps = taps;
  in.channels = channels; in.state = state; in.row_of_token = row_of_token; in.cu_q = cu_q;
  in.prefix_len = prefix_len; in.state_slots = state_slots;
  return in;
}

// out[t][c] for c < channels; `x` rows are in_stride wide, `out` rows out_stride.  With update_state the rows'
// states are brought up to date: rows of one token by the convolution kernel itself where it takes eight channels
// a thread, the others by a second kernel behind it (left out when the caller says that all rows have one token).
B200_EXPORT int b200_causal_taps(const void* x, int in_dtype, int in_stride, const float* scale, const float* w,
                                 int taps, int channels, float* state, const int* row_of_token, const int* cu_q,
                                 const int* prefix_len, const int* state_slots, void* out, int out_dtype,
                                 int out_stride, int identity, int tokens, int num_rows, int update_state,
                                 int all_single, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (channels <= 0 || taps < 1 || taps > TAPS_MAX || num_rows <= 0) return B200_BAD_SIZE;
  if ((channels + 255) / 256 > 65535) return B200_BAD_SIZE;
  if (in_dtype == B200_F32)
    return launch_taps<float>(taps_input<float>(x, in_stride, scale, w, taps, channels, state, row_of_token, cu_q,
                                                prefix_len, state_slots),
                              out, out_dtype, out_stride, identity, tokens, num_rows, update_state, all_single, stream);
  if (in_dtype == B200_BF16)
    return launch_taps<__nv_bfloat16>(taps_input<__nv_bfloat16>(x, in_stride, scale, w, taps, channels, state,
                                                                row_of_token, cu_q, prefix_len, state_slots),
                                      out, out_dtype, out_stride, identity, tokens, num_rows, update_state, all_single, stream);
  return B200_BAD_DTYPE;
}

// Only the state update (for a caller whose own kernel did the convolution).
B200_EXPORT int b200_taps_state_update(const void* x, int in_dtype, int in_stride, const float* scale, int taps,
                                       int channels, float* state, const int* cu_q, const int* prefix_len,
                                       const int* state_slots, int num_rows, int skip_single, cudaStream_t stream) {
  if (num_rows <= 0 || taps <= 1) return 0;
  if (channels <= 0 || taps > TAPS_MAX || (channels + 255) / 256 > 65535) return B200_BAD_SIZE;
  const dim3 sgrid(num_rows, (channels + 255) / 256);
  if (in_dtype == B200_F32)
    taps_state_update_kernel<float><<<sgrid, 256, 0, stream>>>(
        taps_input<float>(x, in_stride, scale, nullptr, taps, channels, state, nullptr, cu_q, prefix_len, state_slots),
        num_rows, skip_single);
  else if (in_dtype == B200_BF16)
    taps_state_update_kernel<__nv_bfloat16><<<sgrid, 256, 0, stream>>>(
        taps_input<__nv_bfloat16>(x, in_stride, scale, nullptr, taps, channels, state, nullptr, cu_q, prefix_len,
                                  state_slots),
        num_rows, skip_single);
  else
    return B200_BAD_DTYPE;
  return b200_check_launch();
}

// The fused form for a step whose rows ALL bring one token (the caller vouches for it): x += y (y may be null), scale
// [tokens] and out [tokens, channels] as b200_residual_scale and b200_causal_taps (with update_state) leave them.
// Refuses (B200_BAD_SIZE / B200_BAD_ALIGN) rows that are no whole 16-byte pieces; the caller then runs the two.
B200_EXPORT int b200_add_norm_taps_single(float* x, const void* y, int y_dtype, const float* gain, float eps,
                                          float* scale, const float* w, int taps, int channels, float* state,
                                          const int* row_of_token, const int* cu_q, const int* prefix_len,
                                          const int* state_slots, void* out, int out_dtype, int identity, int tokens,
                                          cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (channels <= 0 || channels % 8 != 0 || taps < 1 || taps > TAPS_MAX) return B200_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(w)) % 16 != 0)
    return B200_BAD_ALIGN;
  const TapsInput<float> in = taps_input<float>(x, channels, scale, w, taps, channels, state, row_of_token, cu_q,
                                                prefix_len, state_slots);
#define B200_FUSED(TY, TO)                                                                                          \
  add_norm_taps_single_kernel<TY, TO><<<tokens, 256, 0, stream>>>(x, static_cast<const TY*>(y), gain, eps, scale, in, \
                                                                   static_cast<TO*>(out), channels, identity)
  const bool y32 = y == nullptr || y_dtype == B200_F32;
  if (!y32 && y_dtype != B200_BF16) return B200_BAD_DTYPE;
  if (out_dtype == B200_F32) {
    if (y32) B200_FUSED(float, float); else B200_FUSED(__nv_bfloat16, float);
  } else if (out_dtype == B200_BF16) {
    if (y32) B200_FUSED(float, __nv_bfloat16); else B200_FUSED(__nv_bfloat16, __nv_bfloat16);
  } else {
    return B200_BAD_DTYPE;
  }
#undef B200_FUSED
  return b200_check_launch();
}
