// Retention: linear attention with a fixed decay per head, no softmax and no denominator, with the state of every
// request kept in float32.
//
//   S_t = decay_h S_(t-1) + k_t v_t^T        (S: [d, dv] per head)        o_t = S_t^T q_t
//
// q and k are first rotated (half-split pairs (i, i + rot_dim/2) of the first rot_dim coordinates, angle =
// position * inv_freq[i], in float) and k is then multiplied by k_scale.  Everything after the projection is float:
// the rotation, the products, the state and the output o [tokens, heads * dv].
//
// `x` [tokens, in_stride] holds q (heads * d), k (heads * d), v (heads * dv) side by side from column 0.
// state [slots + 1, heads, d, dv]; a row whose prefix_len is 0 starts from zeros; slot 0 takes padding rows.
//
// retention_scan_kernel: grid (rows, heads, column tiles of 32).  A block owns 32 columns of one head's state:
// lane = column, each of the 8 warps keeps ceil(d / 8) rows of those columns in registers.  Tokens are taken eight
// at a time: the block stages their rotated q and k and their v in shared memory, every thread runs the
// recurrence over the eight tokens for its rows and leaves a partial o per token, and the eight warps' partials
// are added in a fixed order.  The recurrence runs token by token in the sequence's order whatever the step's
// cut, so a position's result has the same bits however the prompt was cut.
#include "common.cuh"

constexpr int RT_WARPS = 8;
constexpr int RT_COLS = 32;
constexpr int RT_TOKENS = 8;

template <typename T>
__device__ __forceinline__ float rotated(const T* __restrict__ src, int e, int rot_dim, float pos,
                                         const float* __restrict__ inv_freq) {
  const float y = to_f32<T>(src[e]);
  if (e >= rot_dim) return y;
  const int half = rot_dim >> 1;
  const bool low = e < half;
  const float other = to_f32<T>(src[low ? e + half : e - half]);
  float sn, cs;
  sincosf(pos * inv_freq[low ? e : e - half], &sn, &cs);
  return low ? y * cs - other * sn : y * cs + other * sn;
}

template <typename T, int DI>
__global__ void __launch_bounds__(RT_WARPS * 32)
retention_scan_kernel(const T* __restrict__ x, int in_stride, float* __restrict__ o, float* __restrict__ state,
                      const float* __restrict__ decay, const float* __restrict__ inv_freq, int rot_dim, float k_scale,
                      const int* __restrict__ positions, const int* __restrict__ cu_q,
                      const int* __restrict__ prefix_len, const int* __restrict__ state_slots, int heads, int d, int dv) {
  extern __shared__ float smem[];
  float* qs = smem;                                   // [RT_TOKENS][d]
  float* ks = qs + RT_TOKENS * d;                     // [RT_TOKENS][d]
  float* vs = ks + RT_TOKENS * d;                     // [RT_TOKENS][RT_COLS]
  float* part = vs + RT_TOKENS * RT_COLS;             // [RT_TOKENS][RT_WARPS][RT_COLS]

  const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * RT_COLS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = col0 + lane;
  const bool col_ok = col < dv;
  const int rows_per_warp = (d + RT_WARPS - 1) / RT_WARPS;
  const int i0 = warp * rows_per_warp;
  const int first = cu_q[r], n = cu_q[r + 1] - first;
  const float g = decay[h];
  float* st = state + (static_cast<size_t>(state_slots[r]) * heads + h) * d * dv;
  const bool has_past = prefix_len[r] > 0;

  float S[DI];
#pragma unroll
  for (int ii = 0; ii < DI; ++ii) {
    const int i = i0 + ii;
    S[ii] = (has_past && col_ok && ii < rows_per_warp && i < d) ? st[static_cast<size_t>(i) * dv + col] : 0.0f;
  }
  const int qoff = h * d, koff = heads * d + h * d, voff = 2 * heads * d + h * dv;
  for (int base = 0; base < n; base += RT_TOKENS) {
    const int nt = min(RT_TOKENS, n - base);
    for (int idx = threadIdx.x; idx < nt * d; idx += blockDim.x) {
      const int tb = idx / d, e = idx - tb * d;
      const int t = first + base + tb;
      const T* row = x + static_cast<size_t>(t) * in_stride;
      const float pos = static_cast<float>(positions[t]);
      qs[tb * d + e] = rotated<T>(row + qoff, e, rot_dim, pos, inv_freq);
      ks[tb * d + e] = rotated<T>(row + koff, e, rot_dim, pos, inv_freq) * k_scale;
    }
    for (int idx = threadIdx.x; idx < nt * RT_COLS; idx += blockDim.x) {
      const int tb = idx / RT_COLS, j = idx - tb * RT_COLS;
      vs[idx] = col0 + j < dv ? to_f32<T>(x[static_cast<size_t>(first + base + tb) * in_stride + voff + col0 + j]) : 0.0f;
    }
    __syncthreads();
    for (int tb = 0; tb < nt; ++tb) {
      const float v = vs[tb * RT_COLS + lane];
      const float* kt = ks + tb * d + i0;
      const float* qt = qs + tb * d + i0;
      float acc = 0.0f;
#pragma unroll
      for (int ii = 0; ii < DI; ++ii) {
        if (ii < rows_per_warp && i0 + ii < d) {
          S[ii] = fmaf(g, S[ii], kt[ii] * v);
          acc = fmaf(S[ii], qt[ii], acc);
        }
      }
      part[(tb * RT_WARPS + warp) * RT_COLS + lane] = acc;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * RT_COLS; idx += blockDim.x) {
      const int tb = idx / RT_COLS, j = idx - tb * RT_COLS;
      if (col0 + j < dv) {
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < RT_WARPS; ++w) sum += part[(tb * RT_WARPS + w) * RT_COLS + j];
        o[(static_cast<size_t>(first + base + tb) * heads + h) * dv + col0 + j] = sum;
      }
    }
    __syncthreads();
  }
  if (col_ok) {
#pragma unroll
    for (int ii = 0; ii < DI; ++ii) {
      const int i = i0 + ii;
      if (ii < rows_per_warp && i < d) st[static_cast<size_t>(i) * dv + col] = S[ii];
    }
  }
}

template <typename T, int DI>
static int launch_scan(const void* x, int in_stride, float* o, float* state, const float* decay, const float* inv_freq,
                       int rot_dim, float k_scale, const int* positions, const int* cu_q, const int* prefix_len,
                       const int* state_slots, int num_rows, int heads, int d, int dv, cudaStream_t stream) {
  const size_t smem = (2 * RT_TOKENS * d + RT_TOKENS * RT_COLS + RT_TOKENS * RT_WARPS * RT_COLS) * sizeof(float);
  const dim3 grid(num_rows, heads, (dv + RT_COLS - 1) / RT_COLS);
  retention_scan_kernel<T, DI><<<grid, RT_WARPS * 32, smem, stream>>>(
      static_cast<const T*>(x), in_stride, o, state, decay, inv_freq, rot_dim, k_scale, positions, cu_q, prefix_len,
      state_slots, heads, d, dv);
  return b200_check_launch();
}

template <typename T>
static int dispatch_scan(const void* x, int in_stride, float* o, float* state, const float* decay,
                         const float* inv_freq, int rot_dim, float k_scale, const int* positions, const int* cu_q,
                         const int* prefix_len, const int* state_slots, int num_rows, int heads, int d, int dv,
                         cudaStream_t stream) {
  const int di = (d + RT_WARPS - 1) / RT_WARPS;
#define RT_CASE(N)                                                                                                   \
  if (di <= N)                                                                                                       \
    return launch_scan<T, N>(x, in_stride, o, state, decay, inv_freq, rot_dim, k_scale, positions, cu_q, prefix_len, \
                             state_slots, num_rows, heads, d, dv, stream)
  RT_CASE(4);
  RT_CASE(8);
  RT_CASE(16);
  RT_CASE(32);
  RT_CASE(64);
#undef RT_CASE
  return B200_BAD_SIZE;
}

B200_EXPORT int b200_retention(const void* x, int dtype, int in_stride, float* o, float* state, const float* decay,
                               const float* inv_freq, int rot_dim, float k_scale, const int* positions,
                               const int* cu_q, const int* prefix_len, const int* state_slots, int num_rows, int heads,
                               int d, int dv, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (heads <= 0 || heads > 65535 || d <= 0 || d > 512 || dv <= 0 || rot_dim < 0 || rot_dim > d || (rot_dim & 1))
    return B200_BAD_SIZE;
  if ((dv + RT_COLS - 1) / RT_COLS > 65535) return B200_BAD_SIZE;
  if (dtype == B200_F32)
    return dispatch_scan<float>(x, in_stride, o, state, decay, inv_freq, rot_dim, k_scale, positions, cu_q, prefix_len,
                                state_slots, num_rows, heads, d, dv, stream);
  if (dtype == B200_BF16)
    return dispatch_scan<__nv_bfloat16>(x, in_stride, o, state, decay, inv_freq, rot_dim, k_scale, positions, cu_q,
                                        prefix_len, state_slots, num_rows, heads, d, dv, stream);
  return B200_BAD_DTYPE;
}
