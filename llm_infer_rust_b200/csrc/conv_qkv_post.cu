// Between the packed q/k/v projection and attention, for a mixer whose q, k and v pass through a short causal
// convolution over time: the convolution (inputs before the step come from the request's state, token_conv.cuh),
// the half-split rotation of q and k by angles computed from the position, an optional mix of v with the v of an
// earlier layer, and the stores: q to its buffer, k and v (as they will be attended) into the paged cache.
//
//   u = conv(projection)                                     (no convolution: u = projection)
//   rotation of the first rot_dim coordinates of a head:  (a, b) = (u[i], u[i + rot_dim/2]),
//        angle = position * inv_freq[i]  in float,   a' = a cos - b sin,   b' = b cos + a sin
//   v <- (1 - lambda) v + lambda v_first          (mode 2; mode 1 writes v as v_first, mode 0 does neither)
//
// The cache is [pages + 1, kv_heads, page_size, width] with widths d for keys and dv for values; slot =
// page * page_size + offset.  A slot outside the pool sets an error bit and is skipped.
#include "token_conv.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
conv_qkv_post_kernel(TapsInput<T> in, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                     const float* __restrict__ inv_freq, int rot_dim, const int* __restrict__ positions,
                     const int* __restrict__ slots, int nh, int nkv, int d, int dv, int page_size,
                     long long cache_slots, const float* __restrict__ vmix, float* __restrict__ v_first, int v_mode,
                     int* __restrict__ err) {
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= in.channels) return;
  const TapsRow row = taps_row(in, t);
  const int cq = nh * d, ck = nkv * d;
  float y = taps_value(in, row, t, c, false);
  if (c < cq + ck) {
    const int e = (c < cq ? c : c - cq) % d;
    if (e < rot_dim) {
      const int half = rot_dim >> 1;
      const bool low = e < half;
      const float other = taps_value(in, row, t, low ? c + half : c - half, false);
      const float angle = static_cast<float>(positions[t]) * inv_freq[low ? e : e - half];
      float sn, cs;
      sincosf(angle, &sn, &cs);
      y = low ? y * cs - other * sn : y * cs + other * sn;
    }
    if (c < cq) {
      q_out[static_cast<size_t>(t) * cq + c] = from_f32<T>(y);
      return;
    }
  } else {
    const int cv = c - cq - ck;
    const size_t at = static_cast<size_t>(t) * (nkv * dv) + cv;
    if (v_mode == 1) {
      v_first[at] = y;
    } else if (v_mode == 2) {
      const float lam = vmix[0];
      y = (1.0f - lam) * y + lam * v_first[at];
    }
  }
  if (slots == nullptr) return;
  const int slot = slots[t];
  if (slot < 0 || slot >= cache_slots) {
    atomicOr(err, B200_ERR_SLOT_RANGE);
    return;
  }
  const int page = slot / page_size, off = slot - page * page_size;
  if (c < cq + ck) {
    const int kc = c - cq, kvh = kc / d, e = kc - kvh * d;
    k_cache[((static_cast<size_t>(page) * nkv + kvh) * page_size + off) * d + e] = from_f32<T>(y);
  } else {
    const int cv = c - cq - ck, kvh = cv / dv, e = cv - kvh * dv;
    v_cache[((static_cast<size_t>(page) * nkv + kvh) * page_size + off) * dv + e] = from_f32<T>(y);
  }
}

template <typename T>
static int launch(const void* x, int in_stride, const float* w, int taps, float* state, const int* row_of_token,
                  const int* cu_q, const int* prefix_len, const int* state_slots, void* q_out, void* k_cache,
                  void* v_cache, const float* inv_freq, int rot_dim, const int* positions, const int* slots, int nh,
                  int nkv, int d, int dv, int page_size, long long cache_slots, const float* vmix, float* v_first,
                  int v_mode, int tokens, int* err, cudaStream_t stream) {
  TapsInput<T> in;
  in.x = static_cast<const T*>(x); in.in_stride = in_stride; in.scale = nullptr; in.w = w; in.taps = w ? taps : 1;
  in.channels = nh * d + nkv * d + nkv * dv; in.state = state; in.row_of_token = row_of_token; in.cu_q = cu_q;
  in.prefix_len = prefix_len; in.state_slots = state_slots;
  const dim3 grid(tokens, (in.channels + 255) / 256);
  conv_qkv_post_kernel<T><<<grid, 256, 0, stream>>>(in, static_cast<T*>(q_out), static_cast<T*>(k_cache),
                                                    static_cast<T*>(v_cache), inv_freq, rot_dim, positions, slots, nh,
                                                    nkv, d, dv, page_size, cache_slots, vmix, v_first, v_mode, err);
  return b200_check_launch();
}

// `x` [tokens, in_stride] holds q (nh * d), k (nkv * d), v (nkv * dv) side by side in its first columns.
B200_EXPORT int b200_conv_qkv_post(const void* x, int dtype, int in_stride, const float* w, int taps, float* state,
                                   const int* row_of_token, const int* cu_q, const int* prefix_len,
                                   const int* state_slots, void* q_out, void* k_cache, void* v_cache,
                                   const float* inv_freq, int rot_dim, const int* positions, const int* slots, int nh,
                                   int nkv, int d, int dv, int page_size, long long cache_slots, const float* vmix,
                                   float* v_first, int v_mode, int tokens, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || rot_dim < 0 || rot_dim > d || (rot_dim & 1))
    return B200_BAD_SIZE;
  if (w != nullptr && (taps < 1 || taps > TAPS_MAX)) return B200_BAD_SIZE;
  if ((v_mode == 2 && (vmix == nullptr || v_first == nullptr)) || (v_mode == 1 && v_first == nullptr)) return B200_BAD_SIZE;
  if ((nh * d + nkv * d + nkv * dv + 255) / 256 > 65535) return B200_BAD_SIZE;
  if (dtype == B200_F32)
    return launch<float>(x, in_stride, w, taps, state, row_of_token, cu_q, prefix_len, state_slots, q_out, k_cache,
                         v_cache, inv_freq, rot_dim, positions, slots, nh, nkv, d, dv, page_size, cache_slots, vmix,
                         v_first, v_mode, tokens, err, stream);
  if (dtype == B200_BF16)
    return launch<__nv_bfloat16>(x, in_stride, w, taps, state, row_of_token, cu_q, prefix_len, state_slots, q_out,
                                 k_cache, v_cache, inv_freq, rot_dim, positions, slots, nh, nkv, d, dv, page_size,
                                 cache_slots, vmix, v_first, v_mode, tokens, err, stream);
  return B200_BAD_DTYPE;
}
