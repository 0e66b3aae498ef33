// Between the packed q/k/v projection and attention, for a mixer whose q, k and v pass through a short causal
// convolution over time: the convolution (inputs before the step come from the request's state, token_conv.cuh),
// the half-split rotation of q and k by angles computed from the position, an optional mix of v with the v of an
// earlier layer, and the stores: q to its buffer, k and v (as they will be attended) into the paged cache; then the
// rows' convolution states are brought up to date (as in token_conv.cu).
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

// ------------------------------------------------------------------ eight channels a thread
// The same result for sizes whose rows are whole 16-byte pieces (d, dv, rot_dim / 2 and the rows of `x` multiples
// of 8): a thread takes 8 consecutive channels, and in the rotated part of a head also their 8 partners, so that
// every channel passes the convolution once and every pair takes one sine and cosine.  A head has
// rot_dim / 16 paired items and (d - rot_dim) / 8 single ones; v has dv / 8 single items per head.
template <typename T>
__global__ void __launch_bounds__(128)
conv_qkv_post_vec_kernel(TapsInput<T> in, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                         const float* __restrict__ inv_freq, int rot_dim, const int* __restrict__ positions,
                         const int* __restrict__ slots, int nh, int nkv, int d, int dv, int page_size,
                         long long cache_slots, const float* __restrict__ vmix, float* __restrict__ v_first,
                         int v_mode, int* __restrict__ err) {
  const int t = blockIdx.x;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  const int half = rot_dim >> 1;
  const int per_head = half / 8 + (d - rot_dim) / 8;
  const int qk_items = (nh + nkv) * per_head;
  if (item >= qk_items + nkv * (dv / 8)) return;
  const TapsRow row = taps_row(in, t);
  const bool own = taps_single(in, t);
  const int cq = nh * d, ck = nkv * d;
  int slot = -1, page = 0, off = 0;
  if (slots != nullptr) {
    slot = slots[t];
    if (slot < 0 || slot >= cache_slots) {
      if (item == 0) atomicOr(err, B200_ERR_SLOT_RANGE);
      slot = -1;
    } else {
      page = slot / page_size;
      off = slot - page * page_size;
    }
  }
  float a[8], b[8];
  if (item < qk_items) {
    const int head = item / per_head, part = item - head * per_head;          // q heads first, then k heads
    const bool paired = part < half / 8;
    const int e = paired ? part * 8 : rot_dim + (part - half / 8) * 8;
    const int c = head * d + e;                                               // (q and k channels are contiguous)
    taps_value8(in, row, t, c, false, own, a);
    if (paired) {
      taps_value8(in, row, t, c + half, false, own, b);
      const float pos = static_cast<float>(positions[t]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float sn, cs;
        sincosf(pos * inv_freq[e + i], &sn, &cs);
        const float lo = a[i] * cs - b[i] * sn, hi = b[i] * cs + a[i] * sn;
        a[i] = lo; b[i] = hi;
      }
    }
    T* dst;
    if (head < nh) {
      dst = q_out + static_cast<size_t>(t) * cq + c;
    } else {
      if (slot < 0) return;
      dst = k_cache + ((static_cast<size_t>(page) * nkv + (head - nh)) * page_size + off) * d + e;
    }
    store8<T>(dst, a);
    if (paired) store8<T>(dst + half, b);
    return;
  }
  const int vi = item - qk_items;
  const int kvh = vi / (dv / 8), e = (vi - kvh * (dv / 8)) * 8;
  taps_value8(in, row, t, cq + ck + kvh * dv + e, false, own, a);
  float* vf = v_first + static_cast<size_t>(t) * (nkv * dv) + kvh * dv + e;
  if (v_mode == 1) {
    *reinterpret_cast<float4*>(vf) = make_float4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<float4*>(vf + 4) = make_float4(a[4], a[5], a[6], a[7]);
  } else if (v_mode == 2) {
    const float lam = vmix[0];
    load_floats<float, 8>(vf, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = (1.0f - lam) * a[i] + lam * b[i];
  }
  if (slot < 0) return;
  store8<T>(v_cache + ((static_cast<size_t>(page) * nkv + kvh) * page_size + off) * dv + e, a);
}

template <typename T>
static int launch(const void* x, int in_stride, const float* w, int taps, float* state, const int* row_of_token,
                  const int* cu_q, const int* prefix_len, const int* state_slots, void* q_out, void* k_cache,
                  void* v_cache, const float* inv_freq, int rot_dim, const int* positions, const int* slots, int nh,
                  int nkv, int d, int dv, int page_size, long long cache_slots, const float* vmix, float* v_first,
                  int v_mode, int tokens, int num_rows, int all_single, int* err, cudaStream_t stream) {
  TapsInput<T> in;
  in.x = static_cast<const T*>(x); in.in_stride = in_stride; in.scale = nullptr; in.w = w; in.taps = w ? taps : 1;
  in.channels = nh * d + nkv * d + nkv * dv; in.state = state; in.row_of_token = row_of_token; in.cu_q = cu_q;
  in.prefix_len = prefix_len; in.state_slots = state_slots;
  const int half = rot_dim / 2;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q_out) |
                        reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                        reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(v_first)) % 16 == 0;
  if (aligned && d % 8 == 0 && dv % 8 == 0 && half % 8 == 0 && in_stride % 8 == 0) {
    const int items = (nh + nkv) * (half / 8 + (d - rot_dim) / 8) + nkv * (dv / 8);
    const dim3 vgrid(tokens, (items + 127) / 128);
    conv_qkv_post_vec_kernel<T><<<vgrid, 128, 0, stream>>>(in, static_cast<T*>(q_out), static_cast<T*>(k_cache),
                                                           static_cast<T*>(v_cache), inv_freq, rot_dim, positions, slots,
                                                           nh, nkv, d, dv, page_size, cache_slots, vmix, v_first, v_mode,
                                                           err);
    int rc = b200_check_launch();
    if (rc != 0 || in.taps <= 1 || all_single) return rc;
    taps_state_update_kernel<T><<<dim3(num_rows, (in.channels + 255) / 256), 256, 0, stream>>>(in, num_rows, 1);
    return b200_check_launch();
  }
  const dim3 grid(tokens, (in.channels + 255) / 256);
  conv_qkv_post_kernel<T><<<grid, 256, 0, stream>>>(in, static_cast<T*>(q_out), static_cast<T*>(k_cache),
                                                    static_cast<T*>(v_cache), inv_freq, rot_dim, positions, slots, nh,
                                                    nkv, d, dv, page_size, cache_slots, vmix, v_first, v_mode, err);
  int rc = b200_check_launch();
  if (rc != 0 || in.taps <= 1) return rc;
  taps_state_update_kernel<T><<<dim3(num_rows, (in.channels + 255) / 256), 256, 0, stream>>>(in, num_rows, 0);
  return b200_check_launch();
}

// `x` [tokens, in_stride] holds q (nh * d), k (nkv * d), v (nkv * dv) side by side in its first columns.
B200_EXPORT int b200_conv_qkv_post(const void* x, int dtype, int in_stride, const float* w, int taps, float* state,
                                   const int* row_of_token, const int* cu_q, const int* prefix_len,
                                   const int* state_slots, void* q_out, void* k_cache, void* v_cache,
                                   const float* inv_freq, int rot_dim, const int* positions, const int* slots, int nh,
                                   int nkv, int d, int dv, int page_size, long long cache_slots, const float* vmix,
                                   float* v_first, int v_mode, int tokens, int num_rows, int all_single, int* err,
                                   cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || rot_dim < 0 || rot_dim > d || (rot_dim & 1))
    return B200_BAD_SIZE;
  if (w != nullptr && (taps < 1 || taps > TAPS_MAX)) return B200_BAD_SIZE;
  if ((v_mode == 2 && (vmix == nullptr || v_first == nullptr)) || (v_mode == 1 && v_first == nullptr)) return B200_BAD_SIZE;
  if ((nh * d + nkv * d + nkv * dv + 255) / 256 > 65535) return B200_BAD_SIZE;
  if (dtype == B200_F32)
    return launch<float>(x, in_stride, w, taps, state, row_of_token, cu_q, prefix_len, state_slots, q_out, k_cache,
                         v_cache, inv_freq, rot_dim, positions, slots, nh, nkv, d, dv, page_size, cache_slots, vmix,
                         v_first, v_mode, tokens, num_rows, all_single, err, stream);
  if (dtype == B200_BF16)
    return launch<__nv_bfloat16>(x, in_stride, w, taps, state, row_of_token, cu_q, prefix_len, state_slots, q_out,
                                 k_cache, v_cache, inv_freq, rot_dim, positions, slots, nh, nkv, d, dv, page_size,
                                 cache_slots, vmix, v_first, v_mode, tokens, num_rows, all_single, err, stream);
  return B200_BAD_DTYPE;
}
