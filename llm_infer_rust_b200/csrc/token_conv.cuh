// The short causal convolution over time of token_conv.cu as device functions, so that a kernel which goes on
// with the result (a rotation, a cache store) can compute it where it needs it.
#pragma once
#include "common.cuh"

constexpr int TAPS_MAX = 8;

template <typename TI>
struct TapsInput {
  const TI* x;               // [tokens, in_stride]; channel c of token t at x[t * in_stride + c]
  int in_stride;
  const float* scale;        // per token, or null
  const float* w;            // [channels, taps]
  int taps;
  int channels;
  float* state;              // [slots + 1, taps - 1, channels], oldest first
  const int* row_of_token;
  const int* cu_q;
  const int* prefix_len;
  const int* state_slots;
};

struct TapsRow {
  int local;                 // index of the token inside its row of this step
  bool has_past;             // the row did not start at position 0
  const float* state;        // the row's state
};

template <typename TI>
__device__ __forceinline__ TapsRow taps_row(const TapsInput<TI>& in, int t) {
  const int r = in.row_of_token[t];
  TapsRow row;
  row.local = t - in.cu_q[r];
  row.has_past = in.prefix_len[r] > 0;
  row.state = in.state + static_cast<size_t>(in.state_slots[r]) * (in.taps - 1) * in.channels;
  return row;
}

// The input `back` steps before token t (back >= 0) on channel c.
template <typename TI>
__device__ __forceinline__ float taps_past(const TapsInput<TI>& in, const TapsRow& row, int t, int c, int back) {
  if (back <= row.local) {
    const int s = t - back;
    return to_f32<TI>(in.x[static_cast<size_t>(s) * in.in_stride + c]) * (in.scale ? in.scale[s] : 1.0f);
  }
  if (!row.has_past) return 0.0f;
  const int k = in.taps - 1 - (back - row.local);       // state k holds the input (taps - 1 - k) before the row's first token
  return row.state[static_cast<size_t>(k) * in.channels + c];
}

// sum_j w[c][j] * u[t - taps + 1 + j][c]  (+ u[t][c] with `identity`)
template <typename TI>
__device__ __forceinline__ float taps_value(const TapsInput<TI>& in, const TapsRow& row, int t, int c, bool identity) {
  const float now = taps_past(in, row, t, c, 0);
  if (in.taps <= 0 || in.w == nullptr) return now;
  const float* w = in.w + static_cast<size_t>(c) * in.taps;
  float y = identity ? now : 0.0f;
  for (int j = 0; j < in.taps; ++j) {
    const int back = in.taps - 1 - j;
    y = fmaf(w[j], back == 0 ? now : taps_past(in, row, t, c, back), y);
  }
  return y;
}

// ------------------------------------------------------------------ eight channels at a time
template <typename T>
__device__ __forceinline__ void store8(T* p, const float* v) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint4 u;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(v[0], v[1]); u.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(v[2], v[3]); u.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(v[4], v[5]); u.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(v[6], v[7]); u.w = *reinterpret_cast<uint32_t*>(&h);
    *reinterpret_cast<uint4*>(p) = u;
  }
}

// y[0..8) = the convolution's outputs of channels c .. c + 7 of token t (c a multiple of 8, rows of 16-byte pieces).
// The taps are walked from the oldest input to the newest.  `own_state`: the token is the only one of its row in
// this step, so this thread is the only reader of the row's state on these channels and brings it up to date
// itself (every entry moves one place towards the oldest, the newest input comes last): each entry is written
// after it was read, by the thread that read it.  TAPS > 0: the number of taps at compile time (the eight
// channels' weights are then fetched as 16-byte pieces into registers); 0: read from `in`.
template <typename T, int TAPS>
__device__ __forceinline__ void taps_value8_n(const TapsInput<T>& in, const TapsRow& row, int t, int c, bool identity,
                                              bool own_state, float* y) {
  float now[8], u[8];
  load_floats<T, 8>(in.x + static_cast<size_t>(t) * in.in_stride + c, now);
  if (in.scale != nullptr) {
    const float s = in.scale[t];
#pragma unroll
    for (int i = 0; i < 8; ++i) now[i] *= s;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) y[i] = identity ? now[i] : 0.0f;
  if (in.w == nullptr) {
    if (!identity) {
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = now[i];
    }
    return;
  }
  const int taps = TAPS > 0 ? TAPS : in.taps, hist = taps - 1;
  float wl[TAPS > 0 ? 8 * TAPS : 1] = {};
  if constexpr (TAPS > 0) load_floats<float, 8 * TAPS>(in.w + static_cast<size_t>(c) * TAPS, wl);
  auto weight = [&](int i, int j) { return TAPS > 0 ? wl[i * (TAPS > 0 ? TAPS : 1) + j] : in.w[static_cast<size_t>(c + i) * taps + j]; };
  float* st = const_cast<float*>(row.state);
#pragma unroll
  for (int step = 0; step < (TAPS > 0 ? TAPS - 1 : TAPS_MAX - 1); ++step) {
    const int back = hist - step;
    if (back < 1) break;
    bool have = true;
    if (back <= row.local) {
      load_floats<T, 8>(in.x + static_cast<size_t>(t - back) * in.in_stride + c, u);
      if (in.scale != nullptr) {
        const float s = in.scale[t - back];
#pragma unroll
        for (int i = 0; i < 8; ++i) u[i] *= s;
      }
    } else if (row.has_past) {
      load_floats<float, 8>(st + static_cast<size_t>(hist - (back - row.local)) * in.channels + c, u);
    } else {
      have = false;
#pragma unroll
      for (int i = 0; i < 8; ++i) u[i] = 0.0f;
    }
    if (have) {
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = fmaf(weight(i, step), u[i], y[i]);
    }
    if (own_state && back < hist) store8<float>(st + static_cast<size_t>(hist - 1 - back) * in.channels + c, u);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) y[i] = fmaf(weight(i, hist), now[i], y[i]);
  if (own_state && hist >= 1) store8<float>(st + static_cast<size_t>(hist - 1) * in.channels + c, now);
}

template <typename T>
__device__ __forceinline__ void taps_value8(const TapsInput<T>& in, const TapsRow& row, int t, int c, bool identity,
                                            bool own_state, float* y) {
  switch (in.w != nullptr ? in.taps : 0) {
    case 2: taps_value8_n<T, 2>(in, row, t, c, identity, own_state, y); break;
    case 3: taps_value8_n<T, 3>(in, row, t, c, identity, own_state, y); break;
    case 4: taps_value8_n<T, 4>(in, row, t, c, identity, own_state, y); break;
    default: taps_value8_n<T, 0>(in, row, t, c, identity, own_state, y); break;
  }
}

// Whether token t is the only token of its row in this step.
template <typename TI>
__device__ __forceinline__ bool taps_single(const TapsInput<TI>& in, int t) {
  const int r = in.row_of_token[t];
  return in.cu_q[r + 1] - in.cu_q[r] == 1;
}

// grid (rows, channel tiles of 256): new state k holds the input at position end - (taps - 1) + k.
// skip_single: rows of one token were brought up to date by the convolution kernel itself.
template <typename TI>
__global__ void __launch_bounds__(256)
taps_state_update_kernel(TapsInput<TI> in, int num_rows, int skip_single) {
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= in.channels || r >= num_rows) return;
  const int hist = in.taps - 1;
  const int first = in.cu_q[r], n = in.cu_q[r + 1] - first;
  if (skip_single && n == 1) return;
  const int prefix = in.prefix_len[r];
  const int slot = in.state_slots[r];
  float* st = in.state + static_cast<size_t>(slot) * hist * in.channels;
  float fresh[TAPS_MAX - 1];
#pragma unroll
  for (int k = 0; k < TAPS_MAX - 1; ++k) {
    if (k >= hist) break;
    const int pos = prefix + n - hist + k;            // absolute position that lands in state k
    float v = 0.0f;
    if (pos >= prefix) {
      const int t = first + (pos - prefix);
      v = to_f32<TI>(in.x[static_cast<size_t>(t) * in.in_stride + c]) * (in.scale ? in.scale[t] : 1.0f);
    } else if (pos >= 0 && prefix > 0) {
      v = st[static_cast<size_t>(pos - prefix + hist) * in.channels + c];
    }
    fresh[k] = v;
  }
#pragma unroll
  for (int k = 0; k < TAPS_MAX - 1; ++k) {
    if (k >= hist) break;
    st[static_cast<size_t>(k) * in.channels + c] = fresh[k];
  }
}

