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
