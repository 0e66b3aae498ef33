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

// ------------------------------------------------------------------ prompt portions, in chunks of 64 tokens
// Four kernels.  (1) retention_rotate_kernel: q and k of every token rotated once (k also scaled) into float
// buffers qf, kf [tokens, heads * d].  (2a) retention_chunk_sum_kernel: every chunk's own contribution to the state,
// all chunks at once; (2b) retention_fold_kernel: chunk by chunk, element by element, the state as it stands
// BEFORE each chunk is left in `before` [chunk slot, heads, d, dv] and the row's final state is written.
// (3) retention_chunk_kernel: grid (chunk slots, heads), every chunk on its own:
//     o_i = decay^(i+1) q_i^T S_before + sum over j <= i of decay^(i-j) (q_i . k_j) v_j
// as two small float products in shared memory (A = Q K^T with the decays, then [A | Q diag] [V ; S_before]).
// Chunk slots of row r start at chunk_base[r] (a prefix sum on the device, made by retention_chunk_base_kernel).
// The state after a portion differs from the token-by-token recurrence by the order of float additions only.
constexpr int RC = 64;         // tokens of a chunk
constexpr int RD = 128;        // widest head (keys and values) of the chunked path

template <typename T>
__global__ void __launch_bounds__(256)
retention_rotate_kernel(const T* __restrict__ x, int in_stride, float* __restrict__ qf, float* __restrict__ kf,
                        const float* __restrict__ inv_freq, int rot_dim, float k_scale,
                        const int* __restrict__ positions, int heads, int d) {
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int hd = heads * d;
  if (c >= 2 * hd) return;
  const bool is_k = c >= hd;
  const int cc = is_k ? c - hd : c;
  const int h = cc / d, e = cc - h * d;
  const T* src = x + static_cast<size_t>(t) * in_stride + (is_k ? hd : 0) + h * d;
  const float y = rotated<T>(src, e, rot_dim, static_cast<float>(positions[t]), inv_freq);
  (is_k ? kf : qf)[static_cast<size_t>(t) * hd + cc] = is_k ? y * k_scale : y;
}

__global__ void retention_chunk_base_kernel(const int* __restrict__ cu_q, int num_rows, int* __restrict__ chunk_base) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int at = 0;
    for (int r = 0; r < num_rows; ++r) {
      chunk_base[r] = at;
      at += (cu_q[r + 1] - cu_q[r] + RC - 1) / RC;
    }
    chunk_base[num_rows] = at;
  }
}

// (2a) A block owns a 32 x 64 tile of one chunk's own contribution U = sum over j < L of decay^(L-1-j) k_j v_j^T;
// a thread 4 rows (4 ty ..) of 2 columns (2 tx, 2 tx + 1).  k is multiplied by its power of the decay as it is
// staged, so a token costs a thread one 16-byte load of k that the whole warp shares, one 8-byte load of v and
// 8 FMAs.  U goes where the state before the chunk will stand (`before`); (2b) folds the chunks together.
constexpr int RS_I = 32, RS_J = 64;
template <typename T>
__global__ void __launch_bounds__(256)
retention_chunk_sum_kernel(const T* __restrict__ x, int in_stride, const float* __restrict__ kf,
                           float* __restrict__ before, const float* __restrict__ decay, const int* __restrict__ cu_q,
                           const int* __restrict__ chunk_base, int num_rows, int heads, int d, int dv) {
  __shared__ __align__(16) float ks[RC][RS_I + 4];
  __shared__ __align__(16) float vs[RC][RS_J + 2];
  const int slot = blockIdx.x, h = blockIdx.y;
  if (slot >= chunk_base[num_rows]) return;
  int r = 0;
  while (chunk_base[r + 1] <= slot) ++r;
  const int first = cu_q[r], n = cu_q[r + 1] - first;
  const int base = (slot - chunk_base[r]) * RC;
  const int L = min(RC, n - base);
  const int tiles_v = (dv + RS_J - 1) / RS_J;
  const int ti = blockIdx.z / tiles_v, tj = blockIdx.z - ti * tiles_v;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = tj * RS_J + 2 * tx, row0 = ti * RS_I + 4 * ty;
  const float lg = log2f(decay[h]);
  const int voff = 2 * heads * d + h * dv;
  const bool k_ok = ti * RS_I + tx < d, v0_ok = tj * RS_J + tx < dv, v1_ok = tj * RS_J + 32 + tx < dv;
  const float* kcol = kf + static_cast<size_t>(h) * d + ti * RS_I + tx;
  const T* vcol = x + voff + tj * RS_J + tx;
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int j = ty + 8 * m;
    const size_t t = static_cast<size_t>(first + base + j);
    const float w = L - 1 - j == 0 ? 1.0f : exp2f(static_cast<float>(L - 1 - j) * lg);
    ks[j][tx] = (j < L && k_ok) ? kcol[t * heads * d] * w : 0.0f;
    vs[j][tx] = (j < L && v0_ok) ? to_f32<T>(vcol[t * in_stride]) : 0.0f;
    vs[j][tx + 32] = (j < L && v1_ok) ? to_f32<T>(vcol[t * in_stride + 32]) : 0.0f;
  }
  __syncthreads();
  float U[4][2] = {};
#pragma unroll 8
  for (int j = 0; j < RC; ++j) {                    // rows beyond L hold zeros
    const float4 k4 = *reinterpret_cast<const float4*>(&ks[j][4 * ty]);
    const float2 v2 = *reinterpret_cast<const float2*>(&vs[j][2 * tx]);
    U[0][0] = fmaf(k4.x, v2.x, U[0][0]); U[0][1] = fmaf(k4.x, v2.y, U[0][1]);
    U[1][0] = fmaf(k4.y, v2.x, U[1][0]); U[1][1] = fmaf(k4.y, v2.y, U[1][1]);
    U[2][0] = fmaf(k4.z, v2.x, U[2][0]); U[2][1] = fmaf(k4.z, v2.y, U[2][1]);
    U[3][0] = fmaf(k4.w, v2.x, U[3][0]); U[3][1] = fmaf(k4.w, v2.y, U[3][1]);
  }
  float* dst = before + (static_cast<size_t>(slot) * heads + h) * d * dv;
#pragma unroll
  for (int m = 0; m < 4; ++m)
    if (row0 + m < d && col < dv)
      *reinterpret_cast<float2*>(dst + static_cast<size_t>(row0 + m) * dv + col) = make_float2(U[m][0], U[m][1]);
}

// (2b) grid (rows, heads, pieces of 256 elements): S = the row's state (zeros at a sequence's start); chunk by
// chunk, what `before` holds (U) is replaced by S and S becomes decay^L S + U; the last S is the row's new state.
// One element a thread (many warps an SM) and four chunks' U fetched before the four dependent updates: the walk
// over a row's chunks is a chain of loads, and only loads in flight hide their latency.
__global__ void __launch_bounds__(256)
retention_fold_kernel(float* __restrict__ before, float* __restrict__ state, const float* __restrict__ decay,
                      const int* __restrict__ cu_q, const int* __restrict__ prefix_len,
                      const int* __restrict__ state_slots, const int* __restrict__ chunk_base, int heads, int d, int dv) {
  const int r = blockIdx.x, h = blockIdx.y;
  const int at = blockIdx.z * blockDim.x + threadIdx.x;
  const int size = d * dv;
  if (at >= size) return;
  const int n = cu_q[r + 1] - cu_q[r];
  const int chunks = (n + RC - 1) / RC;
  const float lg = log2f(decay[h]);
  float* st = state + (static_cast<size_t>(state_slots[r]) * heads + h) * size + at;
  float S = prefix_len[r] > 0 ? *st : 0.0f;
  const float whole = exp2f(static_cast<float>(RC) * lg);
  const float last = n % RC == 0 ? whole : exp2f(static_cast<float>(n % RC) * lg);
  float* slot = before + (static_cast<size_t>(chunk_base[r]) * heads + h) * size + at;
  const size_t step = static_cast<size_t>(heads) * size;
  int c = 0;
  for (; c + 4 <= chunks; c += 4) {
    float u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) u[i] = slot[(c + i) * step];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      slot[(c + i) * step] = S;
      S = fmaf(c + i == chunks - 1 ? last : whole, S, u[i]);
    }
  }
  for (; c < chunks; ++c) {
    const float u = slot[c * step];
    slot[c * step] = S;
    S = fmaf(c == chunks - 1 ? last : whole, S, u);
  }
  *st = S;
}

// acc[TM][TN] += sum over k < K of At[k][row0 + a] * B[k][col0 + b]; At and B in shared memory, k-major, with
// row strides, row0 and col0 that are multiples of 4 floats (16-byte loads)
template <int TM, int TN>
__device__ __forceinline__ void tile_product(const float* At, int lda, const float* B, int ldb, int K, int row0,
                                             int col0, float (&acc)[TM][TN]) {
  static_assert(TM % 4 == 0 && TN % 4 == 0, "whole 16-byte pieces");
#pragma unroll 2
  for (int k = 0; k < K; ++k) {
    float a[TM], b[TN];
#pragma unroll
    for (int i = 0; i < TM; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(At + k * lda + row0 + i);
      a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
    }
#pragma unroll
    for (int j = 0; j < TN; j += 4) {
      const float4 v = *reinterpret_cast<const float4*>(B + k * ldb + col0 + j);
      b[j] = v.x; b[j + 1] = v.y; b[j + 2] = v.z; b[j + 3] = v.w;
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// The same with the TM x 8 results in two groups of four columns, col0 .. and 64 + col0 ..: the 16 threads of a
// row then read 16 neighbouring 16-byte pieces of B (no two of a quarter-warp in one bank)
template <int TM>
__device__ __forceinline__ void tile_product_split(const float* At, int lda, const float* B, int ldb, int K, int row0,
                                                   int col0, float (&acc)[TM][8]) {
#pragma unroll 2
  for (int k = 0; k < K; ++k) {
    float a[TM], b[8];
#pragma unroll
    for (int i = 0; i < TM; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(At + k * lda + row0 + i);
      a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
    }
    const float4 lo = *reinterpret_cast<const float4*>(B + k * ldb + col0);
    const float4 hi = *reinterpret_cast<const float4*>(B + k * ldb + 64 + col0);
    b[0] = lo.x; b[1] = lo.y; b[2] = lo.z; b[3] = lo.w; b[4] = hi.x; b[5] = hi.y; b[6] = hi.z; b[7] = hi.w;
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

constexpr int RC_LD = RC + 4;        // row stride of the k-major tiles [e][token]
constexpr int RV_LD = RD + 4;        // row stride of V and of a slab of S_before [k][column]
static_assert(RC * RV_LD <= RD * RC_LD, "V and the slabs of S_before take the place of K");
constexpr size_t kChunkSmemFloats = 2 * RD * RC_LD + RC * RC_LD + RC + 1;      // 87 KB: two blocks an SM

// d a multiple of 4 and dv a multiple of 8 (16-byte pieces of the float and of the bfloat16 rows).
template <typename T>
__global__ void __launch_bounds__(256, 2)
retention_chunk_kernel(const T* __restrict__ x, int in_stride, const float* __restrict__ qf,
                       const float* __restrict__ kf, const float* __restrict__ before, float* __restrict__ o,
                       const float* __restrict__ decay, const int* __restrict__ cu_q,
                       const int* __restrict__ chunk_base, int num_rows, int heads, int d, int dv) {
  extern __shared__ __align__(16) float smem[];
  float* qt = smem;                          // [d][RC_LD]: q, k-major
  float* kt = qt + RD * RC_LD;               // [d][RC_LD]: k, k-major; once A is made: V, then slabs of S_before
  float* at = kt + RD * RC_LD;               // [RC][RC_LD]: A transposed, at[j][i] = decay^(i-j) q_i . k_j (j <= i)
  float* pw = at + RC * RC_LD;               // decay^0 .. decay^RC
  float* vb = kt;                            // [RC][RV_LD]

  const int slot = blockIdx.x, h = blockIdx.y;
  if (slot >= chunk_base[num_rows]) return;
  int r = 0;
  while (chunk_base[r + 1] <= slot) ++r;     // the row of this chunk (a handful of rows)
  const int first = cu_q[r], n = cu_q[r + 1] - first;
  const int base = (slot - chunk_base[r]) * RC;
  const int L = min(RC, n - base);
  const int t0 = first + base;
  const float g = decay[h];
  const int hd = heads * d;
  const int voff = 2 * heads * d + h * dv;

  {
    // q and k: a thread fetches 16-byte pieces (4 consecutive e of one token), four pieces in flight
    const int pieces = d / 4, total = RC * pieces;
    for (int idx0 = threadIdx.x; idx0 < total; idx0 += 4 * blockDim.x) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * blockDim.x;
        const int i = idx / pieces, e = (idx - i * pieces) * 4;
        const bool ok = idx < total && i < L;
        const size_t at_ = static_cast<size_t>(t0 + (ok ? i : 0)) * hd + h * d + e;
        qv[u] = ok ? *reinterpret_cast<const float4*>(qf + at_) : make_float4(0.f, 0.f, 0.f, 0.f);
        kv[u] = ok ? *reinterpret_cast<const float4*>(kf + at_) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * blockDim.x;
        if (idx >= total) continue;
        const int i = idx / pieces, e = (idx - i * pieces) * 4;
        qt[(e + 0) * RC_LD + i] = qv[u].x; qt[(e + 1) * RC_LD + i] = qv[u].y;
        qt[(e + 2) * RC_LD + i] = qv[u].z; qt[(e + 3) * RC_LD + i] = qv[u].w;
        kt[(e + 0) * RC_LD + i] = kv[u].x; kt[(e + 1) * RC_LD + i] = kv[u].y;
        kt[(e + 2) * RC_LD + i] = kv[u].z; kt[(e + 3) * RC_LD + i] = kv[u].w;
      }
    }
  }
  if (threadIdx.x <= RC) pw[threadIdx.x] = threadIdx.x == 0 ? 1.0f : exp2f(static_cast<float>(threadIdx.x) * log2f(g));
  __syncthreads();
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;      // 16 x 16 threads
  // V of this chunk: fetched into registers now (8 columns a piece), stored over K once A is made
  const int vpieces = dv / 8, vtotal = RC * vpieces;
  float vreg[4][8];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int idx = threadIdx.x + u * blockDim.x;
    const int j = idx / vpieces, col = (idx - j * vpieces) * 8;
    if (idx < vtotal && j < L) {
      load_floats<T, 8>(x + static_cast<size_t>(t0 + j) * in_stride + voff + col, vreg[u]);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) vreg[u][q] = 0.0f;
    }
  }
  {
    // A[i][j] for i in 4 ty .., j in 4 tx ..
    float acc[4][4] = {};
    tile_product<4, 4>(qt, RC_LD, kt, RC_LD, d, ty * 4, tx * 4, acc);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int i = ty * 4 + a, j = tx * 4 + b;
        at[j * RC_LD + i] = j <= i ? acc[a][b] * pw[i - j] : 0.0f;
      }
  }
  __syncthreads();                                              // A is whole, K is free
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int idx = threadIdx.x + u * blockDim.x;
    if (idx < vtotal) {
      const int j = idx / vpieces, col = (idx - j * vpieces) * 8;
      *reinterpret_cast<float4*>(vb + j * RV_LD + col) = make_float4(vreg[u][0], vreg[u][1], vreg[u][2], vreg[u][3]);
      *reinterpret_cast<float4*>(vb + j * RV_LD + col + 4) = make_float4(vreg[u][4], vreg[u][5], vreg[u][6], vreg[u][7]);
    }
  }
  // the first slab of S_before on its way while A V runs
  const float* sb = before + (static_cast<size_t>(slot) * heads + h) * d * dv;
  const int spieces = dv / 4;
  float4 sreg[8];
  auto fetch_slab = [&](int e0) {
    const int rows = min(RC, d - e0), total = rows * spieces;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = threadIdx.x + u * blockDim.x;
      const int e = idx / spieces, col = (idx - e * spieces) * 4;
      sreg[u] = idx < total ? *reinterpret_cast<const float4*>(sb + static_cast<size_t>(e0 + e) * dv + col)
                            : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto store_slab = [&](int e0) {
    const int rows = min(RC, d - e0), total = rows * spieces;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = threadIdx.x + u * blockDim.x;
      if (idx < total) {
        const int e = idx / spieces, col = (idx - e * spieces) * 4;
        *reinterpret_cast<float4*>(vb + e * RV_LD + col) = sreg[u];
      }
    }
  };
  __syncthreads();
  fetch_slab(0);
  // o[i][col] for i in 4 ty .., col in 4 tx .. and 64 + 4 tx ..: A V first, then decay^(i+1) q_i^T S_before
  float out[4][8] = {};
  tile_product_split<4>(at, RC_LD, vb, RV_LD, RC, ty * 4, tx * 4, out);
  float inter[4][8] = {};
  for (int e0 = 0; e0 < d; e0 += RC) {
    __syncthreads();                                            // vb is free
    store_slab(e0);
    __syncthreads();
    if (e0 + RC < d) fetch_slab(e0 + RC);
    tile_product_split<4>(qt + e0 * RC_LD, RC_LD, vb, RV_LD, min(RC, d - e0), ty * 4, tx * 4, inter);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = ty * 4 + a;
    if (i >= L) continue;
    const float w = pw[i] * g;                                  // decay^(i+1)
    float* dst = o + (static_cast<size_t>(t0 + i) * heads + h) * dv;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int col = half * 64 + tx * 4;
      if (col < dv)
        *reinterpret_cast<float4*>(dst + col) =
            make_float4(fmaf(w, inter[a][half * 4 + 0], out[a][half * 4 + 0]), fmaf(w, inter[a][half * 4 + 1], out[a][half * 4 + 1]),
                        fmaf(w, inter[a][half * 4 + 2], out[a][half * 4 + 2]), fmaf(w, inter[a][half * 4 + 3], out[a][half * 4 + 3]));
    }
  }
}

template <typename T>
static int launch_chunked(const void* x, int in_stride, float* o, float* state, const float* decay,
                          const float* inv_freq, int rot_dim, float k_scale, const int* positions, const int* cu_q,
                          const int* prefix_len, const int* state_slots, int num_rows, int heads, int d, int dv,
                          int tokens, int max_chunks, float* qf, float* kf, float* before, int* chunk_base,
                          cudaStream_t stream) {
  const T* xt = static_cast<const T*>(x);
  retention_rotate_kernel<T><<<dim3(tokens, (2 * heads * d + 255) / 256), 256, 0, stream>>>(
      xt, in_stride, qf, kf, inv_freq, rot_dim, k_scale, positions, heads, d);
  retention_chunk_base_kernel<<<1, 32, 0, stream>>>(cu_q, num_rows, chunk_base);
  const dim3 ugrid(max_chunks, heads, ((d + RS_I - 1) / RS_I) * ((dv + RS_J - 1) / RS_J));
  retention_chunk_sum_kernel<T><<<ugrid, 256, 0, stream>>>(xt, in_stride, kf, before, decay, cu_q, chunk_base, num_rows,
                                                           heads, d, dv);
  const dim3 fgrid(num_rows, heads, (d * dv + 255) / 256);
  retention_fold_kernel<<<fgrid, 256, 0, stream>>>(before, state, decay, cu_q, prefix_len, state_slots, chunk_base,
                                                    heads, d, dv);
  const size_t smem = kChunkSmemFloats * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(retention_chunk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  retention_chunk_kernel<T><<<dim3(max_chunks, heads), 256, smem, stream>>>(xt, in_stride, qf, kf, before, o, decay, cu_q,
                                                                             chunk_base, num_rows, heads, d, dv);
  return b200_check_launch();
}

// The same result as b200_retention for steps with long rows.  `max_chunks` bounds the step's chunks of 64 tokens
// (sum over rows of ceil(tokens of the row / 64)); scratch: qf, kf [tokens, heads * d] floats, before
// [max_chunks, heads, d, dv] floats, chunk_base [num_rows + 1] ints.  Heads up to 128 wide, d a multiple of 4, dv and
// the rows of x multiples of 8.
B200_EXPORT int b200_retention_chunked(const void* x, int dtype, int in_stride, float* o, float* state,
                                       const float* decay, const float* inv_freq, int rot_dim, float k_scale,
                                       const int* positions, const int* cu_q, const int* prefix_len,
                                       const int* state_slots, int num_rows, int heads, int d, int dv, int tokens,
                                       int max_chunks, float* qf, float* kf, float* before, int* chunk_base,
                                       cudaStream_t stream) {
  if (num_rows <= 0 || tokens <= 0) return 0;
  if (heads <= 0 || heads > 65535 || d <= 0 || d > RD || dv <= 0 || dv > RD || rot_dim < 0 || rot_dim > d ||
      (rot_dim & 1) || max_chunks <= 0 || d % 4 != 0 || dv % 8 != 0 || in_stride % 8 != 0 ||
      reinterpret_cast<uintptr_t>(x) % 16 != 0)
    return B200_BAD_SIZE;
  if (dtype == B200_F32)
    return launch_chunked<float>(x, in_stride, o, state, decay, inv_freq, rot_dim, k_scale, positions, cu_q,
                                 prefix_len, state_slots, num_rows, heads, d, dv, tokens, max_chunks, qf, kf, before,
                                 chunk_base, stream);
  if (dtype == B200_BF16)
    return launch_chunked<__nv_bfloat16>(x, in_stride, o, state, decay, inv_freq, rot_dim, k_scale, positions, cu_q,
                                         prefix_len, state_slots, num_rows, heads, d, dv, tokens, max_chunks, qf, kf,
                                         before, chunk_base, stream);
  return B200_BAD_DTYPE;
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
