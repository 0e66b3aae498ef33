// A mixture of small gated feed-forward experts whose choice is a table lookup: the row of a token's id in an
// integer table [vocab, top] names its experts, each with weight 1 / top.
//
//   expert e:  y = W_down[e] (silu(W_gate[e] x) * (W_up[e] x))          out[t] = (1 / top) sum_k y_(t, k)
//
// Four kernels, nothing goes through the host (a step can be captured in a graph):
//   expert_route       (token, choice) pairs sorted by expert: sorted_token[pos], pos_of_pair[pair], the experts'
//                      ranges and the list of row tiles (expert, first row) that the products walk
//   expert_gate_up     H[pos] = silu(gate) * up for every sorted pair, rows of x gathered by token
//   expert_down        Y[pos] = W_down[e] H[pos], in float
//   expert_combine     out[t] = (sum over k in order of Y[pos_of_pair[t * top + k]]) / top, in float
//
// Weights: gate_up [experts, 2 * ff, width] (an expert's gate rows, then its up rows), down [experts, width, ff].
// float32: FFMA, every output accumulated over k in order (a pair's result does not depend on its place in a tile,
// so the order in which pairs of one expert were sorted does not show).  bfloat16: tensor cores with float
// accumulation, H rounded once to bfloat16.
#include <mma.h>

#include "common.cuh"

constexpr int TM = 64, TN = 64;      // rows (sorted pairs) and columns of a tile

// ------------------------------------------------------------------ routing
// one block; shared memory: 2 * experts + 1 ints
__global__ void __launch_bounds__(1024)
expert_route_kernel(const int* __restrict__ token_ids, const int* __restrict__ table, int vocab, int top, int experts,
                    int tokens, int* __restrict__ sorted_token, int* __restrict__ pos_of_pair,
                    int* __restrict__ expert_start, int* __restrict__ tile_expert, int* __restrict__ tile_first,
                    int* __restrict__ num_tiles, int tile_rows, int* err) {
  extern __shared__ int sm[];
  int* count = sm;                    // [experts]
  int* start = sm + experts;          // [experts + 1]
  const int pairs = tokens * top;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int id = token_ids[i / top];
    int e = (id >= 0 && id < vocab) ? table[static_cast<size_t>(id) * top + i % top] : -1;
    if (e < 0 || e >= experts) { atomicOr(err, B200_ERR_TOKEN_RANGE); e = 0; }
    atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, n = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at;
      expert_start[e] = at;
      for (int r = at; r < at + count[e]; r += tile_rows) { tile_expert[n] = e; tile_first[n] = r; ++n; }
      at += count[e];
    }
    start[experts] = at;
    expert_start[experts] = at;
    *num_tiles = n;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int id = token_ids[i / top];
    int e = (id >= 0 && id < vocab) ? table[static_cast<size_t>(id) * top + i % top] : 0;
    if (e < 0 || e >= experts) e = 0;
    const int pos = start[e] + atomicAdd(&count[e], 1);
    sorted_token[pos] = i / top;
    pos_of_pair[i] = pos;
  }
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// ------------------------------------------------------------------ float32 products
// GATED: C[pos][n] = silu(A . Wg[n]) * (A . Wu[n]) with A rows gathered by sorted_token; else C[pos][n] = A[pos] . W[n].
// grid (column tiles, row tiles); 256 threads, 4 x 4 outputs a thread; k in steps of 16.
template <bool GATED>
__global__ void __launch_bounds__(256)
expert_gemm_f32_kernel(const float* __restrict__ A, int lda, const int* __restrict__ gather,
                       const float* __restrict__ W, long long w_expert_stride, int up_row_offset,
                       float* __restrict__ C, int N, int K, const int* __restrict__ expert_start,
                       const int* __restrict__ tile_expert, const int* __restrict__ tile_first,
                       const int* __restrict__ num_tiles) {
  constexpr int BK = 16;
  if (static_cast<int>(blockIdx.y) >= *num_tiles) return;
  __shared__ float As[BK][TM + 4];
  __shared__ float Ws[GATED ? 2 : 1][BK][TN + 4];
  const int e = tile_expert[blockIdx.y], r0 = tile_first[blockIdx.y];
  const int r_end = min(r0 + TM, expert_start[e + 1]);
  const int n0 = blockIdx.x * TN;
  const float* We = W + e * w_expert_stride;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int arow = r0 + lrow;
  const float* a_src = nullptr;
  if (arow < r_end) a_src = A + static_cast<size_t>(gather ? gather[arow] : arow) * lda;
  const int wn = n0 + lrow;
  float acc[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    float a[4], w[GATED ? 2 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kk = k0 + lk + i;
      a[i] = (a_src != nullptr && kk < K) ? a_src[kk] : 0.0f;
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
        w[g][i] = (wn < N && kk < K) ? We[static_cast<size_t>(wn + g * up_row_offset) * K + kk] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lrow] = a[i];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g) Ws[g][lk + i][lrow] = w[g][i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g) {
        const float4 wv = *reinterpret_cast<const float4*>(&Ws[g][k][tx * 4]);
        const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(ar[i], wr[j], acc[g][i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty * 4 + i;
    if (r >= r_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if constexpr (GATED) C[static_cast<size_t>(r) * N + n] = silu_f(acc[0][i][j]) * acc[1][i][j];
      else C[static_cast<size_t>(r) * N + n] = acc[0][i][j];
    }
  }
}

// ------------------------------------------------------------------ bfloat16 products on tensor cores
// The same tiles; 8 warps, warp w owns rows 16 * (w / 2) .. and columns 32 * (w % 2) .. of the tile (two 16 x 16
// accumulators, four when GATED); k in steps of 64 through shared memory, the next step's operands fetched into
// registers while the tensor cores work on this one (a decode step's products are a chain of such fetches: few rows
// an expert, all of its weights).  TO: bfloat16 (H) or float (Y).
template <bool GATED, typename TO>
__global__ void __launch_bounds__(256)
expert_gemm_bf16_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ gather,
                        const __nv_bfloat16* __restrict__ W, long long w_expert_stride, int up_row_offset,
                        TO* __restrict__ C, int N, int K, const int* __restrict__ expert_start,
                        const int* __restrict__ tile_expert, const int* __restrict__ tile_first,
                        const int* __restrict__ num_tiles) {
  using namespace nvcuda;
  constexpr int BK = 64, LD = BK + 8, G = GATED ? 2 : 1;
  if (static_cast<int>(blockIdx.y) >= *num_tiles) return;
  __shared__ __align__(32) __nv_bfloat16 As[TM][LD];
  __shared__ __align__(32) __nv_bfloat16 Ws[G][TN][LD];
  __shared__ __align__(32) float Cs[8][16][32 + 4];
  const int e = tile_expert[blockIdx.y], r0 = tile_first[blockIdx.y];
  const int r_end = min(r0 + TM, expert_start[e + 1]);
  const int n0 = blockIdx.x * TN;
  const __nv_bfloat16* We = W + e * w_expert_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wr = warp >> 1, wc = warp & 1;
  // loads: thread -> row tid / 4, sixteen k from (tid % 4) * 16, as two pieces of eight
  const int lrow = tid >> 2, lk = (tid & 3) * 16;
  const int arow = r0 + lrow;
  const __nv_bfloat16* a_src = nullptr;
  if (arow < r_end) a_src = A + static_cast<size_t>(gather ? gather[arow] : arow) * lda;
  const int wn = n0 + lrow;
  const __nv_bfloat16* w_src[G];
#pragma unroll
  for (int g = 0; g < G; ++g) w_src[g] = wn < N ? We + static_cast<size_t>(wn + g * up_row_offset) * K : nullptr;
  const bool vec = (K % 8 == 0) && (lda % 8 == 0) && (reinterpret_cast<uintptr_t>(A) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(W) % 16 == 0);
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[G][2];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[g][j], 0.0f);

  // eight elements of a row from k on, zeros beyond K or for a row that does not exist
  auto fetch8 = [&](const __nv_bfloat16* row, int k) -> uint4 {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row == nullptr || k >= K) return v;
    if (vec && k + 8 <= K) return *reinterpret_cast<const uint4*>(row + k);
    __align__(16) __nv_bfloat16 t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = k + i < K ? row[k + i] : __float2bfloat16_rn(0.0f);
    return *reinterpret_cast<const uint4*>(t);
  };
  uint4 ra[2], rw[G][2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    ra[h] = fetch8(a_src, lk + 8 * h);
#pragma unroll
    for (int g = 0; g < G; ++g) rw[g][h] = fetch8(w_src[g], lk + 8 * h);
  }
  for (int k0 = 0; k0 < K; k0 += BK) {
    __syncthreads();                                   // the step before is no longer read
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      *reinterpret_cast<uint4*>(&As[lrow][lk + 8 * h]) = ra[h];
#pragma unroll
      for (int g = 0; g < G; ++g) *reinterpret_cast<uint4*>(&Ws[g][lrow][lk + 8 * h]) = rw[g][h];
    }
    __syncthreads();
    if (k0 + BK < K) {                                 // the next step's operands are on their way during the products
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        ra[h] = fetch8(a_src, k0 + BK + lk + 8 * h);
#pragma unroll
        for (int g = 0; g < G; ++g) rw[g][h] = fetch8(w_src[g], k0 + BK + lk + 8 * h);
      }
    }
#pragma unroll
    for (int ks = 0; ks < BK; ks += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
      wmma::load_matrix_sync(fa, &As[wr * 16][ks], LD);
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
          wmma::load_matrix_sync(fb, &Ws[g][wc * 32 + j * 16][ks], LD);
          wmma::mma_sync(acc[g][j], fa, fb, acc[g][j]);
        }
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if constexpr (GATED) {          // both accumulators have one layout: element i of one meets element i of the other
#pragma unroll
      for (int i = 0; i < acc[0][j].num_elements; ++i) acc[0][j].x[i] = silu_f(acc[0][j].x[i]) * acc[G - 1][j].x[i];
    }
    wmma::store_matrix_sync(&Cs[warp][0][j * 16], acc[0][j], 32 + 4, wmma::mem_row_major);
  }
  __syncwarp();
  for (int i = lane; i < 16 * 32; i += 32) {
    const int rr = i >> 5, cc = i & 31;
    const int r = r0 + wr * 16 + rr, n = n0 + wc * 32 + cc;
    if (r >= r_end || n >= N) continue;
    C[static_cast<size_t>(r) * N + n] = from_f32<TO>(Cs[warp][rr][cc]);
  }
}

// ------------------------------------------------------------------ the experts' outputs back to the tokens
__global__ void __launch_bounds__(256)
expert_combine_kernel(float* __restrict__ out, const float* __restrict__ Y, const int* __restrict__ pos_of_pair,
                      int top, int width, float inv_top) {
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = 0.0f;
    for (int k = 0; k < top; ++k) s += Y[static_cast<size_t>(pos_of_pair[t * top + k]) * width + c];
    out[t * width + c] = s * inv_top;
  }
}

// ------------------------------------------------------------------ C interface
// Ints of scratch that the routing needs for (tokens, top, experts); row tiles of at least 64 rows.
B200_EXPORT long long b200_expert_route_ints(int tokens, int top, int experts) {
  const long long pairs = static_cast<long long>(tokens) * top;
  const long long tiles = (pairs + TM - 1) / TM + experts;
  return 2 * pairs + (experts + 1) + 2 * tiles + 1;
}

// Where the parts of the routing scratch lie.
struct RouteLayout {
  int *sorted_token, *pos_of_pair, *expert_start, *tile_expert, *tile_first, *num_tiles;
  int tiles;
};
static RouteLayout route_layout(int* route, int pairs, int experts) {
  RouteLayout r;
  r.tiles = (pairs + TM - 1) / TM + experts;
  r.sorted_token = route;
  r.pos_of_pair = r.sorted_token + pairs;
  r.expert_start = r.pos_of_pair + pairs;
  r.tile_expert = r.expert_start + experts + 1;
  r.tile_first = r.tile_expert + r.tiles;
  r.num_tiles = r.tile_first + r.tiles;
  return r;
}

// x [tokens, width] -> out [tokens, width] float32.  `h` holds pairs * ff elements of x's dtype, `y` pairs * width
// floats, `route` b200_expert_route_ints(...) ints.
B200_EXPORT int b200_table_experts(const void* x, int dtype, const int* token_ids, const int* table, int vocab, int top,
                                   int experts, const void* gate_up, const void* down, int tokens, int width, int ff,
                                   void* h, float* y, int* route, float* out, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top <= 0 || experts <= 0 || width <= 0 || ff <= 0 || vocab <= 0) return B200_BAD_SIZE;
  const long long pairs_ll = static_cast<long long>(tokens) * top;
  if (pairs_ll > (1ll << 30) || (2 * experts + 1) * sizeof(int) > 48 * 1024) return B200_BAD_SIZE;
  const int pairs = static_cast<int>(pairs_ll);
  const RouteLayout rl = route_layout(route, pairs, experts);
  const int tiles = rl.tiles;
  if (tiles > 65535) return B200_BAD_SIZE;
  int *sorted_token = rl.sorted_token, *pos_of_pair = rl.pos_of_pair, *expert_start = rl.expert_start;
  int *tile_expert = rl.tile_expert, *tile_first = rl.tile_first, *num_tiles = rl.num_tiles;
  expert_route_kernel<<<1, 1024, (2 * experts + 1) * sizeof(int), stream>>>(
      token_ids, table, vocab, top, experts, tokens, sorted_token, pos_of_pair, expert_start, tile_expert, tile_first,
      num_tiles, TM, err);
  int rc = b200_check_launch();
  if (rc != 0) return rc;
  const dim3 g1((ff + TN - 1) / TN, tiles), g2((width + TN - 1) / TN, tiles);
  const long long gu_stride = 2ll * ff * width, dn_stride = static_cast<long long>(width) * ff;
  if (dtype == B200_F32) {
    expert_gemm_f32_kernel<true><<<g1, 256, 0, stream>>>(
        static_cast<const float*>(x), width, sorted_token, static_cast<const float*>(gate_up), gu_stride, ff,
        static_cast<float*>(h), ff, width, expert_start, tile_expert, tile_first, num_tiles);
    expert_gemm_f32_kernel<false><<<g2, 256, 0, stream>>>(
        static_cast<const float*>(h), ff, nullptr, static_cast<const float*>(down), dn_stride, 0, y, width, ff,
        expert_start, tile_expert, tile_first, num_tiles);
  } else if (dtype == B200_BF16) {
    expert_gemm_bf16_kernel<true, __nv_bfloat16><<<g1, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), width, sorted_token, static_cast<const __nv_bfloat16*>(gate_up),
        gu_stride, ff, static_cast<__nv_bfloat16*>(h), ff, width, expert_start, tile_expert, tile_first, num_tiles);
    expert_gemm_bf16_kernel<false, float><<<g2, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(h), ff, nullptr, static_cast<const __nv_bfloat16*>(down), dn_stride, 0, y,
        width, ff, expert_start, tile_expert, tile_first, num_tiles);
  } else {
    return B200_BAD_DTYPE;
  }
  rc = b200_check_launch();
  if (rc != 0) return rc;
  expert_combine_kernel<<<tokens, 256, 0, stream>>>(out, y, pos_of_pair, top, width, 1.0f / static_cast<float>(top));
  return b200_check_launch();
}
