// A routed feed-forward: every token goes through `top` of `n_exp` small gated feed-forwards.
//
// moe_route   one warp per token: scores from the router's float32 logits (sigmoid of each, or a
//             softmax over all), the `top` largest (ties: the lower index), optionally renormalised to
//             sum 1; the token takes a place in each chosen expert's group (an atomic counter per expert).
// moe_gather  one block per (token, choice): the token's input row, multiplied by the choice's weight
//             where the design scales the expert's INPUT, goes to its place in a buffer sorted by
//             expert (row = first row of the expert's group + the place taken above).
// moe_gemm    C[row][n] = sum_k A[row][k] W[expert of row][n][k] over the sorted rows: a CTA owns a tile
//             of rows of ONE expert (it finds expert and rows from the counters, so nothing about the
//             routing passes through the host) and a tile of output features.  Two epilogues: the
//             gated activation act(gate) * up from weight rows n and F + n, stored in the compute type;
//             or float32 rows.  float32 accumulation in K order: a row's result does not depend on the
//             rows it shares a tile with.
// The consumer adds a token's `top` result rows in the order of its choices (hyper.cu, or moe_combine,
// which can multiply each by its choice's weight for designs that scale the expert's OUTPUT).
#include "common.cuh"

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_MAX_TOP = 8;

// ------------------------------------------------------------------ routing
// logits [T][ldz] float32.  expert_of, rank_of [T*top] int32, weight_of [T*top] float32, counts [n_exp] (zero on entry).
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int ldz, int n_tokens, int n_exp, int top, int softmax_scores, int renormalize,
                 int* __restrict__ expert_of, int* __restrict__ rank_of, float* __restrict__ weight_of, int* __restrict__ counts) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n_tokens) return;
  constexpr int PER = MOE_MAX_EXPERTS / 32;
  float s[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    s[i] = e < n_exp ? logits[(size_t)t * ldz + e] : -INFINITY;
    mx = fmaxf(mx, s[i]);
  }
  if (softmax_scores) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      s[i] = lane + 32 * i < n_exp ? expf(s[i] - mx) : -INFINITY;
      if (lane + 32 * i < n_exp) sum += s[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i < n_exp) s[i] /= sum;
  } else {
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i < n_exp) s[i] = 1.f / (1.f + expf(-s[i]));
  }
  float chosen_w[MOE_MAX_TOP];
  int chosen_e[MOE_MAX_TOP];
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (e < n_exp && s[i] > best) {       // (ascending e within a lane: the lower index wins a tie)
        best = s[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    chosen_w[j] = best;
    chosen_e[j] = best_e;
    total += best;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i == best_e) s[i] = -INFINITY;
  }
  if (lane == 0) {
    for (int j = 0; j < top; ++j) {
      const int e = chosen_e[j] < n_exp ? chosen_e[j] : 0;      // (all scores NaN: expert 0 with a NaN weight)
      expert_of[(size_t)t * top + j] = e;
      weight_of[(size_t)t * top + j] = renormalize ? chosen_w[j] / total : chosen_w[j];
      rank_of[(size_t)t * top + j] = atomicAdd(&counts[e], 1);
    }
  }
}

// x [T][ldx] -> xg [row][E] at the pair's place; row_of[pair] = row.  scale_input: the row is multiplied by the weight.
template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const T* __restrict__ x, int ldx, int E, int n_exp, int top, const int* __restrict__ expert_of,
                  const int* __restrict__ rank_of, const float* __restrict__ weight_of, const int* __restrict__ counts,
                  int scale_input, T* __restrict__ xg, int* __restrict__ row_of) {
  __shared__ int sm_row;
  const int pair = blockIdx.x;
  if (threadIdx.x == 0) {
    const int e = expert_of[pair];
    int first = 0;
    for (int i = 0; i < e; ++i) first += counts[i];
    sm_row = first + rank_of[pair];
    row_of[pair] = sm_row;
  }
  __syncthreads();
  const int row = sm_row;
  const float w = scale_input ? weight_of[pair] : 1.f;
  const T* src = x + (size_t)(pair / top) * ldx;
  T* dst = xg + (size_t)row * E;
  for (int i = threadIdx.x; i < E; i += 128) dst[i] = from_f32<T>(to_f32<T>(src[i]) * w);
}

// ------------------------------------------------------------------ the grouped product
__device__ __forceinline__ float moe_act(float z, int act) {
  if (act == 1) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.f + expf(-z));
}

// A [rows][lda]; W [n_exp][w_rows][K]; counts [n_exp].  glu: out[row][n] = act(C[row][n]) * C[row][F + n] in T (N = F);
// else out[row][n] = C[row][n] in float32.  BM x BN outputs per CTA, K in steps of BK
// through shared memory, TM x TN outputs a thread.
template <typename T, int BM>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int w_rows, int K, int N, int n_exp,
                const int* __restrict__ counts, int glu, int act, void* __restrict__ out, int ldo) {
  constexpr int BN = 64, BK = 16;
  constexpr int TM = BM / 16, TN = 4;             // 16 x 16 threads
  __shared__ float sa[BK][BM + 1];
  __shared__ float sb[2][BK][BN + 1];
  __shared__ int tile_e, tile_row0, tile_rows;
  if (threadIdx.x == 0) {
    int left = blockIdx.x, first = 0, e = 0, rows = 0, row0 = 0;
    for (; e < n_exp; ++e) {
      const int c = counts[e];
      const int tiles = (c + BM - 1) / BM;
      if (left < tiles) {
        row0 = first + left * BM;
        rows = min(BM, first + c - row0);
        break;
      }
      left -= tiles;
      first += c;
    }
    tile_e = e;
    tile_row0 = row0;
    tile_rows = rows;          // 0: past the last tile
  }
  __syncthreads();
  const int rows = tile_rows;
  if (rows == 0) return;
  const int row0 = tile_row0;
  const int n0 = blockIdx.y * BN;
  const T* We = W + (size_t)tile_e * w_rows * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[2][TM][TN];
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[g][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
      const int m = idx / BK, k = idx % BK;
      sa[k][m] = (m < rows && k0 + k < K) ? to_f32<T>(A[(size_t)(row0 + m) * lda + k0 + k]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
      const int n = idx / BK, k = idx % BK;
      const bool in = n0 + n < N && k0 + k < K;
      sb[0][k][n] = in ? to_f32<T>(We[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
      if (glu) sb[1][k][n] = in ? to_f32<T>(We[(size_t)(N + n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b0[TN], b1[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = sa[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        b0[j] = sb[0][k][tx * TN + j];
        b1[j] = glu ? sb[1][k][tx * TN + j] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[0][i][j] = fmaf(a[i], b0[j], acc[0][i][j]);
          if (glu) acc[1][i][j] = fmaf(a[i], b1[j], acc[1][i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = ty * TM + i;
    if (m >= rows) continue;
    const size_t row = (size_t)(row0 + m);
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      if (glu) reinterpret_cast<T*>(out)[row * ldo + n] = from_f32<T>(moe_act(acc[0][i][j], act) * acc[1][i][j]);
      else reinterpret_cast<float*>(out)[row * ldo + n] = acc[0][i][j];
    }
  }
}

// y[t][:] = sum over the token's choices, in their order, of rows[row_of[t*top + j]][:] (float32), each times
// weight_of[t*top + j] when that is given; for consumers that want a plain buffer.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ rows, int ld, const int* __restrict__ row_of, const float* __restrict__ weight_of,
                   int top, int E, float* __restrict__ y) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < E; i += 256) {
    float s = 0.f;
    for (int j = 0; j < top; ++j) {
      const float v = rows[(size_t)row_of[(size_t)t * top + j] * ld + i];
      s += weight_of != nullptr ? v * weight_of[(size_t)t * top + j] : v;
    }
    y[(size_t)t * E + i] = s;
  }
}

FERRUM_API int ferrum_moe_max_experts() { return MOE_MAX_EXPERTS; }
FERRUM_API int ferrum_moe_max_top() { return MOE_MAX_TOP; }

// Routing and gathering of one step.  counts: n_exp ints (zeroed here).
FERRUM_API int ferrum_moe_route(const float* logits, int ldz, int n_tokens, int n_exp, int top, int softmax_scores,
                                int renormalize, const void* x, int ldx, int E, int dtype, int scale_input, int* expert_of,
                                int* rank_of, float* weight_of, int* counts, void* xg, int* row_of, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_exp > 0 && n_exp <= MOE_MAX_EXPERTS && top > 0 && top <= MOE_MAX_TOP && top <= n_exp,
                   "moe_route: %d experts, %d per token are outside the kernel's limits (%d, %d)", n_exp, top, MOE_MAX_EXPERTS, MOE_MAX_TOP);
  FERRUM_CHECK_ARG(ldz >= n_exp && ldx >= E && E > 0, "moe_route: rows are shorter than their contents");
  if (n_tokens == 0) return 0;
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * n_exp, stream);
  FERRUM_CHECK_ARG(e == cudaSuccess, "moe_route: cannot clear the counters: %s", cudaGetErrorString(e));
  moe_route_kernel<<<(n_tokens + 3) / 4, 128, 0, stream>>>(logits, ldz, n_tokens, n_exp, top, softmax_scores, renormalize,
                                                           expert_of, rank_of, weight_of, counts);
  FERRUM_CHECK_LAUNCH("moe_route");
  FERRUM_DISPATCH_DTYPE(dtype, T, (moe_gather_kernel<T><<<n_tokens * top, 128, 0, stream>>>(
      (const T*)x, ldx, E, n_exp, top, expert_of, rank_of, weight_of, counts, scale_input, (T*)xg, row_of)));
  FERRUM_CHECK_LAUNCH("moe_gather");
  return 0;
}

// n_rows: the sorted rows (tokens x top).  glu != 0: W holds gate rows 0..N-1 and up rows N..2N-1 per expert
// (w_rows = 2N), out is [n_rows][ldo] in the compute type; else out is float32.
FERRUM_API int ferrum_moe_gemm(const void* A, int lda, const void* W, int w_rows, int K, int N, int n_exp, const int* counts,
                               int n_rows, int dtype, int glu, int act, void* out, int ldo, cudaStream_t stream) {
  FERRUM_CHECK_ARG(K > 0 && N > 0 && lda >= K && ldo >= N && w_rows >= (glu ? 2 * N : N), "moe_gemm: shapes do not agree");
  FERRUM_CHECK_ARG(n_exp > 0 && n_exp <= MOE_MAX_EXPERTS, "moe_gemm: bad number of experts %d", n_exp);
  if (n_rows == 0) return 0;
  const int ntile = (N + 63) / 64;
  FERRUM_CHECK_ARG(ntile <= 65535, "moe_gemm: too many output features");
  if (n_rows <= 256) {
    const dim3 grid((n_rows + 15) / 16 + n_exp, ntile);
    FERRUM_DISPATCH_DTYPE(dtype, T, (moe_gemm_kernel<T, 16><<<grid, 256, 0, stream>>>(
        (const T*)A, lda, (const T*)W, w_rows, K, N, n_exp, counts, glu, act, out, ldo)));
  } else {
    const dim3 grid((n_rows + 63) / 64 + n_exp, ntile);
    FERRUM_DISPATCH_DTYPE(dtype, T, (moe_gemm_kernel<T, 64><<<grid, 256, 0, stream>>>(
        (const T*)A, lda, (const T*)W, w_rows, K, N, n_exp, counts, glu, act, out, ldo)));
  }
  FERRUM_CHECK_LAUNCH("moe_gemm");
  return 0;
}

FERRUM_API int ferrum_moe_combine(const float* rows, int ld, const int* row_of, const float* weight_of, int top, int n_tokens,
                                  int E, float* y, cudaStream_t stream) {
  FERRUM_CHECK_ARG(top > 0 && E > 0 && ld >= E, "moe_combine: bad sizes");
  if (n_tokens == 0) return 0;
  moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(rows, ld, row_of, weight_of, top, E, y);
  FERRUM_CHECK_LAUNCH("moe_combine");
  return 0;
}
