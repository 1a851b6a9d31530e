// A routed feed-forward: every token goes through `top` of `n_exp` small gated feed-forwards.
//
// moe_route   one warp per token: scores from the router's float32 logits (sigmoid of each, or a
//             softmax over all), the `top` largest (ties: the lower index), optionally renormalised to
//             sum 1; the token takes a place in each chosen expert's group (an atomic counter per expert).
//             A correction vector may be added to the scores for the choice alone (the weights stay the
//             plain scores), the weights may be multiplied by a constant, and the last router outputs may
//             be identity experts (numbers n_real .. n_exp - 1: no matrices, no rows in the sorted buffer;
//             the consumer adds weight * the token's own input for them).
// moe_gather  one block per (token, choice): the token's input row, multiplied by the choice's weight
//             where the design scales the expert's INPUT, goes to its place in a buffer sorted by
//             expert (row = first row of the expert's group + the place taken above).
// moe_gemm    C[row][n] = sum_k A[row][k] W[expert of row][n][k] over the sorted rows: a CTA owns a tile
//             of rows of ONE expert (it finds expert and rows from the counters, so nothing about the
//             routing passes through the host) and a tile of output features.  Two epilogues: the
//             gated activation act(gate) * up from weight rows n and F + n, stored in the compute type;
//             or float32 rows.  float32 accumulation in an order that depends on K and on the kernel
//             only: a row's result does not depend on the rows it shares a tile with.  Three kernels:
//             tiles on the CUDA cores (float32, and 16-bit rows that are no 16-byte multiples), a
//             warp per feature when an expert has a few rows (the same types, decoding), and tiles on
//             the tensor cores for 16-bit types.  Which one runs depends on the step's row count, so a
//             token's result in a small and in a large batch agrees to rounding, not bitwise.
// The consumer adds a token's `top` result rows in the order of its choices (hyper.cu, or moe_combine,
// which can multiply each by its choice's weight for designs that scale the expert's OUTPUT).
#include "common.cuh"

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_MAX_TOP = 8;

// ------------------------------------------------------------------ routing
// logits [T][ldz] float32.  expert_of, rank_of [T*top] int32, weight_of [T*top] float32, counts [n_exp] (zero on entry).
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int ldz, int n_tokens, int n_exp, int top, int softmax_scores, int renormalize,
                 int* __restrict__ expert_of, int* __restrict__ rank_of, float* __restrict__ weight_of, int* __restrict__ counts,
                 const float* __restrict__ correction, float weight_scale, int n_real) {
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
  float pick[PER];                          // what the choice goes by: the score, plus the correction when there is one
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    pick[i] = (correction != nullptr && e < n_exp) ? s[i] + correction[e] : s[i];
  }
  float chosen_w[MOE_MAX_TOP];
  int chosen_e[MOE_MAX_TOP];
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY, best_s = 0.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (e < n_exp && pick[i] > best) {    // (ascending e within a lane: the lower index wins a tie)
        best = pick[i];
        best_s = s[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_s = os;
        best_e = oe;
      }
    }
    chosen_w[j] = best_s;
    chosen_e[j] = best_e;
    total += best_s;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i == best_e) pick[i] = -INFINITY;
  }
  if (lane == 0) {
    for (int j = 0; j < top; ++j) {
      const int e = chosen_e[j] < n_exp ? chosen_e[j] : 0;      // (all scores NaN: expert 0 with a NaN weight)
      expert_of[(size_t)t * top + j] = e;
      weight_of[(size_t)t * top + j] = (renormalize ? chosen_w[j] / total : chosen_w[j]) * weight_scale;
      rank_of[(size_t)t * top + j] = e < n_real ? atomicAdd(&counts[e], 1) : 0;      // (an identity expert keeps no rows)
    }
  }
}

// x [T][ldx] -> xg [row][E] at the pair's place; row_of[pair] = row (-1 for an identity expert, which has no row).
// scale_input: the row is multiplied by the weight.
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
    for (int i = 0; i < e && i < n_exp; ++i) first += counts[i];
    sm_row = e < n_exp ? first + rank_of[pair] : -1;
    row_of[pair] = sm_row;
  }
  __syncthreads();
  const int row = sm_row;
  if (row < 0) return;
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
// What the gated epilogue stores for a gate value and an up value (act 2: the clamped unit of common.cuh).
__device__ __forceinline__ float moe_glu(float g, float u, int act, float limit) {
  if (act == GLU_SWISH_CLAMP) return glu_swish_clamp(g, u, limit);
  return moe_act(g, act) * u;
}

// A [rows][lda]; W [n_exp][w_rows][K]; counts [n_exp].  GLU: out[row][n] = act(C[row][n]) * C[row][F + n] in T (N = F);
// else out[row][n] = C[row][n] in float32.  BM x BN outputs per CTA, K in steps of BK
// through shared memory, TM x TN outputs a thread.
template <typename T, int BM, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int w_rows, int K, int N, int n_exp,
                const int* __restrict__ counts, int act, float limit, void* __restrict__ out, int ldo) {
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
      if (GLU) sb[1][k][n] = in ? to_f32<T>(We[(size_t)(N + n0 + n) * K + k0 + k]) : 0.f;
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
        b1[j] = GLU ? sb[1][k][tx * TN + j] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[0][i][j] = fmaf(a[i], b0[j], acc[0][i][j]);
          if (GLU) acc[1][i][j] = fmaf(a[i], b1[j], acc[1][i][j]);
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
      if (GLU) reinterpret_cast<T*>(out)[row * ldo + n] = from_f32<T>(moe_glu(acc[0][i][j], acc[1][i][j], act, limit));
      else reinterpret_cast<float*>(out)[row * ldo + n] = acc[0][i][j];
    }
  }
}

// ------------------------------------------------------------------ the grouped product for a few rows an expert (CUDA cores)
// Decoding: an expert sees a handful of rows and the product is a stream of its weights.  A CTA owns up to 16 sorted
// rows of one expert and 8 output features, one per warp (in the gated form the gate row and its up row); a lane walks
// its elements of K (four consecutive ones of every 128 when rows are float32 on 16-byte boundaries, else every 32nd),
// keeps one float32 sum per row, and the 32 lanes meet in a fixed shuffle tree.  The order of a row's sum is a function
// of K alone.  The rows' elements are read through L1 by all eight warps.
constexpr int MS_ROWS = 16, MS_WARPS = 8;

template <typename T, bool GLU, bool VEC>
__global__ void __launch_bounds__(MS_WARPS * 32)
moe_gemm_skinny_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int w_rows, int K, int N, int n_exp,
                       const int* __restrict__ counts, int act, float limit, void* __restrict__ out, int ldo) {
  __shared__ int tile_e, tile_row0, tile_rows;
  if (threadIdx.x == 0) {
    int left = blockIdx.x, first = 0, e = 0, rows = 0, row0 = 0;
    for (; e < n_exp; ++e) {
      const int c = counts[e];
      const int tiles = (c + MS_ROWS - 1) / MS_ROWS;
      if (left < tiles) {
        row0 = first + left * MS_ROWS;
        rows = min(MS_ROWS, first + c - row0);
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
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.y * MS_WARPS + warp;
  if (rows == 0 || n >= N) return;
  const int row0 = tile_row0;
  const T* w0 = W + ((size_t)tile_e * w_rows + n) * K;
  const T* w1 = w0 + (size_t)N * K;              // the up row (gated form)
  const T* Ar = A + (size_t)row0 * lda;
  float acc0[MS_ROWS], acc1[MS_ROWS];
#pragma unroll
  for (int m = 0; m < MS_ROWS; ++m) acc0[m] = acc1[m] = 0.f;
  if (VEC) {
#pragma unroll 2
    for (int k = lane * 4; k < K; k += 128) {
      const float4 g = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w0) + k);
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
      if (GLU) u = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w1) + k);
#pragma unroll
      for (int m = 0; m < MS_ROWS; ++m) {
        if (m < rows) {
          const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(Ar) + (size_t)m * lda + k);
          acc0[m] = fmaf(a.x, g.x, fmaf(a.y, g.y, fmaf(a.z, g.z, fmaf(a.w, g.w, acc0[m]))));
          if (GLU) acc1[m] = fmaf(a.x, u.x, fmaf(a.y, u.y, fmaf(a.z, u.z, fmaf(a.w, u.w, acc1[m]))));
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float g = to_f32<T>(w0[k]);
      const float u = GLU ? to_f32<T>(w1[k]) : 0.f;
#pragma unroll
      for (int m = 0; m < MS_ROWS; ++m) {
        if (m < rows) {
          const float a = to_f32<T>(Ar[(size_t)m * lda + k]);
          acc0[m] = fmaf(a, g, acc0[m]);
          if (GLU) acc1[m] = fmaf(a, u, acc1[m]);
        }
      }
    }
  }
  float r0 = 0.f, r1 = 0.f;
#pragma unroll
  for (int m = 0; m < MS_ROWS; ++m) {
    if (m < rows) {
      const float s0 = warp_sum(acc0[m]);
      const float s1 = GLU ? warp_sum(acc1[m]) : 0.f;
      if (lane == m) {
        r0 = s0;
        r1 = s1;
      }
    }
  }
  if (lane < rows) {
    const size_t o = (size_t)(row0 + lane) * ldo + n;
    if (GLU) reinterpret_cast<T*>(out)[o] = from_f32<T>(moe_glu(r0, r1, act, limit));
    else reinterpret_cast<float*>(out)[o] = r0;
  }
}

// ------------------------------------------------------------------ the grouped product on the tensor cores (16-bit types)
// The same tiles of rows of one expert, on mma.sync m16n8k16 with float32 accumulators.  A CTA owns BM sorted rows and
// BN output features (in the gated form BN gate rows and the BN up rows that belong to them, two accumulators that the
// epilogue combines).  K runs in blocks of 64 elements (128 bytes a row) through a ring of cp.async stages; rows are
// stored with their 16-byte chunks XOR-swizzled by the row so that ldmatrix reads without bank conflicts.  Rows past the
// group, features past N and chunks past K are filled with zeros by the copies and masked in the stores, so a row's
// result is the K-ordered sum of its own products whatever shares its tile.  Needs K and lda multiples of 8 elements
// and 16-byte aligned operands (the launcher checks; everything else takes the CUDA-core kernel above).
namespace moe_mma {

constexpr int BK = 64;

__device__ __forceinline__ void cp16(void* smem, const void* gmem, int src_bytes) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
template <typename T>
__device__ __forceinline__ void mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1);
template <>
__device__ __forceinline__ void mma<__half>(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma<__nv_bfloat16>(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// element (row, col) of a [rows][64] 16-bit tile whose 16-byte chunks are XOR-swizzled by the row
template <typename T>
__device__ __forceinline__ T* at(T* base, int row, int col) {
  return base + row * BK + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7));
}

template <int BM, int BN, int STAGES, bool GLU>
constexpr int smem_bytes() { return STAGES * (BM + (GLU ? 2 : 1) * BN) * BK * 2; }

template <typename T, int BM, int BN, int WM, int WN, int STAGES, bool GLU>
__global__ void __launch_bounds__(WM * WN * 32)
moe_gemm_mma_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int w_rows, int K, int N, int n_exp,
                    const int* __restrict__ counts, int act, float limit, void* __restrict__ out, int ldo) {
  constexpr int NT = WM * WN * 32;
  constexpr int NB = GLU ? 2 : 1;
  constexpr int MI = BM / WM / 16, NI = BN / WN / 8;
  static_assert(MI >= 1 && NI >= 2 && NI % 2 == 0, "a warp needs 16 rows and 16 features at least");
  constexpr int STAGE = (BM + NB * BN) * BK;      // elements
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* smem = reinterpret_cast<T*>(smem_raw);
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
  const T* Ar = A + (size_t)row0 * lda;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp / WN, wn = warp % WN;
  const int nk = (K + BK - 1) / BK;

  // Every thread copies the same 16-byte chunk column (c) of rows lr, lr + RS, lr + 2 RS, ... of both operands: the
  // rows' pointers, their places in a stage and whether they exist are worked out once; a k-block costs an add and
  // the copy per chunk.
  constexpr int RS = NT / 8;                        // rows between two chunks of a thread (a multiple of 8)
  constexpr int AI = BM / RS, BI = NB * BN / RS;    // chunks a thread copies per k-block
  static_assert(BM % RS == 0 && BN % RS == 0 && RS % 8 == 0, "the copy plan needs whole rounds of the threads");
  const int lr = threadIdx.x >> 3, c = threadIdx.x & 7, kc = c * 8;
  const unsigned smem0 = (unsigned)__cvta_generic_to_shared(smem);
  const unsigned dst0 = (unsigned)((lr * BK + ((c ^ (lr & 7)) << 3)) * 2);      // bytes; row lr + i RS lies i RS rows on
  const T* pa[AI];
  const T* pb[BI];
  unsigned ok_a = 0, ok_b = 0;
#pragma unroll
  for (int i = 0; i < AI; ++i) {
    const int m = lr + i * RS;
    if (m < rows) ok_a |= 1u << i;
    pa[i] = m < rows ? Ar + (size_t)m * lda + kc : A;
  }
#pragma unroll
  for (int i = 0; i < BI; ++i) {
    const int n = lr + i * RS;                      // 0..BN-1 gate (or plain) rows, then the up rows
    const int f = n0 + (n & (BN - 1));
    if (f < N) ok_b |= 1u << i;
    pb[i] = f < N ? We + (size_t)(n < BN ? f : N + f) * K + kc : W;
  }
  auto load = [&](int kb, int stage) {
    const int k0 = kb * BK;
    const bool kin = k0 + kc < K;
    const unsigned sa = smem0 + (unsigned)(stage * STAGE * 2) + dst0;
#pragma unroll
    for (int i = 0; i < AI; ++i) {
      const bool in = kin && ((ok_a >> i) & 1u);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sa + i * RS * BK * 2), "l"(in ? pa[i] + k0 : pa[i]), "r"(in ? 16 : 0) : "memory");
    }
#pragma unroll
    for (int i = 0; i < BI; ++i) {
      const bool in = kin && ((ok_b >> i) & 1u);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sa + (BM + i * RS) * BK * 2), "l"(in ? pb[i] + k0 : pb[i]), "r"(in ? 16 : 0) : "memory");
    }
  };
  // ldmatrix addresses: a lane's row is fixed, and its chunk in k-step kk is (kk / 8 + hi) ^ (row & 7) = (kk / 8) ^ t with
  // t fixed (kk / 8 is even, hi is 0 or 1), so the byte offset within a stage is a fixed one XOR 2 kk.
  const int row_a = wm * (MI * 16) + (lane & 15);
  const unsigned off_a = (unsigned)(row_a * BK * 2 + ((((lane >> 4) ^ (row_a & 7)) & 7) << 4));
  const int row_b = wn * (NI * 8) + (lane & 7) + ((lane >> 4) << 3);
  const unsigned off_b = (unsigned)((BM + row_b) * BK * 2 + (((((lane >> 3) & 1) ^ (row_b & 7)) & 7) << 4));

  float acc[NB][MI][NI][4];
#pragma unroll
  for (int g = 0; g < NB; ++g)
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[g][i][j][r] = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) load(s, s);
    commit();
  }
  for (int kb = 0; kb < nk; ++kb) {
    wait<STAGES - 2>();
    __syncthreads();          // block kb has landed for everyone, and everyone is done with the stage refilled next
    if (kb + STAGES - 1 < nk) load(kb + STAGES - 1, (kb + STAGES - 1) % STAGES);
    commit();
    const unsigned st = smem0 + (unsigned)((kb % STAGES) * STAGE * 2);
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      unsigned a[MI][4];
#pragma unroll
      for (int i = 0; i < MI; ++i) {
        const unsigned ad = st + (off_a ^ (unsigned)(kk * 2)) + i * 16 * BK * 2;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a[i][0]), "=r"(a[i][1]), "=r"(a[i][2]), "=r"(a[i][3]) : "r"(ad));
      }
#pragma unroll
      for (int g = 0; g < NB; ++g)
#pragma unroll
        for (int j = 0; j < NI; j += 2) {
          unsigned b[4];
          const unsigned ad = st + (off_b ^ (unsigned)(kk * 2)) + (g * BN + j * 8) * BK * 2;
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(ad));
#pragma unroll
          for (int i = 0; i < MI; ++i) {
            mma<T>(acc[g][i][j], a[i], b[0], b[1]);
            mma<T>(acc[g][i][j + 1], a[i], b[2], b[3]);
          }
        }
    }
  }
  wait<0>();
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = wm * (MI * 16) + i * 16 + (lane >> 2) + h * 8;
      if (m >= rows) continue;
      const size_t o = (size_t)(row0 + m) * ldo;
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn * (NI * 8) + j * 8 + (lane & 3) * 2 + c;
          if (n >= N) continue;
          if (GLU) reinterpret_cast<T*>(out)[o + n] = from_f32<T>(moe_glu(acc[0][i][j][h * 2 + c], acc[NB - 1][i][j][h * 2 + c], act, limit));
          else reinterpret_cast<float*>(out)[o + n] = acc[0][i][j][h * 2 + c];
        }
    }
}

template <typename T, int BM, int BN, int WM, int WN, int STAGES, bool GLU>
int launch(const T* A, int lda, const T* W, int w_rows, int K, int N, int n_exp, const int* counts, int n_rows, int act, float limit, void* out,
           int ldo, cudaStream_t stream) {
  constexpr int smem = smem_bytes<BM, BN, STAGES, GLU>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_mma_kernel<T, BM, BN, WM, WN, STAGES, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    FERRUM_CHECK_ARG(e == cudaSuccess, "moe_gemm: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const dim3 grid((n_rows + BM - 1) / BM + n_exp, (N + BN - 1) / BN);
  moe_gemm_mma_kernel<T, BM, BN, WM, WN, STAGES, GLU><<<grid, WM * WN * 32, smem, stream>>>(A, lda, W, w_rows, K, N, n_exp, counts, act, limit, out, ldo);
  FERRUM_CHECK_LAUNCH("moe_gemm (tensor cores)");
  return 0;
}

template <typename T>
int run(const void* A, int lda, const void* W, int w_rows, int K, int N, int n_exp, const int* counts, int n_rows, int glu, int act, float limit,
        void* out, int ldo, cudaStream_t stream) {
  const T* a = (const T*)A;
  const T* w = (const T*)W;
  const bool few = n_rows <= 32 * n_exp;        // about 32 rows an expert or fewer: tiles of 16 rows that stream the weights
  if (few) {
    if (glu) return launch<T, 16, 64, 1, 4, 4, true>(a, lda, w, w_rows, K, N, n_exp, counts, n_rows, act, limit, out, ldo, stream);
    return launch<T, 16, 64, 1, 4, 4, false>(a, lda, w, w_rows, K, N, n_exp, counts, n_rows, act, limit, out, ldo, stream);
  }
  if (glu) return launch<T, 128, 64, 4, 2, 3, true>(a, lda, w, w_rows, K, N, n_exp, counts, n_rows, act, limit, out, ldo, stream);
  return launch<T, 128, 128, 4, 2, 3, false>(a, lda, w, w_rows, K, N, n_exp, counts, n_rows, act, limit, out, ldo, stream);
}

}  // namespace moe_mma

// y[t][:] = sum over the token's choices, in their order, of rows[row_of[t*top + j]][:] (float32), each times
// weight_of[t*top + j] when that is given; for consumers that want a plain buffer.  A choice without a row
// (row_of < 0: an identity expert) stands for the token's own input row x[t][:]; `add` (float32 rows, may be null:
// a unit that every token runs through) joins the sum last.
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ rows, int ld, const int* __restrict__ row_of, const float* __restrict__ weight_of,
                   int top, int E, float* __restrict__ y, const T* __restrict__ x, int ldx, const float* __restrict__ add,
                   int ld_add) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < E; i += 256) {
    float s = 0.f;
    for (int j = 0; j < top; ++j) {
      const int r = row_of[(size_t)t * top + j];
      const float v = r >= 0 ? rows[(size_t)r * ld + i] : (x != nullptr ? to_f32<T>(x[(size_t)t * ldx + i]) : 0.f);
      s += weight_of != nullptr ? v * weight_of[(size_t)t * top + j] : v;
    }
    if (add != nullptr) s += add[(size_t)t * ld_add + i];
    y[(size_t)t * E + i] = s;
  }
}

static bool g_moe_cuda_cores = false;
// Tests and measurements: 1 sends 16-bit products to the CUDA-core kernel too.
FERRUM_API int ferrum_moe_cuda_cores(int on) {
  g_moe_cuda_cores = on != 0;
  return 0;
}

FERRUM_API int ferrum_moe_max_experts() { return MOE_MAX_EXPERTS; }
FERRUM_API int ferrum_moe_max_top() { return MOE_MAX_TOP; }

// Routing and gathering of one step.  counts: n_exp ints (zeroed here).
FERRUM_API int ferrum_moe_route(const float* logits, int ldz, int n_tokens, int n_exp, int top, int softmax_scores,
                                int renormalize, const void* x, int ldx, int E, int dtype, int scale_input, int* expert_of,
                                int* rank_of, float* weight_of, int* counts, void* xg, int* row_of, const float* correction,
                                float weight_scale, int n_identity, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_exp > 0 && n_exp <= MOE_MAX_EXPERTS && top > 0 && top <= MOE_MAX_TOP && top <= n_exp,
                   "moe_route: %d experts, %d per token are outside the kernel's limits (%d, %d)", n_exp, top, MOE_MAX_EXPERTS, MOE_MAX_TOP);
  FERRUM_CHECK_ARG(n_identity >= 0 && n_identity < n_exp, "moe_route: %d identity experts among %d router outputs", n_identity, n_exp);
  FERRUM_CHECK_ARG(n_identity == 0 || !scale_input, "moe_route: identity experts go with weights on the experts' results");
  const int n_real = n_exp - n_identity;
  FERRUM_CHECK_ARG(ldz >= n_exp && ldx >= E && E > 0, "moe_route: rows are shorter than their contents");
  if (n_tokens == 0) return 0;
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * n_real, stream);
  FERRUM_CHECK_ARG(e == cudaSuccess, "moe_route: cannot clear the counters: %s", cudaGetErrorString(e));
  moe_route_kernel<<<(n_tokens + 3) / 4, 128, 0, stream>>>(logits, ldz, n_tokens, n_exp, top, softmax_scores, renormalize,
                                                           expert_of, rank_of, weight_of, counts, correction, weight_scale, n_real);
  FERRUM_CHECK_LAUNCH("moe_route");
  FERRUM_DISPATCH_DTYPE(dtype, T, (moe_gather_kernel<T><<<n_tokens * top, 128, 0, stream>>>(
      (const T*)x, ldx, E, n_real, top, expert_of, rank_of, weight_of, counts, scale_input, (T*)xg, row_of)));
  FERRUM_CHECK_LAUNCH("moe_gather");
  return 0;
}

// n_rows: the sorted rows (tokens x top).  glu != 0: W holds gate rows 0..N-1 and up rows N..2N-1 per expert
// (w_rows = 2N), out is [n_rows][ldo] in the compute type; else out is float32.
FERRUM_API int ferrum_moe_gemm(const void* A, int lda, const void* W, int w_rows, int K, int N, int n_exp, const int* counts,
                               int n_rows, int dtype, int glu, int act, float limit, void* out, int ldo, cudaStream_t stream) {
  FERRUM_CHECK_ARG(K > 0 && N > 0 && lda >= K && ldo >= N && w_rows >= (glu ? 2 * N : N), "moe_gemm: shapes do not agree");
  FERRUM_CHECK_ARG(n_exp > 0 && n_exp <= MOE_MAX_EXPERTS, "moe_gemm: bad number of experts %d", n_exp);
  if (n_rows == 0) return 0;
  const int ntile = (N + 63) / 64;
  FERRUM_CHECK_ARG(ntile <= 65535, "moe_gemm: too many output features");
  if (dtype != FERRUM_F32 && !g_moe_cuda_cores && K % 8 == 0 && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(W) & 15) == 0) {
    if (dtype == FERRUM_BF16)
      return moe_mma::run<__nv_bfloat16>(A, lda, W, w_rows, K, N, n_exp, counts, n_rows, glu, act, limit, out, ldo, stream);
    if (dtype == FERRUM_F16) return moe_mma::run<__half>(A, lda, W, w_rows, K, N, n_exp, counts, n_rows, glu, act, limit, out, ldo, stream);
  }
#define MT_LAUNCH(BM)                                                                                                  \
  do {                                                                                                                 \
    if (glu) FERRUM_DISPATCH_DTYPE(dtype, T, (moe_gemm_kernel<T, BM, true><<<grid, 256, 0, stream>>>(                   \
        (const T*)A, lda, (const T*)W, w_rows, K, N, n_exp, counts, act, limit, out, ldo)));                                  \
    else FERRUM_DISPATCH_DTYPE(dtype, T, (moe_gemm_kernel<T, BM, false><<<grid, 256, 0, stream>>>(                      \
        (const T*)A, lda, (const T*)W, w_rows, K, N, n_exp, counts, act, limit, out, ldo)));                                  \
  } while (0)
  if (n_rows <= 32 * n_exp) {         // about 32 rows an expert or fewer: a stream of the weights
    const dim3 grid((n_rows + MS_ROWS - 1) / MS_ROWS + n_exp, (N + MS_WARPS - 1) / MS_WARPS);
    FERRUM_CHECK_ARG(grid.y <= 65535, "moe_gemm: too many output features");
    const bool vec = dtype == FERRUM_F32 && K % 4 == 0 && lda % 4 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(W) & 15) == 0;
#define MS_LAUNCH(T, G, V)                                                                                                   \
  moe_gemm_skinny_kernel<T, G, V><<<grid, MS_WARPS * 32, 0, stream>>>((const T*)A, lda, (const T*)W, w_rows, K, N, n_exp, counts, \
                                                                      act, limit, out, ldo)
    if (vec) {
      if (glu) MS_LAUNCH(float, true, true);
      else MS_LAUNCH(float, false, true);
    } else if (glu) {
      FERRUM_DISPATCH_DTYPE(dtype, T, MS_LAUNCH(T, true, false));
    } else {
      FERRUM_DISPATCH_DTYPE(dtype, T, MS_LAUNCH(T, false, false));
    }
#undef MS_LAUNCH
  } else if (n_rows <= 256) {
    const dim3 grid((n_rows + 15) / 16 + n_exp, ntile);
    MT_LAUNCH(16);
  } else if (n_rows <= 96 * n_exp || !glu) {
    const dim3 grid((n_rows + 63) / 64 + n_exp, ntile);
    MT_LAUNCH(64);
  } else {                            // the gated form with about a hundred rows an expert or more: 2 x 8 x 4 outputs a thread
    const dim3 grid((n_rows + 127) / 128 + n_exp, ntile);
    MT_LAUNCH(128);
  }
#undef MT_LAUNCH
  FERRUM_CHECK_LAUNCH("moe_gemm");
  return 0;
}

FERRUM_API int ferrum_moe_combine(const float* rows, int ld, const int* row_of, const float* weight_of, int top, int n_tokens,
                                  int E, float* y, const void* x, int ldx, int x_dtype, const float* add, int ld_add,
                                  cudaStream_t stream) {
  FERRUM_CHECK_ARG(top > 0 && E > 0 && ld >= E, "moe_combine: bad sizes");
  FERRUM_CHECK_ARG((x == nullptr || ldx >= E) && (add == nullptr || ld_add >= E), "moe_combine: a row is shorter than the width");
  if (n_tokens == 0) return 0;
  FERRUM_DISPATCH_DTYPE(x_dtype, T, (moe_combine_kernel<T><<<n_tokens, 256, 0, stream>>>(rows, ld, row_of, weight_of, top, E, y,
                                                                                       (const T*)x, ldx, add, ld_add)));
  FERRUM_CHECK_LAUNCH("moe_combine");
  return 0;
}
