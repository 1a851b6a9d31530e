// Kernels of the parallel gated block: both sublayers read norms of the same residual row, the
// mixer's input is mixed with the previous token's (token shift), and each sublayer's result is
// scaled by a learned sigmoid gate before both are added to the residual stream.
//
//   n = x / sqrt(mean_g(x^2) + eps)        per group g of E / groups consecutive elements
//   a = n * w1,  b = n * w2                (one normalisation, two weight vectors)
//   m = a + (a_prev - a) * s               a_prev: the a of the request's previous token
//   x += y1 * sigmoid(g1 + c1) + (y2 + c2) * sigmoid(g2 + c3)
//
// Everything here is float32 arithmetic on the float32 residual stream; only a, m and b leave in
// the compute dtype, as inputs of the products that follow.  The previous token's a is found in
// the batch (the row before, recomputed from x with the same reduction tree, so that the value is
// bit-equal to what a step that ended on that token left behind) or, for the first token of a
// portion, in the request's state row.  A portion's last a goes to a staging row first and is
// copied into the state by the block's last kernel: the state is read and written by different
// launches, never by blocks of one grid.
#include "common.cuh"
#include "partials.cuh"

constexpr int GB_THREADS = 256;
constexpr int GB_MAX_GROUPS = 512;

// 1 / sqrt(mean(part^2) + eps) of every group of row xr into inv[0 .. groups): warp w takes groups
// w, w + warps, ...; a lane walks its group with stride 32, then the lanes meet in a butterfly.
// The tree depends on (E, groups) alone.  Ends with a barrier.
__device__ __forceinline__ void group_inverse_rms(const float* __restrict__ xr, int E, int groups, float eps, float* inv) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int Eg = E / groups;
  for (int g = warp; g < groups; g += nw) {
    const float* p = xr + (size_t)g * Eg;
    float ss = 0.f;
    for (int i = lane; i < Eg; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.0f / sqrtf(ss / (float)Eg + eps);
  }
  __syncthreads();
}

// ---------------------------------------------------------------- embedding with scale and learned positions
template <typename T>
__global__ void embedding_scaled_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out, int E,
                                        int V, float scale, const T* __restrict__ pos_table, const int* __restrict__ positions,
                                        int n_pos, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < V;
  if (!ok && threadIdx.x == 0) atomicExch(err, 1);
  const T* row = table + (size_t)(ok ? id : 0) * E;
  const T* prow = nullptr;
  if (pos_table != nullptr) {
    const int p = positions[t];
    if (p < 0 || p >= n_pos) {
      if (threadIdx.x == 0) atomicExch(err, 2);
    } else {
      prow = pos_table + (size_t)p * E;
    }
  }
  float* o = out + (size_t)t * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    float v = ok ? to_f32<T>(row[i]) * scale : 0.f;
    if (prow != nullptr) v += to_f32<T>(prow[i]);
    o[i] = v;
  }
}

// out[t] = table[ids[t]] * scale (+ pos_table[positions[t]] when a position table is given), float32.
FERRUM_API int ferrum_embedding_scaled(const void* table, int dtype, const int* ids, float* out, int n_tokens, int E, int V,
                                       float scale, const void* pos_table, const int* positions, int n_pos, int* err_flag,
                                       cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && E > 0 && V > 0, "embedding: bad sizes T=%d E=%d V=%d", n_tokens, E, V);
  FERRUM_CHECK_ARG(pos_table == nullptr || (positions != nullptr && n_pos > 0), "embedding: positions missing");
  if (n_tokens == 0) return 0;
  const int threads = E >= 1024 ? 256 : 128;
  FERRUM_DISPATCH_DTYPE(dtype, T, launch_kernel(embedding_scaled_kernel<T>, n_tokens, threads, 0, stream, (const T*)table, ids, out, E, V,
                                                scale, (const T*)pos_table, positions, n_pos, err_flag));
  FERRUM_CHECK_LAUNCH("embedding_scaled");
  return 0;
}

// ---------------------------------------------------------------- grouped RMS norm (rows may be gathered)
template <typename TOut>
__global__ void __launch_bounds__(GB_THREADS)
group_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, TOut* __restrict__ out, const int* __restrict__ rows, int E,
                  int groups, float eps) {
  __shared__ float inv[GB_MAX_GROUPS];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * E;
  group_inverse_rms(xr, E, groups, eps, inv);
  const int Eg = E / groups;
  TOut* o = out + (size_t)r * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = from_f32<TOut>(xr[i] * inv[i / Eg] * w[i]);
}

FERRUM_API int ferrum_group_norm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int n_rows, int E,
                                 int groups, float eps, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_rows >= 0 && E > 0 && groups > 0 && groups <= GB_MAX_GROUPS && E % groups == 0,
                   "group norm: bad sizes rows=%d E=%d groups=%d", n_rows, E, groups);
  FERRUM_CHECK_ARG(eps > 0.f, "group norm: eps must be positive");
  if (n_rows == 0) return 0;
  FERRUM_DISPATCH_DTYPE(out_dtype, T, launch_kernel(group_norm_kernel<T>, n_rows, GB_THREADS, 0, stream, x, w, (T*)out, rows, E, groups, eps));
  FERRUM_CHECK_LAUNCH("group_norm");
  return 0;
}

// ---------------------------------------------------------------- both norms and the token shift
// One block per token.  a, m, b: [T, E] in the compute dtype (b and w2 may be null: a layer without
// a second sublayer).  shift null: m = a.  state: [slots, E] float32, the a of every request's last
// token; stage: [requests of the batch, E] float32, receives the a of every portion's last token.
template <typename TOut>
__global__ void __launch_bounds__(GB_THREADS)
norm_pair_shift_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ w2,
                       const float* __restrict__ shift, TOut* __restrict__ a_out, TOut* __restrict__ m_out, TOut* __restrict__ b_out,
                       const int* __restrict__ positions, const int* __restrict__ req_of_token, const int* __restrict__ q_start,
                       const int* __restrict__ slots, const float* __restrict__ state, float* __restrict__ stage, int E, int groups,
                       float eps) {
  __shared__ float inv[GB_MAX_GROUPS], inv_prev[GB_MAX_GROUPS];
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int r = req_of_token[t];
  const bool first = t == q_start[r], last = t == q_start[r + 1] - 1;
  const float* xr = x + (size_t)t * E;
  group_inverse_rms(xr, E, groups, eps, inv);
  // where the previous token's a comes from: 0 nowhere (position 0), 1 the row before, 2 the state
  int prev = 0;
  if (shift != nullptr && positions[t] > 0) prev = first ? 2 : 1;
  const float* xp = xr - E;
  if (prev == 1) group_inverse_rms(xp, E, groups, eps, inv_prev);
  const float* sp = prev == 2 ? state + (size_t)slots[r] * E : nullptr;
  const int Eg = E / groups;
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    const int g = i / Eg;
    const float n = xr[i] * inv[g];
    const float a = n * w1[i];
    float m = a;
    if (shift != nullptr) {
      float ap = 0.f;
      if (prev == 1) ap = xp[i] * inv_prev[g] * w1[i];
      else if (prev == 2) ap = sp[i];
      m = a + (ap - a) * shift[i];
    }
    a_out[(size_t)t * E + i] = from_f32<TOut>(a);
    m_out[(size_t)t * E + i] = from_f32<TOut>(m);
    if (b_out != nullptr) b_out[(size_t)t * E + i] = from_f32<TOut>(n * w2[i]);
    if (last && stage != nullptr) stage[(size_t)r * E + i] = a;
  }
}

FERRUM_API int ferrum_norm_pair_shift(const float* x, const float* w1, const float* w2, const float* shift, void* a_out, void* m_out,
                                      void* b_out, int out_dtype, int n_tokens, const int* positions, const int* req_of_token,
                                      const int* q_start, const int* slots, const float* state, float* stage, int E, int groups,
                                      float eps, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && E > 0 && groups > 0 && groups <= GB_MAX_GROUPS && E % groups == 0,
                   "norm pair: bad sizes T=%d E=%d groups=%d", n_tokens, E, groups);
  FERRUM_CHECK_ARG(eps > 0.f, "norm pair: eps must be positive");
  FERRUM_CHECK_ARG((b_out == nullptr) == (w2 == nullptr), "norm pair: second weight and second output go together");
  FERRUM_CHECK_ARG(shift == nullptr || (state != nullptr && stage != nullptr && slots != nullptr), "norm pair: a token shift needs its state");
  if (n_tokens == 0) return 0;
  FERRUM_DISPATCH_DTYPE(out_dtype, T, launch_kernel(norm_pair_shift_kernel<T>, n_tokens, GB_THREADS, 0, stream, x, w1, w2, shift, (T*)a_out,
                                                    (T*)m_out, (T*)b_out, positions, req_of_token, q_start, slots, state, stage, E, groups, eps));
  FERRUM_CHECK_LAUNCH("norm_pair_shift");
  return 0;
}

// ---------------------------------------------------------------- biased gated linear unit
// act[t, f] = f(gu[t, f] + bg[f]) * (gu[t, F + f] + bu[f]); gu float32 rows of stride ld, act in the
// compute dtype.  kind 0: f = silu; 1: f = gelu with the tanh approximation; 2: the clamped unit of common.cuh
// made of both values and `limit`.  Biases may be null.
__device__ __forceinline__ float glu_act(float z, int kind) {
  if (kind == 0) return z / (1.0f + expf(-z));
  const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  return 0.5f * z * (1.0f + tanhf(u));
}
__device__ __forceinline__ float glu_of(float g, float u, int kind, float limit) {
  return kind == GLU_SWISH_CLAMP ? glu_swish_clamp(g, u, limit) : glu_act(g, kind) * u;
}

template <typename TOut>
__global__ void __launch_bounds__(256)
bias_glu_kernel(const float* __restrict__ gu, int ld, const float* __restrict__ bg, const float* __restrict__ bu, TOut* __restrict__ act,
                int ld_out, int F, int kind, float limit) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.y;
  const float* row = gu + (size_t)t * ld;
  for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < F; f += gridDim.x * blockDim.x) {
    const float g = row[f] + (bg ? bg[f] : 0.f), u = row[F + f] + (bu ? bu[f] : 0.f);
    act[(size_t)t * ld_out + f] = from_f32<TOut>(glu_of(g, u, kind, limit));
  }
}

FERRUM_API int ferrum_bias_glu(const float* gu, int ld, const float* bias_gate, const float* bias_up, void* act, int act_dtype,
                               int ld_out, int n_tokens, int F, int kind, float limit, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && n_tokens <= 65535 * 32 && F > 0 && ld >= 2 * F && ld_out >= F, "bias glu: bad sizes T=%d F=%d", n_tokens, F);
  FERRUM_CHECK_ARG(kind >= 0 && kind <= GLU_SWISH_CLAMP, "bias glu: unknown activation %d", kind);
  if (n_tokens == 0) return 0;
  FERRUM_CHECK_ARG(n_tokens <= 65535, "bias glu: too many tokens");
  const dim3 grid(min((F + 255) / 256, 64), n_tokens);
  FERRUM_DISPATCH_DTYPE(act_dtype, T, launch_kernel(bias_glu_kernel<T>, grid, dim3(256), 0, stream, gu, ld, bias_gate, bias_up, (T*)act, ld_out, F, kind, limit));
  FERRUM_CHECK_LAUNCH("bias_glu");
  return 0;
}

// The same from a product still in partials (deferred mode): one product of 2F + n_extra rows
// (gate | up | extra); the extra columns (another product of the same input) are summed into
// extra[t, :] (float32) on the way.
template <typename TOut>
__global__ void __launch_bounds__(256)
bias_glu_reduce_kernel(const float* __restrict__ bg, const float* __restrict__ bu, TOut* __restrict__ act, int ld_out, int F, int kind, float limit,
                       float* __restrict__ extra, int n_extra, const PartialLayout L) {
  __shared__ PartialTable tab;
  build_partial_table(L, tab);
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.y;
  for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < F + n_extra; f += gridDim.x * blockDim.x) {
    if (f < F) {
      const float g = partial_sum(L, tab, t, f) + (bg ? bg[f] : 0.f), u = partial_sum(L, tab, t, F + f) + (bu ? bu[f] : 0.f);
      act[(size_t)t * ld_out + f] = from_f32<TOut>(glu_of(g, u, kind, limit));
    } else {
      extra[(size_t)t * n_extra + (f - F)] = partial_sum(L, tab, t, 2 * F + (f - F));
    }
  }
}

FERRUM_API int ferrum_bias_glu_reduce(const float* bias_gate, const float* bias_up, void* act, int act_dtype, int ld_out, int n_tokens,
                                      int F, int kind, float limit, float* extra, int n_extra, const float* partials, const int* layout,
                                      cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && n_tokens <= 65535 && F > 0 && ld_out >= F && n_extra >= 0, "bias glu: bad sizes T=%d F=%d", n_tokens, F);
  FERRUM_CHECK_ARG(kind >= 0 && kind <= GLU_SWISH_CLAMP, "bias glu: unknown activation %d", kind);
  FERRUM_CHECK_ARG(n_extra == 0 || extra != nullptr, "bias glu: the extra columns need a place");
  if (n_tokens == 0) return 0;
  PartialLayout L;
  if (int r = partial_make_layout(partials, layout, &L)) return r;
  FERRUM_CHECK_ARG(2 * F + n_extra <= L.tiles * 128 && n_tokens <= L.acc_cols, "bias glu: the partials do not cover the rows");
  const dim3 grid(min((F + n_extra + 255) / 256, 64), n_tokens);
  FERRUM_DISPATCH_DTYPE(act_dtype, T, launch_kernel(bias_glu_reduce_kernel<T>, grid, dim3(256), 0, stream, bias_gate, bias_up, (T*)act, ld_out, F,
                                                    kind, limit, extra, n_extra, L));
  FERRUM_CHECK_LAUNCH("bias_glu_reduce");
  return 0;
}

// ---------------------------------------------------------------- gated residual sum
// x[t, i] += y1[t, i] * sigmoid(g1[t, i] + c1[i]) + (y2[t, i] + c2[i]) * sigmoid(g2[t, i] + c3[i]); the second term is
// left out when y2 is null.  All float32; every operand has its own row stride.  y1 and y2 may each be a
// product still in partials (deferred mode), summed while it is read.  The block of a
// portion's last token also copies the staged row of its request into the state.
__device__ __forceinline__ float gb_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

__global__ void __launch_bounds__(GB_THREADS)
gated_residual_kernel(float* __restrict__ x, int E, const float* __restrict__ y1, int ld_y1, const float* __restrict__ g1, int ld_g1,
                      const float* __restrict__ c1, const float* __restrict__ y2, int ld_y2, const float* __restrict__ c2,
                      const float* __restrict__ g2, int ld_g2, const float* __restrict__ c3, const int* __restrict__ req_of_token,
                      const int* __restrict__ q_start, const int* __restrict__ slots, const float* __restrict__ stage,
                      float* __restrict__ state, const PartialLayout L1, const PartialLayout L2) {
  __shared__ PartialTable tab1, tab2;
  if (L1.ws != nullptr) build_partial_table(L1, tab1);
  if (L2.ws != nullptr) build_partial_table(L2, tab2);
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * E;
  const bool second = y2 != nullptr || L2.ws != nullptr;
  // (with few tokens a row is shared out between gridDim.y blocks: summing partials is several loads per element)
  const int per = (E + gridDim.y - 1) / gridDim.y;
  const int lo = blockIdx.y * per, hi = min(E, lo + per);
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v1 = L1.ws != nullptr ? partial_sum(L1, tab1, t, i) : y1[(size_t)t * ld_y1 + i];
    float add = v1 * gb_sigmoid(g1[(size_t)t * ld_g1 + i] + (c1 ? c1[i] : 0.f));
    if (second) {
      const float v2 = L2.ws != nullptr ? partial_sum(L2, tab2, t, i) : y2[(size_t)t * ld_y2 + i];
      add += (v2 + (c2 ? c2[i] : 0.f)) * gb_sigmoid(g2[(size_t)t * ld_g2 + i] + (c3 ? c3[i] : 0.f));
    }
    xr[i] += add;
  }
  if (state != nullptr) {
    const int r = req_of_token[t];
    if (t == q_start[r + 1] - 1) {
      float* dst = state + (size_t)slots[r] * E;
      const float* src = stage + (size_t)r * E;
      for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) dst[i] = src[i];
    }
  }
}

FERRUM_API int ferrum_gated_residual(float* x, int n_tokens, int E, const float* y1, int ld_y1, const float* g1, int ld_g1,
                                     const float* c1, const float* y2, int ld_y2, const float* c2, const float* g2, int ld_g2,
                                     const float* c3, const int* req_of_token, const int* q_start, const int* slots,
                                     const float* stage, float* state, const float* partials1, const int* layout1,
                                     const float* partials2, const int* layout2, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && E > 0 && (y1 != nullptr || partials1 != nullptr) && g1 != nullptr, "gated residual: bad arguments");
  FERRUM_CHECK_ARG((y2 == nullptr && partials2 == nullptr) || g2 != nullptr, "gated residual: the second term needs its gate");
  PartialLayout L1{nullptr, 0, 0, 0, 0}, L2{nullptr, 0, 0, 0, 0};
  if (partials1 != nullptr) {
    if (int r = partial_make_layout(partials1, layout1, &L1)) return r;
    FERRUM_CHECK_ARG(E <= L1.tiles * 128 && n_tokens <= L1.acc_cols, "gated residual: the partials do not cover the rows");
  }
  if (partials2 != nullptr) {
    if (int r = partial_make_layout(partials2, layout2, &L2)) return r;
    FERRUM_CHECK_ARG(E <= L2.tiles * 128 && n_tokens <= L2.acc_cols, "gated residual: the partials do not cover the rows");
  }
  FERRUM_CHECK_ARG(state == nullptr || (stage != nullptr && slots != nullptr && q_start != nullptr && req_of_token != nullptr),
                   "gated residual: the state copy needs the batch description");
  if (n_tokens == 0) return 0;
  const int slices = n_tokens <= 64 ? max(1, min(16, E / 256)) : 1;
  launch_kernel(gated_residual_kernel, dim3(n_tokens, slices), dim3(GB_THREADS), 0, stream, x, E, y1, ld_y1, g1, ld_g1, c1, y2, ld_y2, c2, g2, ld_g2, c3,
                req_of_token, q_start, slots, stage, state, L1, L2);
  FERRUM_CHECK_LAUNCH("gated_residual");
  return 0;
}
