// Kernels of a block whose norms sit on the sublayers' RESULTS, all float32 arithmetic:
//
// post_norm_add:   h[t] += ls * (rms(y[t]) * w) with rms(v) = v / sqrt(mean(v^2) + eps); `ls` (a layer scale per
//                  element) may be null.  When asked it also leaves the new row in the compute type, which is what
//                  the next sublayer reads (the sublayers of such a block read the residual row itself).  Without y
//                  it only makes that copy (the first block's input).
// dual_norm_mean:  out[t] = (rms(a[t]) * wa + rms(b[t]) * wb) / 2: two branches that read the same input meet.
// head_gate_norm:  per (token, head): out = rms(o_head) * w * sigmoid(gate logits), rounded once to the compute
//                  type; the weight is one vector for all heads or one per head.
//
// One block per token (one warp per token and head in head_gate_norm); a row's sums are taken with one fixed tree,
// so a token's result does not depend on what else is in the batch.
#include "common.cuh"

constexpr int PN_THREADS = 256;

template <typename TX>
__global__ void __launch_bounds__(PN_THREADS)
post_norm_add_kernel(float* __restrict__ h, int E, const float* __restrict__ y, int ldy, const float* __restrict__ w,
                     const float* __restrict__ ls, float eps, TX* __restrict__ xc, int ldx) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  float* hr = h + (size_t)t * E;
  if (y == nullptr) {
    if (xc != nullptr)
      for (int i = threadIdx.x; i < E; i += PN_THREADS) xc[(size_t)t * ldx + i] = from_f32<TX>(hr[i]);
    return;
  }
  const float* yr = y + (size_t)t * ldy;
  float ss = 0.f;
  for (int i = threadIdx.x; i < E; i += PN_THREADS) ss = fmaf(yr[i], yr[i], ss);
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)E + eps);
  for (int i = threadIdx.x; i < E; i += PN_THREADS) {
    const float n = yr[i] * r * w[i];
    const float v = hr[i] + (ls != nullptr ? ls[i] * n : n);
    hr[i] = v;
    if (xc != nullptr) xc[(size_t)t * ldx + i] = from_f32<TX>(v);
  }
}

__global__ void __launch_bounds__(PN_THREADS)
dual_norm_mean_kernel(const float* __restrict__ a, int lda, const float* __restrict__ b, int ldb, const float* __restrict__ wa,
                      const float* __restrict__ wb, float eps, int E, float* __restrict__ out, int ldo) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const float* ar = a + (size_t)t * lda;
  const float* br = b + (size_t)t * ldb;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < E; i += PN_THREADS) {
    sa = fmaf(ar[i], ar[i], sa);
    sb = fmaf(br[i], br[i], sb);
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ra = 1.f / sqrtf(sa / (float)E + eps), rb = 1.f / sqrtf(sb / (float)E + eps);
  for (int i = threadIdx.x; i < E; i += PN_THREADS)
    out[(size_t)t * ldo + i] = 0.5f * (ar[i] * ra * wa[i] + br[i] * rb * wb[i]);
}

template <typename T>
__global__ void __launch_bounds__(128)
head_gate_norm_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gate, int ldg, const float* __restrict__ w,
                      int w_per_head, float eps, int n_tokens, int H, int Dv, T* __restrict__ out, int ldout) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + warp;
  if (item >= (long long)n_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const float* src = o + (size_t)t * ldo + (size_t)h * Dv;
  const float* g = gate != nullptr ? gate + (size_t)t * ldg + (size_t)h * Dv : nullptr;
  const float* wr = w + (w_per_head ? (size_t)h * Dv : 0);
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) ss = fmaf(src[d], src[d], ss);
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)Dv + eps);
  for (int d = lane; d < Dv; d += 32) {
    float v = src[d] * r * wr[d];
    if (g != nullptr) v *= 1.f / (1.f + expf(-g[d]));
    out[(size_t)t * ldout + (size_t)h * Dv + d] = from_f32<T>(v);
  }
}

// h [T, E] float32 += ls * rms(y) * w; xc (may be null): the new rows in the type `x_dtype`.  y null: only the copy.
FERRUM_API int ferrum_post_norm_add(float* h, int E, const float* y, int ldy, const float* w, const float* ls, float eps,
                                    void* xc, int ldx, int x_dtype, int n_tokens, cudaStream_t stream) {
  FERRUM_CHECK_ARG(E > 0 && n_tokens >= 0 && (y == nullptr || (ldy >= E && w != nullptr)) && (xc == nullptr || ldx >= E),
                   "post_norm_add: bad sizes");
  if (n_tokens == 0 || (y == nullptr && xc == nullptr)) return 0;
  FERRUM_DISPATCH_DTYPE(x_dtype, T, (post_norm_add_kernel<T><<<n_tokens, PN_THREADS, 0, stream>>>(h, E, y, ldy, w, ls, eps, (T*)xc, ldx)));
  FERRUM_CHECK_LAUNCH("post_norm_add");
  return 0;
}

FERRUM_API int ferrum_dual_norm_mean(const float* a, int lda, const float* b, int ldb, const float* wa, const float* wb, float eps,
                                     int E, float* out, int ldo, int n_tokens, cudaStream_t stream) {
  FERRUM_CHECK_ARG(E > 0 && n_tokens >= 0 && lda >= E && ldb >= E && ldo >= E, "dual_norm_mean: bad sizes");
  if (n_tokens == 0) return 0;
  dual_norm_mean_kernel<<<n_tokens, PN_THREADS, 0, stream>>>(a, lda, b, ldb, wa, wb, eps, E, out, ldo);
  FERRUM_CHECK_LAUNCH("dual_norm_mean");
  return 0;
}

// o float32 [T, >= H * Dv]; gate: float32 logits with the same layout and a stride of their own (may be null);
// w: [Dv], or [H * Dv] with w_per_head; out [T, >= H * Dv] in the type `dtype`.
FERRUM_API int ferrum_head_gate_norm(const float* o, int ldo, const float* gate, int ldg, const float* w, int w_per_head, float eps,
                                     int n_tokens, int H, int Dv, void* out, int ldout, int dtype, cudaStream_t stream) {
  FERRUM_CHECK_ARG(H > 0 && Dv > 0 && ldo >= H * Dv && ldout >= H * Dv && (gate == nullptr || ldg >= H * Dv), "head_gate_norm: bad sizes");
  if (n_tokens == 0) return 0;
  const long long blocks = ((long long)n_tokens * H + 3) / 4;
  FERRUM_CHECK_ARG(blocks < (1LL << 31), "head_gate_norm: too many rows");
  FERRUM_DISPATCH_DTYPE(dtype, T, (head_gate_norm_kernel<T><<<(unsigned)blocks, 128, 0, stream>>>(o, ldo, gate, ldg, w, w_per_head, eps,
                                                                                              n_tokens, H, Dv, (T*)out, ldout)));
  FERRUM_CHECK_LAUNCH("head_gate_norm");
  return 0;
}
