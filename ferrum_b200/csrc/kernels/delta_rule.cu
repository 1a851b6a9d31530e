// A gated delta rule with one decay per head and key channel, after its input products.
//
// Sizes: H value heads of Dv, G query/key heads of D (value head h reads query/key head h / (H / G)); C = 2 G D + H Dv
// channels pass a short causal convolution.  A token's float32 product row is [q: G D | k: G D | v: H Dv | beta logits: H];
// a second float32 row [H D] holds the decay's logits (a low-rank product made elsewhere).  Per request the state
// row keeps, in float32,
//   S [H][D][Dv]                    the memory of every head (element (d, j) of head h at (h D + d) Dv + j)
//   u [taps - 1][C]                 the last inputs of the convolution
//
// delta_prep:        a warp per (token, slot).  Slots 0 .. 2G + H - 1 are the q, k and v heads: channel c becomes
//                    silu(sum_j w[c][j] * input(t - (taps - 1 - j))[c]) (inputs before the portion's first token come
//                    from u, all zero before a sequence's first token); a q or k head is then divided by
//                    sqrt(sum of its squares + 1e-6), and q also multiplied by D^(-1/2).  The last H slots are the
//                    decays: dec[h][d] = exp(-exp(A_log[h]) * softplus(logit[h D + d] + dt_bias[h D + d])).
// delta_conv_state:  u <- the last taps - 1 inputs after this portion; a launch of its own, so that nobody reads u while
//                    it changes.
// delta_scan:        a block per (request, head, 32 value columns) walks the portion's tokens in order:
//                      S <- dec * S (row d by dec[d]);  e = beta * (v - S^T k);  S <- S + k e^T;  o = S^T q
//                    with beta = sigmoid(its logit).  Four lanes share a column (rows d = 4 i + quarter each) and add
//                    their parts by two shuffles: one fixed tree, token by token whatever the portion, so a token's
//                    result does not depend on how the sequence was cut.
#include "common.cuh"

constexpr int DR_MAX_TAPS = 16;

__device__ __forceinline__ float dr_silu(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float dr_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

__global__ void __launch_bounds__(128)
delta_prep_kernel(const float* __restrict__ proj, int ldp, const float* __restrict__ logit, int ldl, int n_tokens, int H, int G,
                  int D, int Dv, int taps, const float* __restrict__ conv_w, const float* __restrict__ dt_bias,
                  const float* __restrict__ a_log, const float* __restrict__ state, long long state_stride, long long conv_off,
                  const int* __restrict__ req_of_token, const int* __restrict__ q_start, const int* __restrict__ slots,
                  float* __restrict__ qkv, float* __restrict__ dec) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_slots = 2 * G + 2 * H;
  const long long item = (long long)blockIdx.x * 4 + warp;
  if (item >= (long long)n_tokens * n_slots) return;
  const int t = (int)(item / n_slots), slot = (int)(item % n_slots);
  const int C = 2 * G * D + H * Dv;
  if (slot >= 2 * G + H) {                                  // a head's decays
    const int h = slot - 2 * G - H;
    const float rate = expf(a_log[h]);
    for (int d = lane; d < D; d += 32) {
      const int c = h * D + d;
      dec[(size_t)t * H * D + c] = expf(-rate * dr_softplus(logit[(size_t)t * ldl + c] + dt_bias[c]));
    }
    return;
  }
  const bool is_v = slot >= 2 * G;
  const int n = is_v ? Dv : D;
  const int c0 = is_v ? 2 * G * D + (slot - 2 * G) * Dv : slot * D;
  const int r = req_of_token[t];
  const int t0 = q_start[r];
  const int local = t - t0;
  const float* u = state + (long long)slots[r] * state_stride + conv_off;
  float* dst = qkv + (size_t)t * C + c0;
  float ss = 0.f;
  for (int d = lane; d < n; d += 32) {
    const int c = c0 + d;
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = local - (taps - 1 - j);
      const float v = src >= 0 ? proj[(size_t)(t0 + src) * ldp + c] : u[(size_t)(taps - 1 + src) * C + c];
      acc = fmaf(conv_w[(size_t)c * taps + j], v, acc);
    }
    acc = dr_silu(acc);
    dst[d] = acc;
    ss = fmaf(acc, acc, ss);
  }
  if (is_v) return;
  ss = warp_sum(ss);
  float mult = 1.f / sqrtf(ss + 1e-6f);
  if (slot < G) mult *= 1.f / sqrtf((float)D);
  __syncwarp();
  for (int d = lane; d < n; d += 32) dst[d] *= mult;
}

__global__ void __launch_bounds__(256)
delta_conv_state_kernel(const float* __restrict__ proj, int ldp, int C, int taps, float* __restrict__ state, long long state_stride,
                        long long conv_off, const int* __restrict__ q_start, const int* __restrict__ slots, int n_reqs) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_reqs * C) return;
  const int r = (int)(idx / C), c = (int)(idx % C);
  const int t0 = q_start[r], n = q_start[r + 1] - t0;
  float* u = state + (long long)slots[r] * state_stride + conv_off;
  float keep[DR_MAX_TAPS];
#pragma unroll
  for (int s = 0; s < DR_MAX_TAPS; ++s) {
    if (s < taps - 1) {
      const int src = n - (taps - 1) + s;            // position within the portion of the input that row s will hold
      keep[s] = src >= 0 ? proj[(size_t)(t0 + src) * ldp + c] : u[(size_t)(taps - 1 + src) * C + c];
    }
  }
#pragma unroll
  for (int s = 0; s < DR_MAX_TAPS; ++s)
    if (s < taps - 1) u[(size_t)s * C + c] = keep[s];
}

// RQ rows a thread (D <= 4 RQ), TC tokens staged at a time.  Thread: column tid / 4 of the block's 32, rows 4 i + tid % 4.
template <int RQ, int TC>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ qkv, int C, const float* __restrict__ dec, const float* __restrict__ proj, int ldp,
                  int off_beta, float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                  const int* __restrict__ slots, float* __restrict__ o, int ldo, int H, int G, int D, int Dv) {
  constexpr int W = 4 * RQ;
  __shared__ float sq[TC][W], sk[TC][W], sg[TC][W], sv[TC][32], sb[TC];
  const int tid = threadIdx.x, col = tid >> 2, qd = tid & 3;
  const int j = blockIdx.x * 32 + col, h = blockIdx.y, r = blockIdx.z;
  const int g = h / (H / G);
  const int t0 = q_start[r], t1 = q_start[r + 1];
  float* Sg = state + (long long)slots[r] * state_stride + (size_t)h * D * Dv;
  float S[RQ];
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = 4 * i + qd;
    S[i] = (d < D && j < Dv) ? Sg[(size_t)d * Dv + j] : 0.f;
  }
  const int off_q = g * D, off_k = G * D + g * D, off_v = 2 * G * D + h * Dv + blockIdx.x * 32;
  for (int c0 = t0; c0 < t1; c0 += TC) {
    const int nt = min(TC, t1 - c0);
    __syncthreads();                                       // the chunk before has been walked
    for (int idx = tid; idx < nt * W; idx += 128) {
      const int tk = idx / W, d = idx % W;
      const size_t row = (size_t)(c0 + tk);
      sq[tk][d] = d < D ? qkv[row * C + off_q + d] : 0.f;
      sk[tk][d] = d < D ? qkv[row * C + off_k + d] : 0.f;
      sg[tk][d] = d < D ? dec[row * H * D + (size_t)h * D + d] : 1.f;
    }
    for (int idx = tid; idx < nt * 32; idx += 128) {
      const int tk = idx >> 5, c = idx & 31;
      sv[tk][c] = blockIdx.x * 32 + c < Dv ? qkv[(size_t)(c0 + tk) * C + off_v + c] : 0.f;
    }
    if (tid < nt) sb[tid] = 1.f / (1.f + expf(-proj[(size_t)(c0 + tid) * ldp + off_beta + h]));
    __syncthreads();
    for (int tk = 0; tk < nt; ++tk) {
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < RQ; ++i) {
        S[i] *= sg[tk][4 * i + qd];
        part = fmaf(S[i], sk[tk][4 * i + qd], part);
      }
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      const float e = sb[tk] * (sv[tk][col] - part);
      float po = 0.f;
#pragma unroll
      for (int i = 0; i < RQ; ++i) {
        S[i] = fmaf(sk[tk][4 * i + qd], e, S[i]);
        po = fmaf(S[i], sq[tk][4 * i + qd], po);
      }
      po += __shfl_xor_sync(0xffffffffu, po, 1);
      po += __shfl_xor_sync(0xffffffffu, po, 2);
      if (qd == 0 && j < Dv) o[(size_t)(c0 + tk) * ldo + (size_t)h * Dv + j] = po;
    }
  }
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = 4 * i + qd;
    if (d < D && j < Dv) Sg[(size_t)d * Dv + j] = S[i];
  }
}

constexpr int DR_MAX_D = 256;

// proj: float32 rows [q | k | v | beta logits] of stride ldp; logit: float32 rows [H * D] of stride ldl (the decays' logits);
// conv_w: [C][taps]; state: [slots][state_stride] float32 rows, S first and the convolution's inputs from H * D * Dv on;
// qkv [T][C] and dec [T][H * D]: float32 scratch; o: float32 [T][ldo] receives the heads' read-outs [H * Dv].
FERRUM_API int ferrum_delta_rule(const float* proj, int ldp, const float* logit, int ldl, int n_tokens, int n_reqs,
                                 const int* req_of_token, const int* q_start, const int* slots, const float* conv_w, int taps,
                                 const float* dt_bias, const float* a_log, int H, int G, int D, int Dv, float* state,
                                 long long state_stride, float* qkv, float* dec, float* o, int ldo, cudaStream_t stream) {
  FERRUM_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && D > 0 && D <= DR_MAX_D && Dv > 0, "delta_rule: bad head sizes H=%d G=%d D=%d Dv=%d", H, G, D, Dv);
  FERRUM_CHECK_ARG(taps >= 1 && taps <= DR_MAX_TAPS, "delta_rule: %d convolution taps are outside 1..%d", taps, DR_MAX_TAPS);
  const int C = 2 * G * D + H * Dv;
  FERRUM_CHECK_ARG(ldp >= C + H && ldl >= H * D && ldo >= H * Dv, "delta_rule: a row is shorter than its contents");
  FERRUM_CHECK_ARG(state_stride >= (long long)H * D * Dv + (long long)(taps - 1) * C, "delta_rule: the state row is too short");
  FERRUM_CHECK_ARG(n_reqs <= 65535 && H <= 65535, "delta_rule: too many requests or heads");
  if (n_tokens == 0) return 0;
  const long long conv_off = (long long)H * D * Dv;
  {
    const long long blocks = ((long long)n_tokens * (2 * G + 2 * H) + 3) / 4;
    FERRUM_CHECK_ARG(blocks < (1LL << 31), "delta_rule: too many rows");
    delta_prep_kernel<<<(unsigned)blocks, 128, 0, stream>>>(proj, ldp, logit, ldl, n_tokens, H, G, D, Dv, taps, conv_w, dt_bias, a_log,
                                                            state, state_stride, conv_off, req_of_token, q_start, slots, qkv, dec);
    FERRUM_CHECK_LAUNCH("delta_prep");
  }
  if (taps > 1) {
    const long long n = (long long)n_reqs * C;
    delta_conv_state_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(proj, ldp, C, taps, state, state_stride, conv_off, q_start,
                                                                             slots, n_reqs);
    FERRUM_CHECK_LAUNCH("delta_conv_state");
  }
  const dim3 grid((Dv + 31) / 32, H, n_reqs);
#define DR_LAUNCH(RQ, TC)                                                                                                      \
  delta_scan_kernel<RQ, TC><<<grid, 128, 0, stream>>>(qkv, C, dec, proj, ldp, C, state, state_stride, q_start, slots, o, ldo, H, G, D, Dv)
  if (D <= 32) DR_LAUNCH(8, 16);
  else if (D <= 64) DR_LAUNCH(16, 16);
  else if (D <= 128) DR_LAUNCH(32, 16);
  else DR_LAUNCH(64, 8);
#undef DR_LAUNCH
  FERRUM_CHECK_LAUNCH("delta_scan");
  return 0;
}
