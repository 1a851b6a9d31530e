// A matrix-memory recurrence with exponential gates kept stable by a running maximum (the mLSTM cell), after its
// input product.  H heads with keys of D and values of Dv.  A token's float32 product row holds q [H D], k [H D],
// v [H Dv] and one input-gate and one forget-gate logit per head (at offsets the caller gives).  Per request the
// state row keeps, in float32,
//   S [H][D][Dv]      the memory            (element (d, j) of head h at (h D + d) Dv + j)
//   n [H][X][D]       the normaliser, one copy per block of 32 value columns (X = ceil(Dv / 32))
//   m [H][X]          the running maximum, likewise   (all zero before a sequence's first token: m starts at 0)
//
// Per head and token, with i = cap * tanh((logit_i + b_i) / cap) and f = logsigmoid(cap * tanh((logit_f + b_f) / cap)):
//   m' = max(f + m, i);   S <- e^(f + m - m') S + e^(i - m') k v^T;   n <- e^(f + m - m') n + e^(i - m') k
//   o = S^T q' / (max(|n . q'|, e^(-m')) + 1e-6)          with q' = q D^(-1/2)
//
// A block per (request, head, 32 value columns) walks the portion's tokens in order.  Four lanes share a column (rows
// d = 4 i + quarter each, and the same rows of n) and add their parts by two shuffles: one fixed tree, token by token
// whatever the portion, so a token's result does not depend on how the sequence was cut.  Every block of a head works
// out n and m alike and keeps a copy of its own in the state (a block may start after another of its head has finished).
#include "common.cuh"

__device__ __forceinline__ float mm_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <int RQ, int TC>
__global__ void __launch_bounds__(128)
matrix_memory_scan_kernel(const float* __restrict__ proj, int ldp, int off_q, int off_k, int off_v, int off_i, int off_f,
                          const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                          float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                          const int* __restrict__ slots, float* __restrict__ o, int ldo, int H, int D, int Dv) {
  constexpr int W = 4 * RQ;
  __shared__ float sq[TC][W], sk[TC][W], sv[TC][32], si[TC], sf[TC];
  const int tid = threadIdx.x, col = tid >> 2, qd = tid & 3;
  const int j = blockIdx.x * 32 + col, h = blockIdx.y, r = blockIdx.z;
  const int t0 = q_start[r], t1 = q_start[r + 1];
  float* const base = state + (long long)slots[r] * state_stride;
  float* const Sg = base + (size_t)h * D * Dv;
  const int X = gridDim.x;
  float* const ng = base + (size_t)H * D * Dv + ((size_t)h * X + blockIdx.x) * D;
  float* const mg = base + (size_t)H * D * Dv + (size_t)H * X * D + (size_t)h * X + blockIdx.x;
  float S[RQ], n[RQ];
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = 4 * i + qd;
    S[i] = (d < D && j < Dv) ? Sg[(size_t)d * Dv + j] : 0.f;
    n[i] = d < D ? ng[d] : 0.f;
  }
  float m = *mg;
  const float q_scale = 1.f / sqrtf((float)D);
  for (int c0 = t0; c0 < t1; c0 += TC) {
    const int nt = min(TC, t1 - c0);
    __syncthreads();                                       // the chunk before has been walked
    for (int idx = tid; idx < nt * W; idx += 128) {
      const int tk = idx / W, d = idx % W;
      const float* row = proj + (size_t)(c0 + tk) * ldp;
      sq[tk][d] = d < D ? row[off_q + h * D + d] * q_scale : 0.f;
      sk[tk][d] = d < D ? row[off_k + h * D + d] : 0.f;
    }
    for (int idx = tid; idx < nt * 32; idx += 128) {
      const int tk = idx >> 5, c = idx & 31;
      sv[tk][c] = blockIdx.x * 32 + c < Dv ? proj[(size_t)(c0 + tk) * ldp + off_v + h * Dv + blockIdx.x * 32 + c] : 0.f;
    }
    if (tid < nt) {
      const float* row = proj + (size_t)(c0 + tid) * ldp;
      si[tid] = cap * tanhf((row[off_i + h] + bias_i[h]) / cap);
      sf[tid] = mm_logsigmoid(cap * tanhf((row[off_f + h] + bias_f[h]) / cap));
    }
    __syncthreads();
    for (int tk = 0; tk < nt; ++tk) {
      const float fm = sf[tk] + m;
      const float m_new = fmaxf(fm, si[tk]);
      const float a = expf(fm - m_new), b = expf(si[tk] - m_new);
      const float bv = b * sv[tk][col];
      float num = 0.f, nq = 0.f;
#pragma unroll
      for (int i = 0; i < RQ; ++i) {
        const float kk = sk[tk][4 * i + qd], qq = sq[tk][4 * i + qd];
        S[i] = fmaf(kk, bv, a * S[i]);
        n[i] = fmaf(kk, b, a * n[i]);
        num = fmaf(S[i], qq, num);
        nq = fmaf(n[i], qq, nq);
      }
      num += __shfl_xor_sync(0xffffffffu, num, 1);
      nq += __shfl_xor_sync(0xffffffffu, nq, 1);
      num += __shfl_xor_sync(0xffffffffu, num, 2);
      nq += __shfl_xor_sync(0xffffffffu, nq, 2);
      m = m_new;
      if (qd == 0 && j < Dv) o[(size_t)(c0 + tk) * ldo + (size_t)h * Dv + j] = num / (fmaxf(fabsf(nq), expf(-m_new)) + 1e-6f);
    }
  }
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = 4 * i + qd;
    if (d < D && j < Dv) Sg[(size_t)d * Dv + j] = S[i];
    if (col == 0 && d < D) ng[d] = n[i];
  }
  if (tid == 0) *mg = m;
}

constexpr int MM_MAX_D = 256;

// proj: float32 rows of stride ldp holding q, k (H * D each), v (H * Dv) and the gate logits (H each) at the given
// offsets; bias_i, bias_f: [H]; state: [slots][state_stride] float32 rows [S | n | m] (H * D * Dv + ceil(Dv / 32) * (H * D + H) floats); o: float32 [T][ldo] receives the
// heads' read-outs [H * Dv].
FERRUM_API int ferrum_matrix_memory(const float* proj, int ldp, int off_q, int off_k, int off_v, int off_i, int off_f,
                                    const float* bias_i, const float* bias_f, float cap, int n_tokens, int n_reqs,
                                    const int* q_start, const int* slots, int H, int D, int Dv, float* state,
                                    long long state_stride, float* o, int ldo, cudaStream_t stream) {
  FERRUM_CHECK_ARG(H > 0 && D > 0 && D <= MM_MAX_D && Dv > 0, "matrix_memory: bad head sizes H=%d D=%d Dv=%d", H, D, Dv);
  FERRUM_CHECK_ARG(cap > 0.f, "matrix_memory: the gates' cap must be positive");
  FERRUM_CHECK_ARG(ldo >= H * Dv && state_stride >= (long long)H * D * Dv + (long long)((Dv + 31) / 32) * (H * D + H), "matrix_memory: a row is too short");
  FERRUM_CHECK_ARG(n_reqs <= 65535 && H <= 65535, "matrix_memory: too many requests or heads");
  if (n_tokens == 0) return 0;
  const dim3 grid((Dv + 31) / 32, H, n_reqs);
#define MM_LAUNCH(RQ, TC)                                                                                                       \
  matrix_memory_scan_kernel<RQ, TC><<<grid, 128, 0, stream>>>(proj, ldp, off_q, off_k, off_v, off_i, off_f, bias_i, bias_f, cap, state, \
                                                              state_stride, q_start, slots, o, ldo, H, D, Dv)
  if (D <= 32) MM_LAUNCH(8, 16);
  else if (D <= 64) MM_LAUNCH(16, 16);
  else if (D <= 128) MM_LAUNCH(32, 16);
  else MM_LAUNCH(64, 8);
#undef MM_LAUNCH
  FERRUM_CHECK_LAUNCH("matrix_memory_scan");
  return 0;
}
