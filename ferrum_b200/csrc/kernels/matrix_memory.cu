// A matrix-memory recurrence with exponential gates kept stable by a running maximum (the mLSTM cell), after its
// input product.  H heads with keys of D and values of Dv.  A token's float32 product row holds q [H D], k [H D],
// v [H Dv] and one input-gate and one forget-gate logit per head (at offsets the caller gives).  Per request the
// state row keeps, in float32,
//   S [H][D][Dv]      the memory            (element (d, j) of head h at (h D + d) Dv + j)
//   n [H][X][D]       the normaliser, one copy per eight value columns (X = ceil(Dv / 8))
//   m [H][X]          the running maximum, likewise   (all zero before a sequence's first token: m starts at 0)
//
// Per head and token, with i = cap * tanh((logit_i + b_i) / cap) and f = logsigmoid(cap * tanh((logit_f + b_f) / cap)):
//   m' = max(f + m, i);   S <- e^(f + m - m') S + e^(i - m') k v^T;   n <- e^(f + m - m') n + e^(i - m') k
//   o = S^T q' / (max(|n . q'|, e^(-m')) + 1e-6)          with q' = q D^(-1/2)
//
// A block per (request, head, a group of value columns) walks the portion's tokens in order.  D / 8 lanes share a column
// (eight rows each, and the same rows of n) and add their parts by shuffles: one fixed tree, token by token whatever the
// portion, so a token's result does not depend on how the sequence was cut.  Every block of a head works out n and m
// alike and keeps copies of its own in the state (a block may start after another block of its head has finished).
#include "common.cuh"

constexpr int MM_COPY_COLS = 8;      // value columns per copy of n and m in the state row

__device__ __forceinline__ float mm_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

__device__ __forceinline__ void mm_cp_async4(float* smem, const float* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void mm_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void mm_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// The two log gates of every (token, head), off the walk: gates[t][h] = i, gates[t][H + h] = f.
__global__ void __launch_bounds__(256)
matrix_memory_gates_kernel(const float* __restrict__ proj, int ldp, int off_i, int off_f, const float* __restrict__ bias_i,
                           const float* __restrict__ bias_f, float cap, int n_tokens, int H, float* __restrict__ gates) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * H) return;
  const int t = (int)(idx / H), h = (int)(idx % H);
  const float* row = proj + (size_t)t * ldp;
  gates[(size_t)t * 2 * H + h] = cap * tanhf((row[off_i + h] + bias_i[h]) / cap);
  gates[(size_t)t * 2 * H + H + h] = mm_logsigmoid(cap * tanhf((row[off_f + h] + bias_f[h]) / cap));
}

// LPC lanes share a value column (D <= 8 LPC): lane q of them holds rows d = LPC i + q, i < 8, of the column and of n in
// registers, and a block of 256 threads walks 256 / LPC columns.  TC tokens are staged at a time; a staged token row keeps
// the lanes' elements apart (lane q at 12 q + i: a lane reads its rows four at a time, the lanes' 16-byte reads spread over
// the banks).  The chunk after the one being walked is on its way meanwhile, element by element with cp.async straight to
// its place; a token's operands are read one token ahead of their use.  A block reads the copy of n and m that belongs to
// its first eight columns and writes the copies of all its columns, so whichever block shape walks the next portion finds
// every copy up to date.
template <int LPC, int TC>
__global__ void __launch_bounds__(256)
matrix_memory_scan_kernel(const float* __restrict__ proj, int ldp, int off_q, int off_k, int off_v, const float* __restrict__ gates,
                          float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                          const int* __restrict__ slots, float* __restrict__ o, int ldo, int H, int D, int Dv) {
  constexpr int RQ = 8, QS = RQ + 4, W = LPC * QS, WD = LPC * RQ, CB = 256 / LPC;
  constexpr int LD = (TC * 2 * WD + 255) / 256;
  static_assert(TC * CB <= 256 && CB % MM_COPY_COLS == 0, "one copy a thread brings a chunk's values");
  __shared__ __align__(16) float sq[2][TC + 1][W], sk[2][TC + 1][W];          // (one row more: the walk reads a token ahead)
  __shared__ float sv[2][TC][CB], si[2][TC], sf[2][TC];
  __shared__ float so[2][TC][CB], sn[2][TC][CB], sm[2][TC];         // a chunk's sums and maxima: its read-outs are formed and written after its walk
  const int tid = threadIdx.x, col = tid / LPC, q = tid % LPC;
  const int j = blockIdx.x * CB + col, h = blockIdx.y, r = blockIdx.z;
  const int t0 = q_start[r], t1 = q_start[r + 1];
  float* const base = state + (long long)slots[r] * state_stride;
  float* const Sg = base + (size_t)h * D * Dv;
  const int X = (Dv + MM_COPY_COLS - 1) / MM_COPY_COLS;                      // copies of n and m: one per eight value columns
  const int x0 = blockIdx.x * (CB / MM_COPY_COLS);                           // this block's first copy
  float* const ng = base + (size_t)H * D * Dv + (size_t)h * X * D;           // [X][D]
  float* const mg = base + (size_t)H * D * Dv + (size_t)H * X * D + (size_t)h * X;
  auto stage = [&](int c0, int b) {              // a chunk's elements on their way into buffer b
    const int nt = min(TC, t1 - c0);
#pragma unroll
    for (int it = 0; it < LD; ++it) {
      const int idx = tid + it * 256;
      const int which = idx / (TC * WD), tk = (idx / WD) % TC, d = idx % WD;
      if (idx < TC * 2 * WD) {
        float* dst = (which == 0 ? &sq[b][tk][0] : &sk[b][tk][0]) + (d % LPC) * QS + d / LPC;
        if (tk < nt && d < D) mm_cp_async4(dst, proj + (size_t)(c0 + tk) * ldp + (which == 0 ? off_q : off_k) + h * D + d);
        else *dst = 0.f;
      }
    }
    if (tid < TC * CB) {
      const int tk = tid / CB, c = tid % CB;
      if (tk < nt && blockIdx.x * CB + c < Dv) mm_cp_async4(&sv[b][tk][c], proj + (size_t)(c0 + tk) * ldp + off_v + h * Dv + blockIdx.x * CB + c);
      else sv[b][tk][c] = 0.f;
    }
    if (tid < nt) {
      mm_cp_async4(&si[b][tid], gates + (size_t)(c0 + tid) * 2 * H + h);
      mm_cp_async4(&sf[b][tid], gates + (size_t)(c0 + tid) * 2 * H + H + h);
    }
    mm_cp_async_commit();
  };
  if (t0 < t1) stage(t0, 0);
  float S[RQ], n[RQ];
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = LPC * i + q;
    S[i] = (d < D && j < Dv) ? Sg[(size_t)d * Dv + j] : 0.f;
    n[i] = d < D ? ng[(size_t)x0 * D + d] : 0.f;
  }
  float m = mg[x0];
  const float q_scale = 1.f / sqrtf((float)D);
  mm_cp_async_wait_all();
  __syncthreads();
  int b = 0;
  for (int c0 = t0; c0 < t1; c0 += TC, b ^= 1) {
    const int nt = min(TC, t1 - c0);
    if (c0 + TC < t1) stage(c0 + TC, b ^ 1);     // (that buffer was last read before the barrier that ended the chunk before)
    const float4* k4 = reinterpret_cast<const float4*>(&sk[b][0][q * QS]);
    const float4* q4 = reinterpret_cast<const float4*>(&sq[b][0][q * QS]);
    float4 ka = k4[0], kb = k4[1], qa = q4[0], qb = q4[1];
    float ig = si[b][0], fg = sf[b][0], vj = sv[b][0][col];
    for (int tk = 0; tk < nt; ++tk) {
      // the next token's operands (past the chunk's last token: the spare row, never used)
      const int nx = (tk + 1) * (W / 4), tn = min(tk + 1, TC - 1);
      const float4 ka2 = k4[nx], kb2 = k4[nx + 1], qa2 = q4[nx], qb2 = q4[nx + 1];
      const float ig2 = si[b][tn], fg2 = sf[b][tn], vj2 = sv[b][tn][col];
      const float fm = fg + m;
      const float m_new = fmaxf(fm, ig);
      const float a = expf(fm - m_new), bb = expf(ig - m_new);
      const float bv = bb * vj;
      S[0] = fmaf(ka.x, bv, a * S[0]); S[1] = fmaf(ka.y, bv, a * S[1]); S[2] = fmaf(ka.z, bv, a * S[2]); S[3] = fmaf(ka.w, bv, a * S[3]);
      S[4] = fmaf(kb.x, bv, a * S[4]); S[5] = fmaf(kb.y, bv, a * S[5]); S[6] = fmaf(kb.z, bv, a * S[6]); S[7] = fmaf(kb.w, bv, a * S[7]);
      n[0] = fmaf(ka.x, bb, a * n[0]); n[1] = fmaf(ka.y, bb, a * n[1]); n[2] = fmaf(ka.z, bb, a * n[2]); n[3] = fmaf(ka.w, bb, a * n[3]);
      n[4] = fmaf(kb.x, bb, a * n[4]); n[5] = fmaf(kb.y, bb, a * n[5]); n[6] = fmaf(kb.z, bb, a * n[6]); n[7] = fmaf(kb.w, bb, a * n[7]);
      float num = (fmaf(S[4], qb.x, S[0] * qa.x) + fmaf(S[5], qb.y, S[1] * qa.y)) + (fmaf(S[6], qb.z, S[2] * qa.z) + fmaf(S[7], qb.w, S[3] * qa.w));
      float nq = (fmaf(n[4], qb.x, n[0] * qa.x) + fmaf(n[5], qb.y, n[1] * qa.y)) + (fmaf(n[6], qb.z, n[2] * qa.z) + fmaf(n[7], qb.w, n[3] * qa.w));
#pragma unroll
      for (int off = 1; off < LPC; off <<= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, num, off), o2 = __shfl_xor_sync(0xffffffffu, nq, off);
        num += o1;
        nq += o2;
      }
      m = m_new;
      if (q == 0) {
        so[b][tk][col] = num;
        sn[b][tk][col] = nq;
        if (col == 0) sm[b][tk] = m_new;
      }
      ka = ka2; kb = kb2; qa = qa2; qb = qb2;
      ig = ig2; fg = fg2; vj = vj2;
    }
    mm_cp_async_wait_all();
    __syncthreads();
    if (tid < nt * CB) {                         // (the next chunk's walk fills the other buffers; a barrier lies before these are written again)
      const int tk = tid / CB, c = tid % CB;
      if (blockIdx.x * CB + c < Dv)
        o[(size_t)(c0 + tk) * ldo + (size_t)h * Dv + blockIdx.x * CB + c] =
            so[b][tk][c] * q_scale / (fmaxf(fabsf(sn[b][tk][c]) * q_scale, expf(-sm[b][tk])) + 1e-6f);
    }
  }
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = LPC * i + q;
    if (d < D && j < Dv) Sg[(size_t)d * Dv + j] = S[i];
    // column c of the block's first columns stores copy x0 + c (every column's n is the same)
    if (col < CB / MM_COPY_COLS && x0 + col < X && d < D) ng[(size_t)(x0 + col) * D + d] = n[i];
  }
  if (q == 0 && col < CB / MM_COPY_COLS && x0 + col < X) mg[x0 + col] = m;
}

constexpr int MM_MAX_D = 256;

// proj: float32 rows of stride ldp holding q, k (H * D each), v (H * Dv) and the gate logits (H each) at the given
// offsets; bias_i, bias_f: [H]; gates: float32 scratch [T][2 H]; state: [slots][state_stride] float32 rows [S | n | m] (`ferrum_matrix_memory_state_floats` floats); o: float32 [T][ldo] receives the
// heads' read-outs [H * Dv].
FERRUM_API long long ferrum_matrix_memory_state_floats(int H, int D, int Dv) {
  return (long long)H * D * Dv + (long long)((Dv + MM_COPY_COLS - 1) / MM_COPY_COLS) * ((long long)H * D + H);
}

FERRUM_API int ferrum_matrix_memory(const float* proj, int ldp, int off_q, int off_k, int off_v, int off_i, int off_f,
                                    const float* bias_i, const float* bias_f, float cap, int n_tokens, int n_reqs,
                                    const int* q_start, const int* slots, int H, int D, int Dv, float* state,
                                    long long state_stride, float* gates, float* o, int ldo, cudaStream_t stream) {
  FERRUM_CHECK_ARG(H > 0 && D > 0 && D <= MM_MAX_D && Dv > 0, "matrix_memory: bad head sizes H=%d D=%d Dv=%d", H, D, Dv);
  FERRUM_CHECK_ARG(cap > 0.f, "matrix_memory: the gates' cap must be positive");
  FERRUM_CHECK_ARG(ldo >= H * Dv && state_stride >= ferrum_matrix_memory_state_floats(H, D, Dv), "matrix_memory: a row is too short");
  FERRUM_CHECK_ARG(n_reqs <= 65535 && H <= 65535, "matrix_memory: too many requests or heads");
  if (n_tokens == 0) return 0;
  {
    const long long n = (long long)n_tokens * H;
    matrix_memory_gates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(proj, ldp, off_i, off_f, bias_i, bias_f, cap, n_tokens, H, gates);
    FERRUM_CHECK_LAUNCH("matrix_memory_gates");
  }
#define MM_LAUNCH(LPC, TC)                                                                                                      \
  matrix_memory_scan_kernel<LPC, TC><<<dim3((Dv + 256 / LPC - 1) / (256 / LPC), H, n_reqs), 256, 0, stream>>>(                  \
      proj, ldp, off_q, off_k, off_v, gates, state, state_stride, q_start, slots, o, ldo, H, D, Dv)
  if (D <= 32) MM_LAUNCH(4, 4);
  else if (D <= 64) MM_LAUNCH(8, 8);
  else if (D <= 128) MM_LAUNCH(16, 8);
  else MM_LAUNCH(32, 4);
#undef MM_LAUNCH
  FERRUM_CHECK_LAUNCH("matrix_memory_scan");
  return 0;
}
