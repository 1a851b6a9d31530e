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
// A block per (request, head, 32 value columns) walks the portion's tokens in order, token by token whatever the portion,
// and the sums over the rows have one fixed tree, so a token's result does not depend on how the sequence was cut.  Every
// block of a head works out n and m alike and keeps copies of its own in the state (a block may start after another block
// of its head has finished).
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

// A block of 128 threads walks 32 value columns: thread (rg, cq) holds rows d = rg RQ .. rg RQ + RQ - 1 (sixteen row groups,
// D <= 16 RQ) of the four columns 4 cq .. 4 cq + 3, and the same rows of n, in registers.  The memory's update needs no sum
// across rows, so nothing crosses lanes or warps inside the walk: a token's k and q are broadcast reads of shared memory,
// and every value read serves four columns (what bounds such a walk is the path from shared memory to the registers: a
// 16-byte read a lane takes four cycles of it per warp, whatever is broadcast).  Each thread leaves its part of S^T q (and
// of n . q) in shared memory; after a chunk the block adds the sixteen parts in row order (one fixed tree) and writes the
// read-outs.  TC tokens are staged at a time, the next chunk on its way meanwhile (cp.async).  A block reads the copy of n
// and m that belongs to its first eight columns and writes the copies of all its columns.
constexpr int MM_THREADS = 128, MM_RG = 16, MM_CB = 32;

template <int RQ, int TC>
__global__ void __launch_bounds__(MM_THREADS)
matrix_memory_scan_kernel(const float* __restrict__ proj, int ldp, int off_q, int off_k, int off_v, const float* __restrict__ gates,
                          float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                          const int* __restrict__ slots, float* __restrict__ o, int ldo, int H, int D, int Dv) {
  constexpr int DP = MM_RG * RQ, NT = MM_THREADS, CB = MM_CB;
  constexpr int LD = (TC * 2 * DP + NT - 1) / NT, LV = (TC * CB + NT - 1) / NT;
  static_assert(RQ % 4 == 0 && TC <= NT, "rows are read four at a time");
  __shared__ __align__(16) float sq[2][TC][DP], sk[2][TC][DP], sv[2][TC][CB], pn[MM_RG][TC][CB];
  __shared__ float si[2][TC], sf[2][TC], pq[MM_RG][TC], sm[TC];      // pn, pq, sm: the threads' parts of a chunk's sums, and its maxima
  const int tid = threadIdx.x, cq = tid % (CB / 4), rg = tid / (CB / 4);
  const int j0 = blockIdx.x * CB + 4 * cq, h = blockIdx.y, r = blockIdx.z;
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
      const int idx = tid + it * NT;
      const int which = idx / (TC * DP), tk = (idx / DP) % TC, d = idx % DP;
      if (idx < TC * 2 * DP) {
        float* dst = which == 0 ? &sq[b][tk][d] : &sk[b][tk][d];
        if (tk < nt && d < D) mm_cp_async4(dst, proj + (size_t)(c0 + tk) * ldp + (which == 0 ? off_q : off_k) + h * D + d);
        else *dst = 0.f;
      }
    }
#pragma unroll
    for (int it = 0; it < LV; ++it) {
      const int idx = tid + it * NT;
      const int tk = idx / CB, c = idx % CB;
      if (idx < TC * CB) {
        if (tk < nt && blockIdx.x * CB + c < Dv) mm_cp_async4(&sv[b][tk][c], proj + (size_t)(c0 + tk) * ldp + off_v + h * Dv + blockIdx.x * CB + c);
        else sv[b][tk][c] = 0.f;
      }
    }
    if (tid < nt) {
      mm_cp_async4(&si[b][tid], gates + (size_t)(c0 + tid) * 2 * H + h);
      mm_cp_async4(&sf[b][tid], gates + (size_t)(c0 + tid) * 2 * H + H + h);
    }
    mm_cp_async_commit();
  };
  if (t0 < t1) stage(t0, 0);
  float S[4][RQ], n[RQ];
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = rg * RQ + i;
#pragma unroll
    for (int c = 0; c < 4; ++c) S[c][i] = (d < D && j0 + c < Dv) ? Sg[(size_t)d * Dv + j0 + c] : 0.f;
    n[i] = d < D ? ng[(size_t)x0 * D + d] : 0.f;
  }
  float m = mg[x0];
  const float q_scale = 1.f / sqrtf((float)D);
  mm_cp_async_wait_all();
  __syncthreads();
  int b = 0;
  for (int c0 = t0; c0 < t1; c0 += TC, b ^= 1) {
    const int nt = min(TC, t1 - c0);
    if (c0 + TC < t1) stage(c0 + TC, b ^ 1);     // (that buffer was last read before the barriers that ended the chunk before)
    for (int tk = 0; tk < nt; ++tk) {
      const float fm = sf[b][tk] + m;
      const float m_new = fmaxf(fm, si[b][tk]);
      const float a = expf(fm - m_new), bb = expf(si[b][tk] - m_new);
      const float4 v4 = *reinterpret_cast<const float4*>(&sv[b][tk][4 * cq]);
      const float bv0 = bb * v4.x, bv1 = bb * v4.y, bv2 = bb * v4.z, bv3 = bb * v4.w;
      const float4* k4 = reinterpret_cast<const float4*>(&sk[b][tk][rg * RQ]);
      const float4* q4 = reinterpret_cast<const float4*>(&sq[b][tk][rg * RQ]);
      float u0 = 0.f, u1 = 0.f, u2 = 0.f, u3 = 0.f, w = 0.f;
#pragma unroll
      for (int i = 0; i < RQ / 4; ++i) {
        const float4 kk = k4[i], qq = q4[i];
        const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int x = 4 * i + e;
          S[0][x] = fmaf(kv[e], bv0, a * S[0][x]);
          S[1][x] = fmaf(kv[e], bv1, a * S[1][x]);
          S[2][x] = fmaf(kv[e], bv2, a * S[2][x]);
          S[3][x] = fmaf(kv[e], bv3, a * S[3][x]);
          n[x] = fmaf(kv[e], bb, a * n[x]);
          u0 = fmaf(S[0][x], qv[e], u0);
          u1 = fmaf(S[1][x], qv[e], u1);
          u2 = fmaf(S[2][x], qv[e], u2);
          u3 = fmaf(S[3][x], qv[e], u3);
          w = fmaf(n[x], qv[e], w);
        }
      }
      m = m_new;
      *reinterpret_cast<float4*>(&pn[rg][tk][4 * cq]) = make_float4(u0, u1, u2, u3);
      if (cq == 0) {
        pq[rg][tk] = w;
        if (rg == 0) sm[tk] = m_new;
      }
    }
    mm_cp_async_wait_all();
    __syncthreads();
    for (int idx = tid; idx < nt * CB; idx += NT) {
      const int tk = idx / CB, c = idx % CB;
      if (blockIdx.x * CB + c < Dv) {
        float num = 0.f, nq = 0.f;
#pragma unroll
        for (int g = 0; g < MM_RG; ++g) {
          num += pn[g][tk][c];
          nq += pq[g][tk];
        }
        o[(size_t)(c0 + tk) * ldo + (size_t)h * Dv + blockIdx.x * CB + c] =
            num * q_scale / (fmaxf(fabsf(nq) * q_scale, expf(-sm[tk])) + 1e-6f);
      }
    }
    __syncthreads();                             // (the parts are read: the next chunk's walk may write them)
  }
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = rg * RQ + i;
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (d < D && j0 + c < Dv) Sg[(size_t)d * Dv + j0 + c] = S[c][i];
    // column quad c of the first quads stores copy x0 + c of the thread's rows (every column's n is the same)
    if (cq < CB / MM_COPY_COLS && x0 + cq < X && d < D) ng[(size_t)(x0 + cq) * D + d] = n[i];
  }
  if (rg == 0 && cq < CB / MM_COPY_COLS && x0 + cq < X) mg[x0 + cq] = m;
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
#define MM_LAUNCH(RQ, TC)                                                                                                       \
  matrix_memory_scan_kernel<RQ, TC><<<dim3((Dv + MM_CB - 1) / MM_CB, H, n_reqs), MM_THREADS, 0, stream>>>(                      \
      proj, ldp, off_q, off_k, off_v, gates, state, state_stride, q_start, slots, o, ldo, H, D, Dv)
  if (D <= 64) MM_LAUNCH(4, 8);
  else if (D <= 128) MM_LAUNCH(8, 8);
  else MM_LAUNCH(16, 4);
#undef MM_LAUNCH
  FERRUM_CHECK_LAUNCH("matrix_memory_scan");
  return 0;
}
