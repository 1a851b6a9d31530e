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
//                    decays: dec[h][d] = exp(-exp(A_log[h]) * softplus(logit[h D + d] + dt_bias[h D + d])), and behind
//                    them beta[h] = sigmoid(its logit): a token's row of `dec` is [H D | H].
// delta_conv_state:  u <- the last taps - 1 inputs after this portion; a launch of its own, so that nobody reads u while
//                    it changes.
// delta_scan:        a block per (request, head, a group of value columns) walks the portion's tokens in order:
//                      S <- dec * S (row d by dec[d]);  e = beta * (v - S^T k);  S <- S + k e^T;  o = S^T q
//                    (o is formed as S^T q of the decayed S plus e (k . q), so that both sums over the rows and k . q
//                    cross the lanes side by side)
//                    with beta = sigmoid(its logit).  Four lanes share a column (a quarter of the rows each, summed in
//                    row order) and add their parts by two shuffles: one fixed tree, token by token whatever the
//                    portion, so a token's result does not depend on how the sequence was cut.
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
  if (slot >= 2 * G + H) {                                  // a head's decays, and its beta behind all heads' decays
    const int h = slot - 2 * G - H;
    const float rate = expf(a_log[h]);
    float* row = dec + (size_t)t * (H * D + H);
    for (int d = lane; d < D; d += 32) {
      const int c = h * D + d;
      row[c] = expf(-rate * dr_softplus(logit[(size_t)t * ldl + c] + dt_bias[c]));
    }
    if (lane == 0) row[H * D + h] = 1.f / (1.f + expf(-proj[(size_t)t * ldp + C + h]));
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

__device__ __forceinline__ void dr_cp_async4(float* smem, const float* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void dr_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void dr_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void dr_cp_async16(float* smem, const float* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}

// The walk for steps of single tokens (a few tokens a request).  Four lanes share a value column: lane q of them holds the rows d = q RQ .. q RQ + RQ - 1 (D <= 4 RQ) of C neighbouring
// columns in registers, and a block of 64 threads walks 16 C columns.  What bounds such a walk is the path between shared
// memory and the registers, which a 16-byte read and a shuffle each occupy for four cycles per warp: so a lane keeps many
// rows (two shuffle levels per sum instead of four), every k, q and decay it reads serves its C columns, and k stays in
// registers between the two halves of a token's step.  TC tokens are staged at a time (a quarter's rows 16 bytes apart from
// the next quarter's, so that the quarters' reads fall into different banks), the next chunk on its way meanwhile by
// cp.async straight to its place (16 bytes a copy where the rows allow; loads into registers that were still pending held
// up the walk's own shared-memory reads); a chunk's read-outs leave together after its walk.  Its reads and writes of the
// state are whole 64-byte pieces of a row per warp, which is what a step of single tokens consists of; over a prompt its one
// or two warps a block run a token's long rows slower than the kernel below (measured: 1,030 against 600 us for 2,048 tokens).
template <int RQ, int C, int TC>
__global__ void __launch_bounds__(64)
delta_scan_rows_kernel(const float* __restrict__ qkv, int Cw, const float* __restrict__ dec, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ o,
                  int ldo, int H, int G, int D, int Dv, int vec) {
  constexpr int NT = 64, QS = RQ + 4, W = 4 * QS, WD = 4 * RQ, CB = (NT / 4) * C;
  static_assert(RQ % 4 == 0 && TC <= NT, "rows are read four at a time");
  __shared__ __align__(16) float sq[2][TC][W], sk[2][TC][W], sg[2][TC][W];
  __shared__ float sv[2][TC][CB], sb[2][TC], so[2][TC][CB];
  const int tid = threadIdx.x, q = tid & 3, cp = tid >> 2;
  const int jb = blockIdx.x * CB, j0 = jb + cp * C, h = blockIdx.y, r = blockIdx.z;
  const int g = h / (H / G);
  const int t0 = q_start[r], t1 = q_start[r + 1];
  const int ldd = H * D + H;
  float* Sg = state + (long long)slots[r] * state_stride + (size_t)h * D * Dv;
  const int off_q = g * D, off_k = G * D + g * D, off_v = 2 * G * D + h * Dv + jb;
  auto stage = [&](int c0, int b) {              // a chunk's elements on their way into buffer b
    const int nt = min(TC, t1 - c0);
    if (vec) {                                   // rows of whole 16-byte groups: a copy brings four rows
      for (int idx = tid; idx < TC * 3 * (WD / 4); idx += NT) {
        const int which = idx / (TC * (WD / 4)), tk = (idx / (WD / 4)) % TC, d = (idx % (WD / 4)) * 4;
        float* dst = (which == 0 ? &sq[b][tk][0] : (which == 1 ? &sk[b][tk][0] : &sg[b][tk][0])) + (d / RQ) * QS + d % RQ;
        if (tk < nt && d < D) {
          const size_t row = (size_t)(c0 + tk);
          dr_cp_async16(dst, which == 0 ? qkv + row * Cw + off_q + d : (which == 1 ? qkv + row * Cw + off_k + d : dec + row * ldd + (size_t)h * D + d));
        } else {
          const float fill = which == 2 ? 1.f : 0.f;
          *reinterpret_cast<float4*>(dst) = make_float4(fill, fill, fill, fill);
        }
      }
    } else {
      for (int idx = tid; idx < TC * 3 * WD; idx += NT) {
        const int which = idx / (TC * WD), tk = (idx / WD) % TC, d = idx % WD;
        float* dst = (which == 0 ? &sq[b][tk][0] : (which == 1 ? &sk[b][tk][0] : &sg[b][tk][0])) + (d / RQ) * QS + d % RQ;
        if (tk < nt && d < D) {
          const size_t row = (size_t)(c0 + tk);
          dr_cp_async4(dst, which == 0 ? qkv + row * Cw + off_q + d : (which == 1 ? qkv + row * Cw + off_k + d : dec + row * ldd + (size_t)h * D + d));
        } else {
          *dst = which == 2 ? 1.f : 0.f;
        }
      }
    }
    for (int idx = tid; idx < TC * CB; idx += NT) {
      const int tk = idx / CB, c = idx % CB;
      if (tk < nt && jb + c < Dv) dr_cp_async4(&sv[b][tk][c], qkv + (size_t)(c0 + tk) * Cw + off_v + c);
      else sv[b][tk][c] = 0.f;
    }
    if (tid < nt) dr_cp_async4(&sb[b][tid], dec + (size_t)(c0 + tid) * ldd + H * D + h);
    dr_cp_async_commit();
  };
  if (t0 < t1) stage(t0, 0);
  float S[C][RQ];
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = q * RQ + i;
#pragma unroll
    for (int c = 0; c < C; ++c) S[c][i] = (d < D && j0 + c < Dv) ? Sg[(size_t)d * Dv + j0 + c] : 0.f;
  }
  dr_cp_async_wait_all();
  __syncthreads();
  int b = 0;
  for (int c0 = t0; c0 < t1; c0 += TC, b ^= 1) {
    const int nt = min(TC, t1 - c0);
    if (c0 + TC < t1) stage(c0 + TC, b ^ 1);     // (that buffer was last read before the barrier that ended the chunk before)
    for (int tk = 0; tk < nt; ++tk) {
      const float4* g4 = reinterpret_cast<const float4*>(&sg[b][tk][q * QS]);
      const float4* k4 = reinterpret_cast<const float4*>(&sk[b][tk][q * QS]);
      const float4* q4 = reinterpret_cast<const float4*>(&sq[b][tk][q * QS]);
      const float beta = sb[b][tk];
      float vj[C], part[C], po[C], kq = 0.f, kr[RQ];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        vj[c] = sv[b][tk][cp * C + c];
        part[c] = 0.f;
        po[c] = 0.f;
      }
      // The read-out sees the token's write: (S + k e^T)^T q = S^T q + e (k . q).  So S^T k, S^T q (both of the decayed S)
      // and k . q are summed across the lanes side by side, and one chain of shuffles serves the token.
#pragma unroll
      for (int i = 0; i < RQ / 4; ++i) {
        const float4 gg = g4[i], kk = k4[i], qq = q4[i];
        const float gv[4] = {gg.x, gg.y, gg.z, gg.w}, kv[4] = {kk.x, kk.y, kk.z, kk.w}, qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int x = 4 * i + e;
          kr[x] = kv[e];
          kq = fmaf(kv[e], qv[e], kq);
#pragma unroll
          for (int c = 0; c < C; ++c) {
            S[c][x] *= gv[e];
            part[c] = fmaf(S[c][x], kv[e], part[c]);
            po[c] = fmaf(S[c][x], qv[e], po[c]);
          }
        }
      }
#pragma unroll
      for (int off = 1; off < 4; off <<= 1) {
        float t1v[C], t2v[C];
#pragma unroll
        for (int c = 0; c < C; ++c) {
          t1v[c] = __shfl_xor_sync(0xffffffffu, part[c], off);
          t2v[c] = __shfl_xor_sync(0xffffffffu, po[c], off);
        }
        const float t3 = __shfl_xor_sync(0xffffffffu, kq, off);
#pragma unroll
        for (int c = 0; c < C; ++c) {
          part[c] += t1v[c];
          po[c] += t2v[c];
        }
        kq += t3;
      }
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const float e = beta * (vj[c] - part[c]);
        po[c] = fmaf(e, kq, po[c]);
#pragma unroll
        for (int x = 0; x < RQ; ++x) S[c][x] = fmaf(kr[x], e, S[c][x]);
        if (q == 0) so[b][tk][cp * C + c] = po[c];
      }
    }
    dr_cp_async_wait_all();
    __syncthreads();
    for (int idx = tid; idx < nt * CB; idx += NT) {      // (the next chunk's walk fills the other buffer; a barrier lies before this one is written again)
      const int tk = idx / CB, c = idx % CB;
      if (jb + c < Dv) o[(size_t)(c0 + tk) * ldo + (size_t)h * Dv + jb + c] = so[b][tk][c];
    }
  }
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = q * RQ + i;
#pragma unroll
    for (int c = 0; c < C; ++c)
      if (d < D && j0 + c < Dv) Sg[(size_t)d * Dv + j0 + c] = S[c][i];
  }
}

// The walk for portions of many tokens.  LPC lanes share a value column (D <= 8 LPC): lane q of them holds rows d = LPC i + q, i < 8, of the column in registers,
// and a block of 256 threads walks 256 / LPC columns.  TC tokens are staged at a time; a staged token row keeps the lanes'
// elements apart (lane q at 12 q + i, so that a lane reads its rows four at a time and the lanes' 16-byte reads spread over
// the banks).  The chunk after the one being walked is on its way meanwhile, element by element with cp.async straight to
// its place (loads into registers that were still pending held up the walk's own shared-memory reads and its stores); a
// token's operands are read one token ahead of their use.
template <int LPC, int TC>
__global__ void __launch_bounds__(256)
delta_scan_lanes_kernel(const float* __restrict__ qkv, int C, const float* __restrict__ dec, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ o,
                  int ldo, int H, int G, int D, int Dv) {
  constexpr int RQ = 8, QS = RQ + 4, W = LPC * QS, WD = LPC * RQ, CB = 256 / LPC;
  constexpr int LD = (TC * 3 * WD + 255) / 256;
  static_assert(TC * CB <= 256 && TC <= 256, "one copy a thread brings a chunk's values");
  __shared__ __align__(16) float sq[2][TC + 1][W], sk[2][TC + 1][W], sg[2][TC + 1][W];      // (one row more: the walk reads a token ahead)
  __shared__ float sv[2][TC][CB], sb[2][TC], so[2][TC][CB];    // (so: a chunk's read-outs, written out together after its walk)
  const int tid = threadIdx.x, col = tid / LPC, q = tid % LPC;
  const int j = blockIdx.x * CB + col, h = blockIdx.y, r = blockIdx.z;
  const int g = h / (H / G);
  const int t0 = q_start[r], t1 = q_start[r + 1];
  const int ldd = H * D + H;
  float* Sg = state + (long long)slots[r] * state_stride + (size_t)h * D * Dv;
  const int off_q = g * D, off_k = G * D + g * D, off_v = 2 * G * D + h * Dv + blockIdx.x * CB;
  auto stage = [&](int c0, int b) {              // a chunk's elements on their way into buffer b
    const int nt = min(TC, t1 - c0);
#pragma unroll
    for (int it = 0; it < LD; ++it) {
      const int idx = tid + it * 256;
      const int which = idx / (TC * WD), tk = (idx / WD) % TC, d = idx % WD;
      if (idx < TC * 3 * WD) {
        float* dst = (which == 0 ? &sq[b][tk][0] : (which == 1 ? &sk[b][tk][0] : &sg[b][tk][0])) + (d % LPC) * QS + d / LPC;
        if (tk < nt && d < D) {
          const size_t row = (size_t)(c0 + tk);
          dr_cp_async4(dst, which == 0 ? qkv + row * C + off_q + d : (which == 1 ? qkv + row * C + off_k + d : dec + row * ldd + (size_t)h * D + d));
        } else {
          *dst = which == 2 ? 1.f : 0.f;
        }
      }
    }
    if (tid < TC * CB) {
      const int tk = tid / CB, c = tid % CB;
      if (tk < nt && blockIdx.x * CB + c < Dv) dr_cp_async4(&sv[b][tk][c], qkv + (size_t)(c0 + tk) * C + off_v + c);
      else sv[b][tk][c] = 0.f;
    }
    if (tid < nt) dr_cp_async4(&sb[b][tid], dec + (size_t)(c0 + tid) * ldd + H * D + h);
    dr_cp_async_commit();
  };
  if (t0 < t1) stage(t0, 0);
  float S[RQ];
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = LPC * i + q;
    S[i] = (d < D && j < Dv) ? Sg[(size_t)d * Dv + j] : 0.f;
  }
  dr_cp_async_wait_all();
  __syncthreads();
  int b = 0;
  for (int c0 = t0; c0 < t1; c0 += TC, b ^= 1) {
    const int nt = min(TC, t1 - c0);
    if (c0 + TC < t1) stage(c0 + TC, b ^ 1);     // (that buffer was last read before the barrier that ended the chunk before)
    const float4* g4 = reinterpret_cast<const float4*>(&sg[b][0][q * QS]);
    const float4* k4 = reinterpret_cast<const float4*>(&sk[b][0][q * QS]);
    const float4* q4 = reinterpret_cast<const float4*>(&sq[b][0][q * QS]);
    float4 ga = g4[0], gb = g4[1], ka = k4[0], kb = k4[1], qa = q4[0], qb = q4[1];
    float beta = sb[b][0], vj = sv[b][0][col];
    for (int tk = 0; tk < nt; ++tk) {
      // the next token's operands (past the chunk's last token: the spare row, never used)
      const int nx = (tk + 1) * (W / 4);
      const float4 ga2 = g4[nx], gb2 = g4[nx + 1], ka2 = k4[nx], kb2 = k4[nx + 1], qa2 = q4[nx], qb2 = q4[nx + 1];
      const float beta2 = sb[b][min(tk + 1, TC - 1)], vj2 = sv[b][min(tk + 1, TC - 1)][col];
      // The read-out sees the token's write: (S + k e^T)^T q = S^T q + e (k . q).  So S^T k, S^T q (both of the decayed S)
      // and k . q are summed across the lanes side by side, and one chain of shuffles serves the token.
      float kq = (fmaf(kb.x, qb.x, ka.x * qa.x) + fmaf(kb.y, qb.y, ka.y * qa.y)) + (fmaf(kb.z, qb.z, ka.z * qa.z) + fmaf(kb.w, qb.w, ka.w * qa.w));
      S[0] *= ga.x; S[1] *= ga.y; S[2] *= ga.z; S[3] *= ga.w;
      S[4] *= gb.x; S[5] *= gb.y; S[6] *= gb.z; S[7] *= gb.w;
      float part = (fmaf(S[4], kb.x, S[0] * ka.x) + fmaf(S[5], kb.y, S[1] * ka.y)) + (fmaf(S[6], kb.z, S[2] * ka.z) + fmaf(S[7], kb.w, S[3] * ka.w));
      float po = (fmaf(S[4], qb.x, S[0] * qa.x) + fmaf(S[5], qb.y, S[1] * qa.y)) + (fmaf(S[6], qb.z, S[2] * qa.z) + fmaf(S[7], qb.w, S[3] * qa.w));
#pragma unroll
      for (int off = 1; off < LPC; off <<= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, part, off), o2 = __shfl_xor_sync(0xffffffffu, po, off);
        const float o3 = __shfl_xor_sync(0xffffffffu, kq, off);
        part += o1;
        po += o2;
        kq += o3;
      }
      const float e = beta * (vj - part);
      po = fmaf(e, kq, po);
      S[0] = fmaf(ka.x, e, S[0]); S[1] = fmaf(ka.y, e, S[1]); S[2] = fmaf(ka.z, e, S[2]); S[3] = fmaf(ka.w, e, S[3]);
      S[4] = fmaf(kb.x, e, S[4]); S[5] = fmaf(kb.y, e, S[5]); S[6] = fmaf(kb.z, e, S[6]); S[7] = fmaf(kb.w, e, S[7]);
      if (q == 0) so[b][tk][col] = po;
      ga = ga2; gb = gb2; ka = ka2; kb = kb2; qa = qa2; qb = qb2;
      beta = beta2; vj = vj2;
    }
    dr_cp_async_wait_all();
    __syncthreads();
    if (tid < nt * CB) {                         // (the next chunk's walk fills the other buffer; a barrier lies before this one is written again)
      const int tk = tid / CB, c = tid % CB;
      if (blockIdx.x * CB + c < Dv) o[(size_t)(c0 + tk) * ldo + (size_t)h * Dv + blockIdx.x * CB + c] = so[b][tk][c];
    }
  }
#pragma unroll
  for (int i = 0; i < RQ; ++i) {
    const int d = LPC * i + q;
    if (d < D && j < Dv) Sg[(size_t)d * Dv + j] = S[i];
  }
}

constexpr int DR_MAX_D = 256;
constexpr int DR_ROWS_MAX_TOKENS = 4;     // the longest portion of a step that still takes the single-token walk

// proj: float32 rows [q | k | v | beta logits] of stride ldp; logit: float32 rows [H * D] of stride ldl (the decays' logits);
// conv_w: [C][taps]; state: [slots][state_stride] float32 rows, S first and the convolution's inputs from H * D * Dv on;
// qkv [T][C] and dec [T][H * D + H]: float32 scratch; o: float32 [T][ldo] receives the heads' read-outs [H * Dv].
FERRUM_API int ferrum_delta_rule(const float* proj, int ldp, const float* logit, int ldl, int n_tokens, int n_reqs,
                                 const int* req_of_token, const int* q_start, const int* slots, const float* conv_w, int taps,
                                 const float* dt_bias, const float* a_log, int H, int G, int D, int Dv, float* state,
                                 long long state_stride, float* qkv, float* dec, float* o, int ldo, int max_q_len, cudaStream_t stream) {
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
  if (max_q_len > DR_ROWS_MAX_TOKENS) {
#define DR_LAUNCH_LANES(LPC, TC)                                                                                               \
  delta_scan_lanes_kernel<LPC, TC><<<dim3((Dv + 256 / LPC - 1) / (256 / LPC), H, n_reqs), 256, 0, stream>>>(                  \
      qkv, C, dec, state, state_stride, q_start, slots, o, ldo, H, G, D, Dv)
    if (D <= 32) DR_LAUNCH_LANES(4, 4);
    else if (D <= 64) DR_LAUNCH_LANES(8, 8);
    else if (D <= 128) DR_LAUNCH_LANES(16, 8);
    else DR_LAUNCH_LANES(32, 4);
#undef DR_LAUNCH_LANES
    FERRUM_CHECK_LAUNCH("delta_scan");
    return 0;
  }
  // whole 16-byte groups of rows in every staged array, on 16-byte borders
  const int vec = D % 4 == 0 && C % 4 == 0 && (H * D + H) % 4 == 0 && (G * D) % 4 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)dec & 15) == 0;
  // one column a thread while that still leaves blocks for every SM to spare (a prompt of one request), else two
  const bool wide = (long long)((Dv + 15) / 16) * H * n_reqs > 160;
#define DR_LAUNCH(RQ, CC, TC)                                                                                                  \
  delta_scan_rows_kernel<RQ, CC, TC><<<dim3((Dv + 16 * CC - 1) / (16 * CC), H, n_reqs), 64, 0, stream>>>(                           \
      qkv, C, dec, state, state_stride, q_start, slots, o, ldo, H, G, D, Dv, vec)
  if (D <= 32) { if (wide) DR_LAUNCH(8, 2, 16); else DR_LAUNCH(8, 1, 16); }
  else if (D <= 64) { if (wide) DR_LAUNCH(16, 2, 16); else DR_LAUNCH(16, 1, 16); }
  else if (D <= 128) { if (wide) DR_LAUNCH(32, 2, 8); else DR_LAUNCH(32, 1, 8); }
  else DR_LAUNCH(64, 1, 4);
#undef DR_LAUNCH
  FERRUM_CHECK_LAUNCH("delta_scan");
  return 0;
}
