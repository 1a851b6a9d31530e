// What surrounds the attention kernel for mixers whose heads are shaped before and after it:
//
// qkv_shape: reads one float32 row per token [q heads | k heads | v heads | ...] as a product left
// it, and per head, in float32, in this order: adds the projection's bias; divides a query or key head
// by its root mean square and multiplies by a weight vector shared by all heads (`qnorm_w`, `knorm_w`), or
// (`whole_norm`) divides it by the root mean square of the token's WHOLE query (key) projection, all heads at
// once, and multiplies by a weight vector as long as that projection;
// turns the leading `rope_dim` elements of a query or key head by the token's position (table of
// cos/sin per position and pair; pairs (i, i + rope_dim/2) or (2i, 2i+1)); then, when asked, divides
// the whole head by its root mean square (no weight); multiplies a query head by a temperature of its
// position, 1 + coef * ln(floor((pos + 1) / every) + 1); turns a value head over all of its elements
// by a table of its own; blends a value head with the same token's value head of an earlier layer,
// (1 - lambda) v + lambda v_first (`vmix_mode` 2), or leaves its own there for later layers (1).
// Queries go out in the compute type [T, Hq, Dp], keys and values go to the token's place in the
// paged cache (rows of Dp elements, zero past the head's own size: Dp = max(key size, value size)
// lets one page layout hold both).  With `v_from_k` the row has no value heads: the value of a KV head is
// its key head as the product left it (before bias-free norm and turn), of the key's size.
//
// attention_finish: reads the attention's float32 output [T, Hq, Dp]; turns each head back by the
// query's position (the inverse of the value rotation), multiplies by a sigmoid gate whose logits lie
// in the product's row, and writes [T, Hq, Dv] in the compute type for the output projection.
//
// One warp per (token, head).  Every step of a head is float32; the only rounding is the store.
#include "common.cuh"

constexpr int AP_WARPS = 4;
constexpr int AP_MAX_D = 256;

// What a head may need beyond rotation and unit norm; every pointer may be null.
struct HeadExtras {
  const float* bias;        // [Hq*Dk + Hkv*Dk + Hkv*Dv], laid out like the product's row
  const float* qnorm_w;     // [Dk]
  const float* knorm_w;     // [Dk]
  float qtemp_coef;
  int qtemp_every;          // 0: no temperature
  int vmix_mode;            // 0: none; 1: leave this layer's values in v_first; 2: blend with v_first
  float* v_first;           // [T, ld_first] float32
  int ld_first;
  const float* v_lambda;    // one float on the device
  int whole_norm;           // 1: qnorm_w is [Hq*Dk], knorm_w [Hkv*Dk], and the mean square runs over the whole projection
  int v_from_k;             // 1: the row is [q heads | k heads]; value head g is key head g as projected
};

template <typename T>
__global__ void __launch_bounds__(AP_WARPS * 32)
qkv_shape_kernel(const float* __restrict__ proj, int ldp, int n_tokens, const int* __restrict__ positions,
                 const int* __restrict__ req_of_token, const int* __restrict__ block_table, int table_width,
                 const float* __restrict__ cs_qk, int rope_dim, int qk_pairing, int n_pos_qk,
                 const float* __restrict__ cs_v, int v_pairing, int n_pos_v, int unit_norm, float eps,
                 T* __restrict__ q_out, int ldq, T* __restrict__ plane, long long page_stride, int page_size,
                 int Hq, int Hkv, int Dk, int Dv, int Dp, int writes, int* __restrict__ err, const HeadExtras x) {
  __shared__ float rows[AP_WARPS][AP_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = Hq + (writes ? 2 * Hkv : 0);
  const long long item = (long long)blockIdx.x * AP_WARPS + warp;
  if (item >= (long long)n_tokens * slots) return;
  const int t = (int)(item / slots), slot = (int)(item % slots);
  const int pos = positions[t];
  float* const row = rows[warp];
  const bool is_v = slot >= Hq + Hkv;
  const int D = is_v ? Dv : Dk;
  const int src_off = slot < Hq ? slot * Dk : (slot < Hq + Hkv ? Hq * Dk + (slot - Hq) * Dk :
                      (x.v_from_k ? Hq * Dk + (slot - Hq - Hkv) * Dk : (Hq + Hkv) * Dk + (slot - Hq - Hkv) * Dv));
  const float* src = proj + (size_t)t * ldp + src_off;
  if (x.bias != nullptr) {
    for (int d = lane; d < D; d += 32) row[d] = src[d] + x.bias[src_off + d];
  } else {
    for (int d = lane; d < D; d += 32) row[d] = src[d];
  }
  __syncwarp();
  const float* nw = is_v ? nullptr : (slot < Hq ? x.qnorm_w : x.knorm_w);
  if (nw != nullptr && x.whole_norm) {       // RMS norm over all heads of the projection at once, before any turn
    const int first = slot < Hq ? 0 : Hq * Dk, n = (slot < Hq ? Hq : Hkv) * Dk, head = slot < Hq ? slot : slot - Hq;
    const float* all = proj + (size_t)t * ldp + first;
    float ss = 0.f;
    for (int d = lane; d < n; d += 32) {
      const float v = all[d] + (x.bias != nullptr ? x.bias[first + d] : 0.f);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)n + eps);
    for (int d = lane; d < D; d += 32) row[d] = row[d] * r * nw[head * Dk + d];
    __syncwarp();
  } else if (nw != nullptr) {                // weighted RMS norm of the head, before any turn
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss = fmaf(row[d], row[d], ss);
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)D + eps);
    for (int d = lane; d < D; d += 32) row[d] = row[d] * r * nw[d];
    __syncwarp();
  }
  const float* cs = is_v ? cs_v : cs_qk;
  const int R = is_v ? Dv : rope_dim;
  const int pairing = is_v ? v_pairing : qk_pairing;
  if (cs != nullptr && R > 0) {
    if (pos < 0 || pos >= (is_v ? n_pos_v : n_pos_qk)) {
      if (lane == 0) atomicExch(err, 2);
    } else {
      const float2* tab = reinterpret_cast<const float2*>(cs) + (size_t)pos * (R / 2);
      for (int i = lane; i < R / 2; i += 32) {
        const int a = pairing == 1 ? i : 2 * i, b = pairing == 1 ? i + R / 2 : 2 * i + 1;
        const float2 c = tab[i];
        const float u = row[a], v = row[b];
        row[a] = u * c.x - v * c.y;
        row[b] = v * c.x + u * c.y;
      }
      __syncwarp();
    }
  }
  float mult = 1.f;
  if (unit_norm && !is_v) {
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss = fmaf(row[d], row[d], ss);
    ss = warp_sum(ss);
    mult = 1.f / sqrtf(ss / (float)D + eps);
  }
  if (slot < Hq && x.qtemp_every > 0) mult *= 1.f + x.qtemp_coef * logf((float)((pos + 1) / x.qtemp_every + 1));
  if (is_v && x.vmix_mode != 0) {
    float* first = x.v_first + (size_t)t * x.ld_first + (size_t)(slot - Hq - Hkv) * Dv;
    if (x.vmix_mode == 1) {
      for (int d = lane; d < D; d += 32) first[d] = row[d];
    } else {
      const float lam = *x.v_lambda;
      for (int d = lane; d < D; d += 32) row[d] = (1.f - lam) * row[d] + lam * first[d];
    }
    __syncwarp();
  }
  T* dst;
  if (slot < Hq) {
    dst = q_out + (size_t)t * ldq + (size_t)slot * Dp;
  } else {
    const int kvh = is_v ? slot - Hq - Hkv : slot - Hq;
    const int lp = pos / page_size;
    const int page = (pos >= 0 && lp < table_width) ? block_table[(size_t)req_of_token[t] * table_width + lp] : -1;
    if (page < 0) {
      if (lane == 0) atomicExch(err, pos >= 0 && lp < table_width ? 4 : 3);
      return;
    }
    dst = plane + (long long)page * page_stride + ((long long)((is_v ? Hkv : 0) + kvh) * page_size + pos % page_size) * Dp;
  }
  for (int d = lane; d < Dp; d += 32) dst[d] = from_f32<T>(d < D ? row[d] * mult : 0.f);
}

template <typename T>
__global__ void __launch_bounds__(AP_WARPS * 32)
attention_finish_kernel(const float* __restrict__ o, int ldo, int n_tokens, const int* __restrict__ positions,
                        const float* __restrict__ cs_v, int v_pairing, int n_pos_v, const float* __restrict__ gate,
                        int ldg, T* __restrict__ out, int ldout, int Hq, int Dv, int Dp, int* __restrict__ err) {
  pdl_launch();      // the product that follows may fetch its weights meanwhile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * AP_WARPS + warp;
  if (item >= (long long)n_tokens * Hq) return;
  const int t = (int)(item / Hq), h = (int)(item % Hq);
  const float* src = o + (size_t)t * ldo + (size_t)h * Dp;
  const float* g = gate != nullptr ? gate + (size_t)t * ldg + (size_t)h * Dv : nullptr;
  T* dst = out + (size_t)t * ldout + (size_t)h * Dv;
  const int pos = positions[t];
  if (cs_v != nullptr) {
    if (pos < 0 || pos >= n_pos_v) {
      if (lane == 0) atomicExch(err, 2);
      return;
    }
    const float2* tab = reinterpret_cast<const float2*>(cs_v) + (size_t)pos * (Dv / 2);
    for (int i = lane; i < Dv / 2; i += 32) {
      const int a = v_pairing == 1 ? i : 2 * i, b = v_pairing == 1 ? i + Dv / 2 : 2 * i + 1;
      const float2 c = tab[i];
      const float u = src[a], v = src[b];
      float ra = u * c.x + v * c.y, rb = v * c.x - u * c.y;      // the turn by minus the angle
      if (g != nullptr) {
        ra *= 1.f / (1.f + expf(-g[a]));
        rb *= 1.f / (1.f + expf(-g[b]));
      }
      dst[a] = from_f32<T>(ra);
      dst[b] = from_f32<T>(rb);
    }
  } else {
    for (int d = lane; d < Dv; d += 32) {
      float r = src[d];
      if (g != nullptr) r *= 1.f / (1.f + expf(-g[d]));
      dst[d] = from_f32<T>(r);
    }
  }
}

FERRUM_API int ferrum_qkv_shape(const float* proj, int ldp, int n_tokens, const int* positions, const int* req_of_token,
                                const int* block_table, int table_width, const float* cs_qk, int rope_dim, int qk_pairing,
                                int n_pos_qk, const float* cs_v, int v_pairing, int n_pos_v, int unit_norm, float eps,
                                void* q_out, int ldq, void* plane, long long page_stride, int page_size, int dtype, int Hq,
                                int Hkv, int Dk, int Dv, int Dp, int writes, int* err, const float* bias,
                                const float* qnorm_w, const float* knorm_w, float qtemp_coef, int qtemp_every,
                                int vmix_mode, float* v_first, int ld_first, const float* v_lambda, int whole_norm, int v_from_k,
                                cudaStream_t stream) {
  FERRUM_CHECK_ARG(Hq > 0 && Hkv > 0 && Dk > 0 && Dv > 0 && Dp >= Dk && Dp >= Dv && Dp <= AP_MAX_D,
                   "qkv_shape: bad head sizes Dk=%d Dv=%d Dp=%d", Dk, Dv, Dp);
  FERRUM_CHECK_ARG(rope_dim >= 0 && rope_dim <= Dk && rope_dim % 2 == 0, "qkv_shape: bad rotary size %d", rope_dim);
  FERRUM_CHECK_ARG(cs_v == nullptr || Dv % 2 == 0, "qkv_shape: a rotated value needs an even size");
  FERRUM_CHECK_ARG(page_size > 0 && table_width > 0, "qkv_shape: bad cache arguments");
  FERRUM_CHECK_ARG(qtemp_every >= 0 && vmix_mode >= 0 && vmix_mode <= 2, "qkv_shape: bad temperature or value-mix arguments");
  FERRUM_CHECK_ARG(vmix_mode == 0 || (v_first != nullptr && ld_first >= Hkv * Dv && (vmix_mode == 1 || v_lambda != nullptr)),
                   "qkv_shape: value mixing needs the first layer's values and a blend factor");
  if (n_tokens == 0) return 0;
  FERRUM_CHECK_ARG(!v_from_k || (Dv == Dk && bias == nullptr && cs_v == nullptr && vmix_mode == 0),
                   "qkv_shape: values taken from the keys have the keys' size, no bias, no turn and no blend");
  const HeadExtras extras{bias, qnorm_w, knorm_w, qtemp_coef, qtemp_every, vmix_mode, v_first, ld_first, v_lambda, whole_norm, v_from_k};
  const long long items = (long long)n_tokens * (Hq + (writes ? 2 * Hkv : 0));
  const long long blocks = (items + AP_WARPS - 1) / AP_WARPS;
  FERRUM_CHECK_ARG(blocks < (1LL << 31), "qkv_shape: too many rows");
  FERRUM_DISPATCH_DTYPE(dtype, T, (qkv_shape_kernel<T><<<(unsigned)blocks, AP_WARPS * 32, 0, stream>>>(
      proj, ldp, n_tokens, positions, req_of_token, block_table, table_width, cs_qk, rope_dim, qk_pairing, n_pos_qk, cs_v,
      v_pairing, n_pos_v, unit_norm, eps, (T*)q_out, ldq, (T*)plane, page_stride, page_size, Hq, Hkv, Dk, Dv, Dp, writes,
      err, extras)));
  FERRUM_CHECK_LAUNCH("qkv_shape");
  return 0;
}

FERRUM_API int ferrum_attention_finish(const float* o, int ldo, int n_tokens, const int* positions, const float* cs_v,
                                       int v_pairing, int n_pos_v, const float* gate, int ldg, void* out, int ldout,
                                       int dtype, int Hq, int Dv, int Dp, int* err, cudaStream_t stream) {
  FERRUM_CHECK_ARG(Hq > 0 && Dv > 0 && Dp >= Dv, "attention_finish: bad head sizes Dv=%d Dp=%d", Dv, Dp);
  FERRUM_CHECK_ARG(cs_v == nullptr || Dv % 2 == 0, "attention_finish: a rotated value needs an even size");
  if (n_tokens == 0) return 0;
  const long long blocks = ((long long)n_tokens * Hq + AP_WARPS - 1) / AP_WARPS;
  FERRUM_CHECK_ARG(blocks < (1LL << 31), "attention_finish: too many rows");
  FERRUM_DISPATCH_DTYPE(dtype, T, (attention_finish_kernel<T><<<(unsigned)blocks, AP_WARPS * 32, 0, stream>>>(
      o, ldo, n_tokens, positions, cs_v, v_pairing, n_pos_v, gate, ldg, (T*)out, ldout, Hq, Dv, Dp, err)));
  FERRUM_CHECK_LAUNCH("attention_finish");
  return 0;
}
