// Several copies of the residual stream ("streams") around every sublayer, float32 throughout.
//
// A model with S streams keeps X[t][s][:] (s < S, rows of E floats, a token's S rows next to each
// other).  A sublayer with the small tensors a [S], M [S][S] (indexed [from][to]) and b [S] reads
//     u = sum_s a[s] X[s]                        and feeds  rms(u) * w  to its mixer or feed-forward,
// and its result y goes back as
//     X'[t] = sum_s M[s][t] X[s] + b[t] y        for all t at once, from the old rows.
// One kernel does both ends: it first applies the WRITE of the sublayer before it (whose y arrives as
// a float32 buffer, as a product left in partials, or as `top` rows per token to be added in order:
// the results of a token's chosen experts), stores the new rows, and then makes the READ and the RMS
// norm of the sublayer that follows from the rows it still holds.  Either half may be absent: the
// first sublayer of a model only reads, a flush only writes.  With `rows` the kernel works on the
// listed tokens only and stores nothing (the last read of a model: the plain sum of the streams of
// the rows whose logits are wanted, a == null).
//
// One block per token; a thread walks elements e = tid, tid + 256, ... (four consecutive ones at a time, with 16-byte
// accesses, when the rows allow it and the kernel is built for the number of streams); u stays in shared memory
// between the sum of squares and the scaling.  Sums over s run in ascending order, the block's
// reduction tree is fixed: a token's result does not depend on the batch.
#include "common.cuh"
#include "partials.cuh"

constexpr int HC_MAX_STREAMS = 8;
constexpr int HC_THREADS = 256;

struct HyperWrite {
  const float* y;          // [T][ldy] float32, or null
  int ldy;
  const int* y_rows;       // [T][top] rows of y to add up for a token, or null (row t itself)
  int top;
  const float* mix;        // [S][S], [from][to]
  const float* out;        // [S]
};

// V: consecutive elements a thread handles at once (4: rows of X, y and out start on 16-byte boundaries and E is a
// multiple of 4, so that a thread's loads are 16 bytes wide and S + 1 of them are in flight before the arithmetic).
// SC: the number of streams when the kernel is built for one (its loops and registers are then exactly that many), else 0.
template <typename TOut, int V, int SC>
__global__ void __launch_bounds__(HC_THREADS)
hyper_step_kernel(float* __restrict__ X, int S_any, int E, const int* __restrict__ rows, const HyperWrite w, const PartialLayout L,
                  int has_write, int store, const float* __restrict__ in_w, const float* __restrict__ norm_w, float eps,
                  TOut* __restrict__ out) {
  constexpr int SM = SC > 0 ? SC : HC_MAX_STREAMS;
  const int S = SC > 0 ? SC : S_any;
  extern __shared__ __align__(16) float hc_u[];      // E floats
  __shared__ float red[32];
  __shared__ float sm_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], sm_out[HC_MAX_STREAMS], sm_in[HC_MAX_STREAMS];
  __shared__ PartialTable tab;
  if (L.ws != nullptr) build_partial_table(L, tab);  // shapes only
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int t = rows != nullptr ? rows[r] : r;
  if (threadIdx.x < S * S && has_write) sm_mix[threadIdx.x] = w.mix[threadIdx.x];
  if (threadIdx.x < S) {
    if (has_write) sm_out[threadIdx.x] = w.out[threadIdx.x];
    sm_in[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float* xt = X + (size_t)t * S * E;
  float ss = 0.f;
  for (int e = threadIdx.x * V; e < E; e += HC_THREADS * V) {
    float x[SM][V];
#pragma unroll
    for (int s = 0; s < SM; ++s) {
      if (V == 4) {
        const float4 v = s < S ? *reinterpret_cast<const float4*>(xt + (size_t)s * E + e) : make_float4(0.f, 0.f, 0.f, 0.f);
        x[s][0] = v.x; x[s][1] = v.y; x[s][2 % V] = v.z; x[s][3 % V] = v.w;
      } else {
        x[s][0] = s < S ? xt[(size_t)s * E + e] : 0.f;
      }
    }
    if (has_write) {
      float y[V];
      if (L.ws != nullptr) {
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = partial_sum(L, tab, t, e + i);
      } else if (w.y_rows != nullptr) {
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = 0.f;
        for (int j = 0; j < w.top; ++j) {
          const float* src = w.y + (size_t)w.y_rows[(size_t)t * w.top + j] * w.ldy + e;
          if (V == 4) {
            const float4 v = *reinterpret_cast<const float4*>(src);
            y[0] += v.x; y[1 % V] += v.y; y[2 % V] += v.z; y[3 % V] += v.w;
          } else {
            y[0] += src[0];
          }
        }
      } else {
        const float* src = w.y + (size_t)t * w.ldy + e;
        if (V == 4) {
          const float4 v = *reinterpret_cast<const float4*>(src);
          y[0] = v.x; y[1 % V] = v.y; y[2 % V] = v.z; y[3 % V] = v.w;
        } else {
          y[0] = src[0];
        }
      }
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float nx[SM];
#pragma unroll
        for (int d = 0; d < SM; ++d) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < SM; ++s)
            if (s < S && d < S) acc = fmaf(sm_mix[s * S + d], x[s][i], acc);
          nx[d] = d < S ? fmaf(sm_out[d], y[i], acc) : 0.f;
        }
#pragma unroll
        for (int s = 0; s < SM; ++s) x[s][i] = nx[s];
      }
      if (store) {
#pragma unroll
        for (int s = 0; s < SM; ++s) {
          if (s < S) {
            if (V == 4) *reinterpret_cast<float4*>(xt + (size_t)s * E + e) = make_float4(x[s][0], x[s][1 % V], x[s][2 % V], x[s][3 % V]);
            else xt[(size_t)s * E + e] = x[s][0];
          }
        }
      }
    }
    if (out != nullptr) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < SM; ++s)
          if (s < S) u = fmaf(sm_in[s], x[s][i], u);
        hc_u[e + i] = u;
        ss = fmaf(u, u, ss);
      }
    }
  }
  if (out == nullptr) return;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)E + eps);
  TOut* o = out + (size_t)r * E;
  for (int e = threadIdx.x; e < E; e += HC_THREADS) o[e] = from_f32<TOut>(hc_u[e] * inv * norm_w[e]);
}

FERRUM_API int ferrum_hyper_max_streams() { return HC_MAX_STREAMS; }

// X: [tokens][S][E] float32.  rows (n_rows entries) or null (rows 0 .. n_rows-1).
// The write half runs when mix != null: y (float32 rows of ldy floats; with y_rows, `top` of them are
// summed per token) or partials + layout.  store: the new rows go back to X (0 with `rows`).
// The read half runs when out != null: in_w [S] or null (all ones), norm_w [E], out [n_rows][E] of out_dtype.
FERRUM_API int ferrum_hyper_step(float* X, int S, int E, const int* rows, int n_rows, const float* y, int ldy, const int* y_rows,
                                 int top, const float* partials, const int* layout, const float* mix, const float* out_w,
                                 int store, const float* in_w, const float* norm_w, float eps, void* out, int out_dtype,
                                 cudaStream_t stream) {
  FERRUM_CHECK_ARG(S >= 1 && S <= HC_MAX_STREAMS && E > 0, "hyper_step: %d streams of %d are outside the kernel's limits (up to %d)",
                   S, E, HC_MAX_STREAMS);
  const int has_write = mix != nullptr;
  FERRUM_CHECK_ARG(!has_write || (out_w != nullptr && (y != nullptr || partials != nullptr)), "hyper_step: a write needs y and its weights");
  FERRUM_CHECK_ARG(!has_write || partials != nullptr || ldy >= E, "hyper_step: rows of y are shorter than the streams'");
  FERRUM_CHECK_ARG(y_rows == nullptr || top > 0, "hyper_step: bad number of rows per token");
  FERRUM_CHECK_ARG(out == nullptr || (norm_w != nullptr && eps > 0.f), "hyper_step: a read needs the norm's weight");
  FERRUM_CHECK_ARG(!(store && rows != nullptr), "hyper_step: listed rows are read only");
  FERRUM_CHECK_ARG(out != nullptr || (has_write && store), "hyper_step: nothing to do");
  if (n_rows == 0) return 0;
  PartialLayout L{nullptr, 0, 0, 0, 0};
  if (has_write && partials != nullptr) {
    if (int r = partial_make_layout(partials, layout, &L)) return r;
    FERRUM_CHECK_ARG(E <= L.tiles * 128, "hyper_step: the partials cover %d features, the rows have %d", L.tiles * 128, E);
  }
  const HyperWrite w{y, ldy, y_rows, top, mix, out_w};
  const size_t smem = out != nullptr ? (size_t)E * sizeof(float) : 0;
  FERRUM_CHECK_ARG(smem <= 200 * 1024, "hyper_step: a row of %d floats does not fit shared memory", E);
#define HC_LAUNCH(T, V, SC)                                                                                                  \
  do {                                                                                                                   \
    if (smem > 48 * 1024) {                                                                                              \
      static size_t reserved = 0;                                                                                        \
      if (smem > reserved) {                                                                                             \
        cudaError_t e = cudaFuncSetAttribute(hyper_step_kernel<T, V, SC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        FERRUM_CHECK_ARG(e == cudaSuccess, "hyper_step: cannot reserve shared memory: %s", cudaGetErrorString(e));      \
        reserved = smem;                                                                                                 \
      }                                                                                                                  \
    }                                                                                                                    \
    launch_kernel(hyper_step_kernel<T, V, SC>, n_rows, HC_THREADS, smem, stream, X, S, E, rows, w, L, has_write, store, in_w, \
                  norm_w, eps, (T*)out);                                                                                 \
  } while (0)
  const bool wide = E % 4 == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0 &&
                    (y == nullptr || (ldy % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0));
#define HC_LAUNCH_S(T, V)                              \
  do {                                                 \
    if (S == 1) HC_LAUNCH(T, V, 1);                    \
    else if (S == 2) HC_LAUNCH(T, V, 2);               \
    else if (S == 3) HC_LAUNCH(T, V, 3);               \
    else if (S == 4) HC_LAUNCH(T, V, 4);               \
    else HC_LAUNCH(T, 1, 0);                           \
  } while (0)
  if (wide) {
    if (out == nullptr) HC_LAUNCH_S(float, 4);
    else FERRUM_DISPATCH_DTYPE(out_dtype, T, HC_LAUNCH_S(T, 4));
  } else {
    if (out == nullptr) HC_LAUNCH(float, 1, 0);
    else FERRUM_DISPATCH_DTYPE(out_dtype, T, HC_LAUNCH(T, 1, 0));
  }
#undef HC_LAUNCH_S
#undef HC_LAUNCH
  FERRUM_CHECK_LAUNCH("hyper_step");
  return 0;
}
