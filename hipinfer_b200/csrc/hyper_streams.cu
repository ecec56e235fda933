// Residual streams with learned mixing (hyper-connections). Instead of one residual row a token has S rows x_1 .. x_S,
// kept as one 32-bit row [S][W] (all equal to the embedding at the start). A sublayer reads a weighted sum of them and
// its result is written back into all of them while they are mixed among themselves:
//     u = sum_s a[s] x_s                       the sublayer's input, then its norm: h = u / rms(u) * w
//     x_t <- sum_s M[s][t] x_s + m * b[t] * y  for all t at once from the old rows (y the sublayer's result, m a constant)
// S = 1 with a = b = M = 1 is the plain pre-norm residual with a multiplier. Everything is 32-bit.
//
// streams_norm_kernel:        h = rms norm of u (optionally of chosen rows only; a == nullptr: the plain sum of the rows)
// streams_update_kernel:      the write-back alone
// streams_update_norm_kernel: the write-back and the NEXT reader's u and norm in one pass over the row
// streams_expand_kernel:      S copies of an embedding row
#include "common.cuh"

constexpr int HS_MAX = 8;          // most streams
constexpr int HS_THREADS = 256;

struct StreamCoef {
  float a[HS_MAX];                 // read weights of the sublayer that reads next
  float b[HS_MAX];                 // write weights (already times m)
  float M[HS_MAX][HS_MAX];         // [from][to]
};

__device__ __forceinline__ void hs_load_coef(StreamCoef& c, int S, const float* a, const float* b, const float* M, float m) {
  for (int s = 0; s < S; s++) {
    c.a[s] = a ? a[s] : 1.f;
    c.b[s] = b ? m * b[s] : m;
    for (int t = 0; t < S; t++) c.M[s][t] = M ? M[s * S + t] : (s == t ? 1.f : 0.f);
  }
}

template <typename TW, typename TO>
__global__ void __launch_bounds__(HS_THREADS) streams_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                                                  const float* __restrict__ a, const TW* __restrict__ w,
                                                                  TO* __restrict__ out, int S, int W, float eps) {
  __shared__ float sh[32];
  hb_pdl_launch();
  hb_pdl_wait();
  const int r = blockIdx.x;
  const float* row = x + (size_t)(rows ? rows[r] : r) * S * W;
  float coef[HS_MAX];
  for (int s = 0; s < S; s++) coef[s] = a ? a[s] : 1.f;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += HS_THREADS) {
    float u = 0.f;
    for (int s = 0; s < S; s++) u = fmaf(coef[s], row[(size_t)s * W + i], u);
    ss = fmaf(u, u, ss);
  }
  const float f = rsqrtf(hb_block_sum(ss, sh) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += HS_THREADS) {
    float u = 0.f;
    for (int s = 0; s < S; s++) u = fmaf(coef[s], row[(size_t)s * W + i], u);
    out[(size_t)r * W + i] = hb_from_float<TO>(u * f * hb_to_float(w[i]));
  }
}

HB_EXPORT int hb_streams_norm(const float* x, const int* rows, int n_rows, const float* a, const void* w, int w_dt, void* out,
                              int o_dt, int S, int W, float eps, cudaStream_t s) {
  if (n_rows <= 0) return 0;
  if (S < 1 || S > HS_MAX) HB_FAIL("hb_streams_norm: %d streams (1 to %d are supported)", S, HS_MAX);
  HB_DISPATCH_2(w_dt, o_dt, "hb_streams_norm",
                (hb_launch(streams_norm_kernel<TA, TB>, n_rows, HS_THREADS, 0, s, x, rows, a, (const TA*)w, (TB*)out, S, W, eps)));
  HB_CHECK_LAUNCH("hb_streams_norm");
  return 0;
}

__global__ void __launch_bounds__(HS_THREADS) streams_update_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                                    const float* __restrict__ b, const float* __restrict__ M,
                                                                    float m, long T, int S, int W) {
  hb_pdl_launch();
  StreamCoef c;
  hs_load_coef(c, S, nullptr, b, M, m);
  hb_pdl_wait();
  const long n = T * W;
  for (long i = (long)blockIdx.x * HS_THREADS + threadIdx.x; i < n; i += (long)gridDim.x * HS_THREADS) {
    const long t = i / W;
    const int col = (int)(i - t * W);
    float* row = x + (size_t)t * S * W + col;
    float old[HS_MAX];
    for (int s = 0; s < S; s++) old[s] = row[(size_t)s * W];
    const float yy = y[i];
    for (int to = 0; to < S; to++) {
      float v = c.b[to] * yy;
      for (int s = 0; s < S; s++) v = fmaf(c.M[s][to], old[s], v);
      row[(size_t)to * W] = v;
    }
  }
}

HB_EXPORT int hb_streams_update(float* x, const float* y, const float* b, const float* M, float m, int T, int S, int W,
                                cudaStream_t s) {
  if (T <= 0) return 0;
  if (S < 1 || S > HS_MAX) HB_FAIL("hb_streams_update: %d streams (1 to %d are supported)", S, HS_MAX);
  const long n = (long)T * W;
  const int blocks = (int)((n + HS_THREADS - 1) / HS_THREADS < 148 * 16 ? (n + HS_THREADS - 1) / HS_THREADS : 148 * 16);
  hb_launch(streams_update_kernel, blocks, HS_THREADS, 0, s, x, y, b, M, m, (long)T, S, W);
  HB_CHECK_LAUNCH("hb_streams_update");
  return 0;
}

// One block a row: the write-back of the sublayer that has just run, then u and the norm of the one that reads next. The
// thread that wrote a column reads it back in the second pass, so nothing is exchanged but the sum of squares.
template <typename TW, typename TO>
__global__ void __launch_bounds__(HS_THREADS) streams_update_norm_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                                         const float* __restrict__ b, const float* __restrict__ M,
                                                                         float m, const float* __restrict__ a_next,
                                                                         const TW* __restrict__ w_next, TO* __restrict__ out,
                                                                         int S, int W, float eps) {
  __shared__ float sh[32];
  hb_pdl_launch();
  StreamCoef c;
  hs_load_coef(c, S, a_next, b, M, m);
  hb_pdl_wait();
  const int r = blockIdx.x;
  float* row = x + (size_t)r * S * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += HS_THREADS) {
    float old[HS_MAX];
    for (int s = 0; s < S; s++) old[s] = row[(size_t)s * W + i];
    const float yy = y[(size_t)r * W + i];
    float u = 0.f;
    for (int to = 0; to < S; to++) {
      float v = c.b[to] * yy;
      for (int s = 0; s < S; s++) v = fmaf(c.M[s][to], old[s], v);
      row[(size_t)to * W + i] = v;
      u = fmaf(c.a[to], v, u);
    }
    ss = fmaf(u, u, ss);
  }
  const float f = rsqrtf(hb_block_sum(ss, sh) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += HS_THREADS) {
    float u = 0.f;
    for (int s = 0; s < S; s++) u = fmaf(c.a[s], row[(size_t)s * W + i], u);
    out[(size_t)r * W + i] = hb_from_float<TO>(u * f * hb_to_float(w_next[i]));
  }
}

// The same for rows of up to HS_THREADS * 4 * HS_KEEP columns (a multiple of four) and a stream count known to the compiler:
// four columns a load, and u stays in registers between the two passes, so a row is read once and written once.
constexpr int HS_KEEP = 4;

template <typename TW, typename TO, int S>
__global__ void __launch_bounds__(HS_THREADS) streams_update_norm_vec_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                                             const float* __restrict__ b, const float* __restrict__ M,
                                                                             float m, const float* __restrict__ a_next,
                                                                             const TW* __restrict__ w_next, TO* __restrict__ out,
                                                                             int W, float eps) {
  __shared__ float sh[32];
  hb_pdl_launch();
  float ca[S], cb[S], cm[S][S];
#pragma unroll
  for (int s = 0; s < S; s++) {
    ca[s] = a_next ? a_next[s] : 1.f;
    cb[s] = b ? m * b[s] : m;
#pragma unroll
    for (int t = 0; t < S; t++) cm[s][t] = M ? M[s * S + t] : (s == t ? 1.f : 0.f);
  }
  hb_pdl_wait();
  const int r = blockIdx.x;
  float* row = x + (size_t)r * S * W;
  float4 uu[HS_KEEP];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < HS_KEEP; k++) {
    const int i = (k * HS_THREADS + threadIdx.x) * 4;
    uu[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < W) {
      float4 old[S];
#pragma unroll
      for (int s = 0; s < S; s++) old[s] = *(const float4*)(row + (size_t)s * W + i);
      const float4 yy = *(const float4*)(y + (size_t)r * W + i);
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int to = 0; to < S; to++) {
        float4 v = make_float4(cb[to] * yy.x, cb[to] * yy.y, cb[to] * yy.z, cb[to] * yy.w);
#pragma unroll
        for (int s = 0; s < S; s++) {
          v.x = fmaf(cm[s][to], old[s].x, v.x);
          v.y = fmaf(cm[s][to], old[s].y, v.y);
          v.z = fmaf(cm[s][to], old[s].z, v.z);
          v.w = fmaf(cm[s][to], old[s].w, v.w);
        }
        *(float4*)(row + (size_t)to * W + i) = v;
        u.x = fmaf(ca[to], v.x, u.x);
        u.y = fmaf(ca[to], v.y, u.y);
        u.z = fmaf(ca[to], v.z, u.z);
        u.w = fmaf(ca[to], v.w, u.w);
      }
      uu[k] = u;
      ss = fmaf(u.x, u.x, ss);
      ss = fmaf(u.y, u.y, ss);
      ss = fmaf(u.z, u.z, ss);
      ss = fmaf(u.w, u.w, ss);
    }
  }
  const float f = rsqrtf(hb_block_sum(ss, sh) / (float)W + eps);
#pragma unroll
  for (int k = 0; k < HS_KEEP; k++) {
    const int i = (k * HS_THREADS + threadIdx.x) * 4;
    if (i < W) {
      const float4 wv = hb_load4(w_next + i);
      hb_store4(out + (size_t)r * W + i, make_float4(uu[k].x * f * wv.x, uu[k].y * f * wv.y, uu[k].z * f * wv.z, uu[k].w * f * wv.w));
    }
  }
}

HB_EXPORT int hb_streams_update_norm(float* x, const float* y, const float* b, const float* M, float m, const float* a_next,
                                     const void* w_next, int w_dt, void* out, int o_dt, int T, int S, int W, float eps,
                                     cudaStream_t s) {
  if (T <= 0) return 0;
  if (S < 1 || S > HS_MAX) HB_FAIL("hb_streams_update_norm: %d streams (1 to %d are supported)", S, HS_MAX);
  const bool vec = W % 4 == 0 && W <= HS_THREADS * 4 * HS_KEEP && S <= 4 &&
                   !(((uintptr_t)x | (uintptr_t)y | (uintptr_t)out | (uintptr_t)w_next) & 15);
#define HS_VEC(SS)                                                                                                    \
  HB_DISPATCH_2(w_dt, o_dt, "hb_streams_update_norm",                                                                 \
                (hb_launch(streams_update_norm_vec_kernel<TA, TB, SS>, T, HS_THREADS, 0, s, x, y, b, M, m, a_next,    \
                           (const TA*)w_next, (TB*)out, W, eps)))
  if (vec && S == 1) HS_VEC(1);
  else if (vec && S == 2) HS_VEC(2);
  else if (vec && S == 3) HS_VEC(3);
  else if (vec && S == 4) HS_VEC(4);
  else
    HB_DISPATCH_2(w_dt, o_dt, "hb_streams_update_norm",
                  (hb_launch(streams_update_norm_kernel<TA, TB>, T, HS_THREADS, 0, s, x, y, b, M, m, a_next, (const TA*)w_next,
                             (TB*)out, S, W, eps)));
#undef HS_VEC
  HB_CHECK_LAUNCH("hb_streams_update_norm");
  return 0;
}

__global__ void __launch_bounds__(HS_THREADS) streams_expand_kernel(const float* __restrict__ x, float* __restrict__ xs, long T,
                                                                    int S, int W) {
  hb_pdl_launch();
  hb_pdl_wait();
  const long n = T * W;
  for (long i = (long)blockIdx.x * HS_THREADS + threadIdx.x; i < n; i += (long)gridDim.x * HS_THREADS) {
    const long t = i / W;
    const int col = (int)(i - t * W);
    const float v = x[i];
    for (int s = 0; s < S; s++) xs[((size_t)t * S + s) * W + col] = v;
  }
}

HB_EXPORT int hb_streams_expand(const float* x, float* xs, int T, int S, int W, cudaStream_t s) {
  if (T <= 0) return 0;
  const long n = (long)T * W;
  const int blocks = (int)((n + HS_THREADS - 1) / HS_THREADS < 148 * 16 ? (n + HS_THREADS - 1) / HS_THREADS : 148 * 16);
  hb_launch(streams_expand_kernel, blocks, HS_THREADS, 0, s, x, xs, (long)T, S, W);
  HB_CHECK_LAUNCH("hb_streams_expand");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// A gated activation with biases and limits, and small row operations that go with it.
//   gate/up come as one 32-bit product result [M][2 I], interleaved in groups of `group` columns (group gate columns,
//   group up columns, ...), the bias [2 I] in the same order.
//   kind 0: silu(g) * u        kind 1: gelu_tanh(g) * u
//   kind 2: g' = min(g, L), u' = clamp(u, -L, L); g' * sigmoid(alpha g') * (u' + 1)
// ---------------------------------------------------------------------------------------------------------------------
// One activation, the same arithmetic in both kernels.
__device__ __forceinline__ float glu_one(float g, float u, int kind, float limit, float alpha) {
  if (kind == 0) return g / (1.f + expf(-g)) * u;
  if (kind == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

template <typename TW, typename TO>
__global__ void __launch_bounds__(256) glu_bias_kernel(const float* __restrict__ gu, long ld, const TW* __restrict__ bias,
                                                       TO* __restrict__ out, long ldo, long M, int I, int group, int kind,
                                                       float limit, float alpha) {
  hb_pdl_launch();
  hb_pdl_wait();
  const long n = M * I;
  for (long idx = (long)blockIdx.x * 256 + threadIdx.x; idx < n; idx += (long)gridDim.x * 256) {
    const long mrow = idx / I;
    const int i = (int)(idx - mrow * I);
    const int cg = (i / group) * 2 * group + i % group, cu = cg + group;
    float g = gu[mrow * ld + cg], u = gu[mrow * ld + cu];
    if (bias) {
      g += hb_to_float(bias[cg]);
      u += hb_to_float(bias[cu]);
    }
    out[mrow * ldo + i] = hb_from_float<TO>(glu_one(g, u, kind, limit, alpha));
  }
}

// Four output columns a thread (groups that are multiples of four, 16-byte aligned rows): the same values, fewer and
// wider loads and stores.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256) glu_bias_vec_kernel(const float* __restrict__ gu, long ld, const TW* __restrict__ bias,
                                                           TO* __restrict__ out, long ldo, long M, int I, int group, int kind,
                                                           float limit, float alpha) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int I4 = I >> 2;
  const long n = M * I4;
  for (long idx = (long)blockIdx.x * 256 + threadIdx.x; idx < n; idx += (long)gridDim.x * 256) {
    const long mrow = idx / I4;
    const int i = (int)(idx - mrow * I4) << 2;
    const int cg = (i / group) * 2 * group + i % group, cu = cg + group;
    float4 g = *(const float4*)(gu + mrow * ld + cg), u = *(const float4*)(gu + mrow * ld + cu);
    if (bias) {
      const float4 bg = hb_load4(bias + cg), bu = hb_load4(bias + cu);
      g.x += bg.x; g.y += bg.y; g.z += bg.z; g.w += bg.w;
      u.x += bu.x; u.y += bu.y; u.z += bu.z; u.w += bu.w;
    }
    hb_store4(out + mrow * ldo + i, make_float4(glu_one(g.x, u.x, kind, limit, alpha), glu_one(g.y, u.y, kind, limit, alpha),
                                                glu_one(g.z, u.z, kind, limit, alpha), glu_one(g.w, u.w, kind, limit, alpha)));
  }
}

HB_EXPORT int hb_glu_bias(const float* gu, long ld, const void* bias, int b_dt, void* out, int o_dt, long ldo, int M, int I,
                          int group, int kind, float limit, float alpha, cudaStream_t s) {
  if (M <= 0 || I <= 0) return 0;
  if (kind < 0 || kind > 2 || group <= 0 || I % group) HB_FAIL("hb_glu_bias: kind %d, %d columns in groups of %d", kind, I, group);
  if (group % 4 == 0 && ld % 4 == 0 && ldo % 4 == 0 && !(((uintptr_t)gu | (uintptr_t)out | (uintptr_t)bias) & 15)) {
    const long n4 = (long)M * (I / 4);
    const int blocks4 = (int)((n4 + 255) / 256 < 148 * 16 ? (n4 + 255) / 256 : 148 * 16);
    HB_DISPATCH_2(b_dt, o_dt, "hb_glu_bias",
                  (hb_launch(glu_bias_vec_kernel<TA, TB>, blocks4, 256, 0, s, gu, ld, (const TA*)bias, (TB*)out, ldo, (long)M, I,
                             group, kind, limit, alpha)));
    HB_CHECK_LAUNCH("hb_glu_bias");
    return 0;
  }
  const long n = (long)M * I;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  HB_DISPATCH_2(b_dt, o_dt, "hb_glu_bias",
                (hb_launch(glu_bias_kernel<TA, TB>, blocks, 256, 0, s, gu, ld, (const TA*)bias, (TB*)out, ldo, (long)M, I, group,
                           kind, limit, alpha)));
  HB_CHECK_LAUNCH("hb_glu_bias");
  return 0;
}

// x[m][n] = x[m][n] * scale (+ bias[n]): the scaled logits; a projection's bias
template <typename TW>
__global__ void __launch_bounds__(256) scale_bias_rows_kernel(float* __restrict__ x, long ld, const TW* __restrict__ bias,
                                                              float scale, long M, int N) {
  hb_pdl_launch();
  hb_pdl_wait();
  const long n = M * N;
  for (long idx = (long)blockIdx.x * 256 + threadIdx.x; idx < n; idx += (long)gridDim.x * 256) {
    const long mrow = idx / N;
    const int c = (int)(idx - mrow * N);
    float v = x[mrow * ld + c] * scale;
    if (bias) v += hb_to_float(bias[c]);
    x[mrow * ld + c] = v;
  }
}

HB_EXPORT int hb_scale_bias_rows(float* x, long ld, const void* bias, int b_dt, float scale, int M, int N, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  const long n = (long)M * N;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  HB_DISPATCH_1(b_dt, "hb_scale_bias_rows",
                (hb_launch(scale_bias_rows_kernel<TA>, blocks, 256, 0, s, x, ld, (const TA*)bias, scale, (long)M, N)));
  HB_CHECK_LAUNCH("hb_scale_bias_rows");
  return 0;
}
