// A routed feed-forward (mixture of experts): every token runs `top` of E small gated feed-forward layers.
//     z = Wr h (32-bit);  s = sigmoid(z);  the `top` largest s choose the experts (ties: the lower index)
//     out = sum over the chosen e of Wd_e (silu(Wg_e v) * (Wu_e v)),  v = s_e h
// The score multiplies the expert's INPUT. Experts have no biases, so Wg_e (s h) = s (Wg_e h): the products run on h and
// the score enters the activation in 32-bit, silu(s g) * (s u).
// A second form (route mode 1, `at_output`): z = Wr h + b; the `top` largest LOGITS choose; the weights are the softmax over
// the chosen logits alone and multiply the expert's RESULT, which, the down product being linear, is the activation times
// the weight, silu(g) * u * s, again in 32-bit.
//
// moe_route_kernel          scores and the chosen experts of every row: expert [T][top], weight [T][top]
// Few rows (decoding): no sorting, nothing on the host
//   moe_gate_up_rows_kernel a block per ((row, choice), tile of the expert's hidden rows): act [T * top][F]
//   moe_down_rows_kernel    a block per (row, tile of output columns): the choices' results summed in their order
// Some rows (decoding in a batch): the pairs sorted by expert on the device, then
//   moe_grouped_kernel      a block per (expert, tile of output features): the expert's weights are read once for all of
//   moe_grouped_mma_kernel  its rows (a round of them at a time), for the gate/up product and for the down product;
//                           nothing on the host, so the step replays from a CUDA graph. The second is the bfloat16 form on
//                           warp MMAs, the first takes any element types and sizes
// Many rows (prompt portions): the (row, choice) pairs are sorted by expert, so that each expert's rows are one
// contiguous block that an ordinary product takes
//   moe_sort_kernel         offsets [E + 1], pos [pair] -> sorted row, src [sorted row] -> pair
//   moe_gather_kernel       the sorted copy of the input rows
//   moe_act_kernel          silu(s g) * (s u) on the sorted rows' 32-bit [g | u]
//   moe_combine_kernel      out[t] += sum over the choices, in their order, of the sorted results
#include "common.cuh"

constexpr int MR_THREADS = 128;

template <typename TA, typename TW>
__global__ void __launch_bounds__(MR_THREADS) moe_route_kernel(const TA* __restrict__ xn, long ldx, const TW* __restrict__ router,
                                                               const TW* __restrict__ bias, int* __restrict__ expert,
                                                               float* __restrict__ weight, int W, int E, int top, int mode) {
  extern __shared__ float mr_sm[];     // [W] the row, [E] the scores
  float* row = mr_sm;
  float* sc = mr_sm + W;
  hb_pdl_launch();
  hb_pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < W; i += MR_THREADS) row[i] = hb_to_float(xn[(size_t)t * ldx + i]);
  __syncthreads();
  for (int e = warp; e < E; e += MR_THREADS / 32) {
    const TW* wr = router + (size_t)e * W;
    float acc = 0.f;
    for (int i = lane; i < W; i += 32) acc = fmaf(row[i], hb_to_float(wr[i]), acc);
    acc = hb_warp_sum(acc);
    if (bias) acc += hb_to_float(bias[e]);
    if (lane == 0) sc[e] = mode == 0 ? 1.f / (1.f + expf(-acc)) : acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float first = 0.f, den = 0.f;
    for (int k = 0; k < top; k++) {
      int best = -1;
      float bs = 0.f;
      for (int e = 0; e < E; e++) {
        const float v = sc[e];
        if (v != v) continue;          // NaN marks an expert that is taken
        if (best < 0 || v > bs) {
          bs = v;
          best = e;
        }
      }
      if (best < 0) best = 0;          // every score NaN (bad weights or input): stay inside the tables
      expert[(size_t)t * top + k] = best;
      if (mode == 0) weight[(size_t)t * top + k] = bs;
      else {
        // softmax over the chosen logits alone: the first chosen one is the largest
        if (k == 0) first = bs;
        const float ex = expf(bs - first);
        weight[(size_t)t * top + k] = ex;
        den += ex;
      }
      sc[best] = __int_as_float(0x7fc00000);
    }
    if (mode != 0)
      for (int k = 0; k < top; k++) weight[(size_t)t * top + k] /= den;
  }
}

// mode 0: the scores are sigmoid(z) and the chosen scores are the weights; mode 1: the largest logits z choose and the
// weights are the softmax over the chosen logits alone. bias (the router's element type, or null) is added to z.
HB_EXPORT int hb_moe_route(const void* xn, int x_dt, long ldx, const void* router, const void* bias, int w_dt, int* expert,
                           float* weight, int T, int W, int E, int top, int mode, cudaStream_t s) {
  if (T <= 0) return 0;
  if (top < 1 || top > E) HB_FAIL("hb_moe_route: top %d of %d experts", top, E);
  const size_t smem = (size_t)(W + E) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_moe_route: a row of %d with %d experts does not fit shared memory", W, E);
  HB_DISPATCH_2(x_dt, w_dt, "hb_moe_route", do {
    auto kern = moe_route_kernel<TA, TB>;
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(kern, dim3(T), dim3(MR_THREADS), smem, s, (const TA*)xn, ldx, (const TB*)router, (const TB*)bias, expert, weight,
              W, E, top, mode);
  } while (0));
  HB_CHECK_LAUNCH("hb_moe_route");
  return 0;
}

// A warp's dot product of a weight row with a 32-bit row in shared memory: lanes take groups of four columns (scalar
// columns where K is no multiple of four), the lanes' sums are joined in a fixed order.
template <typename TW>
__device__ __forceinline__ float moe_warp_dot(const TW* __restrict__ w, const float* __restrict__ a, int K, int lane, bool vec) {
  float acc = 0.f;
  if (vec) {
    for (int i = lane * 4; i < K; i += 128) {
      const float4 wv = hb_load4(w + i);
      const float4 av = *(const float4*)(a + i);
      acc = fmaf(wv.x, av.x, acc);
      acc = fmaf(wv.y, av.y, acc);
      acc = fmaf(wv.z, av.z, acc);
      acc = fmaf(wv.w, av.w, acc);
    }
  } else {
    for (int i = lane; i < K; i += 32) acc = fmaf(hb_to_float(w[i]), a[i], acc);
  }
  return hb_warp_sum(acc);
}

constexpr int MG_THREADS = 256, MG_ROWS = 32;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(MG_THREADS) moe_gate_up_rows_kernel(const TA* __restrict__ xn, long ldx,
                                                                      const TW* __restrict__ wgu, const int* __restrict__ expert,
                                                                      const float* __restrict__ weight, TO* __restrict__ act,
                                                                      int W, int F, int top, int vec, int at_output) {
  extern __shared__ __align__(16) float mg_row[];      // [W]
  hb_pdl_launch();
  hb_pdl_wait();
  const int pair = blockIdx.y, t = pair / top, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < W; i += MG_THREADS) mg_row[i] = hb_to_float(xn[(size_t)t * ldx + i]);
  __syncthreads();
  const int e = expert[pair];
  const float sw = weight[pair];
  const float s = at_output ? 1.f : sw, so = at_output ? sw : 1.f;     // the weight multiplies the input, or the result
  const TW* we = wgu + (size_t)e * 2 * F * W;          // [gate rows (F) | up rows (F)][W]
  const int j1 = min(F, (int)(blockIdx.x + 1) * MG_ROWS);
  for (int j = blockIdx.x * MG_ROWS + warp; j < j1; j += MG_THREADS / 32) {
    const float g = s * moe_warp_dot(we + (size_t)j * W, mg_row, W, lane, vec);
    const float u = s * moe_warp_dot(we + (size_t)(F + j) * W, mg_row, W, lane, vec);
    if (lane == 0) act[(size_t)pair * F + j] = hb_from_float<TO>(g / (1.f + expf(-g)) * u * so);
  }
}

HB_EXPORT int hb_moe_gate_up_rows(const void* xn, int x_dt, long ldx, const void* wgu, int w_dt, const int* expert,
                                  const float* weight, void* act, int T, int W, int F, int top, int at_output, cudaStream_t s) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)W * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_moe_gate_up_rows: a row of %d does not fit shared memory", W);
  const int vec = (W % 4 == 0) ? 1 : 0;
  dim3 grid((F + MG_ROWS - 1) / MG_ROWS, T * top);
  if (grid.y > 65535) HB_FAIL("hb_moe_gate_up_rows: %d rows x %d choices are too many for this kernel", T, top);
  // the activation has the input's element type
  HB_DISPATCH_2(x_dt, w_dt, "hb_moe_gate_up_rows", do {
    auto kern = moe_gate_up_rows_kernel<TA, TB, TA>;
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(kern, grid, dim3(MG_THREADS), smem, s, (const TA*)xn, ldx, (const TB*)wgu, expert, weight, (TA*)act, W, F, top, vec, at_output);
  } while (0));
  HB_CHECK_LAUNCH("hb_moe_gate_up_rows");
  return 0;
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(MG_THREADS) moe_down_rows_kernel(const TA* __restrict__ act, const TW* __restrict__ wd,
                                                                   const int* __restrict__ expert, float* __restrict__ y, long ldy,
                                                                   int W, int F, int top, int vec) {
  extern __shared__ __align__(16) float md_act[];      // [top][F4], F4 = F rounded up to four
  hb_pdl_launch();
  hb_pdl_wait();
  const int t = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int F4 = (F + 3) & ~3;
  for (int i = threadIdx.x; i < top * F; i += MG_THREADS) {
    const int k = i / F, j = i - k * F;
    md_act[k * F4 + j] = hb_to_float(act[((size_t)t * top + k) * F + j]);
  }
  __syncthreads();
  const int n1 = min(W, (int)(blockIdx.x + 1) * MG_ROWS);
  for (int n = blockIdx.x * MG_ROWS + warp; n < n1; n += MG_THREADS / 32) {
    float acc = 0.f;
    for (int k = 0; k < top; k++) {
      const int e = expert[(size_t)t * top + k];
      acc += moe_warp_dot(wd + ((size_t)e * W + n) * F, md_act + k * F4, F, lane, vec);
    }
    if (lane == 0) y[(size_t)t * ldy + n] += acc;
  }
}

HB_EXPORT int hb_moe_down_rows(const void* act, int a_dt, const void* wd, int w_dt, const int* expert, float* y, long ldy, int T,
                               int W, int F, int top, cudaStream_t s) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)top * ((F + 3) & ~3) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_moe_down_rows: %d x %d activations do not fit shared memory", top, F);
  const int vec = (F % 4 == 0) ? 1 : 0;
  dim3 grid((W + MG_ROWS - 1) / MG_ROWS, T);
  if (grid.y > 65535) HB_FAIL("hb_moe_down_rows: %d rows are too many for this kernel", T);
  HB_DISPATCH_2(a_dt, w_dt, "hb_moe_down_rows", do {
    auto kern = moe_down_rows_kernel<TA, TB>;
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(kern, grid, dim3(MG_THREADS), smem, s, (const TA*)act, (const TB*)wd, expert, y, ldy, W, F, top, vec);
  } while (0));
  HB_CHECK_LAUNCH("hb_moe_down_rows");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Some rows: one product kernel over all experts' blocks of sorted rows.
//   out[r][n] = sum_k w[e][n][k] a[row(r)][k]   for offsets[e] <= r < offsets[e + 1], e = blockIdx.y
// row(r) = src[r] / top where src is given (the step's input rows, gathered on the fly), else r. A warp owns MX_NW output
// features and MX_RB rows at a time: a weight row comes from memory once a round of rows, the rows wait in shared memory in
// their own element type, K in segments of KS. A (row, feature) sum runs in the same order whatever else is in the round.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int MX_THREADS = 256, MX_RB = 8, MX_NW = 4, MX_TILE = (MX_THREADS / 32) * MX_NW;

template <typename T> struct MxVec4;
template <> struct MxVec4<float> { using type = float4; };
template <> struct MxVec4<__nv_bfloat16> { using type = uint2; };

// One round: R rows (the first nr of them live) against the block's MX_TILE output features.
template <typename TA, typename TW, int R>
__device__ __forceinline__ void mx_round(const TA* __restrict__ a, long lda, const int* mx_row, int nr, const TW* __restrict__ we,
                                         float* __restrict__ out, TA* rows, int g0, int n0, int Nout, int K, int KS, int vec) {
  using V4 = typename MxVec4<TA>::type;
  const int tid = threadIdx.x, lane = tid & 31;
  float acc[MX_NW][R];
#pragma unroll
  for (int q = 0; q < MX_NW; q++)
#pragma unroll
    for (int r = 0; r < R; r++) acc[q][r] = 0.f;
  for (int k0 = 0; k0 < K; k0 += KS) {
    const int kn = min(KS, K - k0);
    __syncthreads();                                        // the segment before has been read; mx_row is written
    if (vec) {
      const int per = kn >> 2;
      for (int r = 0; r < nr; r++) {
        const TA* ar = a + (size_t)mx_row[r] * lda + k0;
#pragma unroll 4
        for (int i = tid; i < per; i += MX_THREADS) *(V4*)(rows + (size_t)r * KS + 4 * i) = *(const V4*)(ar + 4 * i);
      }
    } else {
      for (int r = 0; r < nr; r++) {
        const TA* ar = a + (size_t)mx_row[r] * lda + k0;
        for (int i = tid; i < kn; i += MX_THREADS) rows[(size_t)r * KS + i] = ar[i];
      }
    }
    __syncthreads();
    if (vec) {
#pragma unroll 2
      for (int i = lane * 4; i < kn; i += 128) {
        float4 wv[MX_NW];
#pragma unroll
        for (int q = 0; q < MX_NW; q++)
          wv[q] = n0 + q < Nout ? hb_load4(we + (size_t)(n0 + q) * K + k0 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < R; r++) {
          const float4 av = hb_load4(rows + (size_t)r * KS + i);
#pragma unroll
          for (int q = 0; q < MX_NW; q++) {
            acc[q][r] = fmaf(wv[q].x, av.x, acc[q][r]);
            acc[q][r] = fmaf(wv[q].y, av.y, acc[q][r]);
            acc[q][r] = fmaf(wv[q].z, av.z, acc[q][r]);
            acc[q][r] = fmaf(wv[q].w, av.w, acc[q][r]);
          }
        }
      }
    } else {
      for (int i = lane; i < kn; i += 32) {
        float wv[MX_NW];
#pragma unroll
        for (int q = 0; q < MX_NW; q++) wv[q] = n0 + q < Nout ? hb_to_float(we[(size_t)(n0 + q) * K + k0 + i]) : 0.f;
#pragma unroll
        for (int r = 0; r < R; r++) {
          const float av = hb_to_float(rows[(size_t)r * KS + i]);
#pragma unroll
          for (int q = 0; q < MX_NW; q++) acc[q][r] = fmaf(wv[q], av, acc[q][r]);
        }
      }
    }
  }
  // rows beyond nr hold whatever shared memory held: their sums are never stored
#pragma unroll
  for (int q = 0; q < MX_NW; q++)
#pragma unroll
    for (int r = 0; r < R; r++) {
      const float v = hb_warp_sum(acc[q][r]);
      if (lane == 0 && n0 + q < Nout && r < nr) out[(size_t)(g0 + r) * Nout + n0 + q] = v;
    }
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(MX_THREADS) moe_grouped_kernel(const TA* __restrict__ a, long lda, const int* __restrict__ src,
                                                                 int top, const TW* __restrict__ w, const int* __restrict__ offsets,
                                                                 float* __restrict__ out, int Nout, int K, int KS, int vec) {
  extern __shared__ __align__(16) unsigned char mx_raw[];
  __shared__ int mx_row[MX_RB];
  TA* rows = (TA*)mx_raw;                                   // [MX_RB][KS]
  hb_pdl_launch();
  hb_pdl_wait();
  const int e = blockIdx.y, lo = offsets[e], hi = offsets[e + 1];
  if (lo >= hi) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n0 = blockIdx.x * MX_TILE + warp * MX_NW;
  const TW* we = w + (size_t)e * Nout * K;
  for (int g0 = lo; g0 < hi; g0 += MX_RB) {
    const int nr = min(MX_RB, hi - g0);
    __syncthreads();                                        // the round before has read its row numbers
    if (tid < nr) mx_row[tid] = src ? src[g0 + tid] / top : g0 + tid;
    // a round of few rows does the sums of few rows; which form a row meets changes nothing in its sums
    if (nr == 1) mx_round<TA, TW, 1>(a, lda, mx_row, nr, we, out, rows, g0, n0, Nout, K, KS, vec);
    else if (nr == 2) mx_round<TA, TW, 2>(a, lda, mx_row, nr, we, out, rows, g0, n0, Nout, K, KS, vec);
    else if (nr <= 4) mx_round<TA, TW, 4>(a, lda, mx_row, nr, we, out, rows, g0, n0, Nout, K, KS, vec);
    else mx_round<TA, TW, MX_RB>(a, lda, mx_row, nr, we, out, rows, g0, n0, Nout, K, KS, vec);
  }
}

// The same product on warp MMAs (bfloat16 rows and weights, K a multiple of 32). The weights are the MMA's row operand,
// 16 output features a warp, and come straight from memory: a lane reads 8 consecutive k of feature g and of feature
// g + 8 (16 bytes each) per block of 32 k; the rows are the column operand, 8 a tile, up to 4 tiles a round, from shared
// memory in segments of MM_KS k (twice and four times as many where a round has at most 16 or 8 rows). Inside a block of 32 k the lanes' k are dealt to the MMA's k slots in another order than
// memory's, the same for both operands, which a sum over k does not see. 32-bit accumulation; a (row, feature) sum does
// not depend on the other rows of the round.
constexpr int MM_THREADS = 128, MM_KS = 1024, MM_LD = MM_KS + 32, MM_ROWS = 32, MM_TILE = 16 * (MM_THREADS / 32);

__device__ __forceinline__ void mm_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>
__device__ __forceinline__ void mm_round(const __nv_bfloat16* __restrict__ a, long lda, const int* mm_row, int nr,
                                         const __nv_bfloat16* __restrict__ we, float* __restrict__ out, __nv_bfloat16* rows, int g0,
                                         int n0, int Nout, int K) {
  constexpr int KS = MM_KS * 4 / NT, LD = KS + 32;           // the same shared memory holds fewer rows of more k
  const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[nt][i] = 0.f;
  // features past the end read the last feature's weights; their sums are not stored
  const __nv_bfloat16* wa = we + (size_t)min(n0 + g, Nout - 1) * K + t * 8;
  const __nv_bfloat16* wb = we + (size_t)min(n0 + g + 8, Nout - 1) * K + t * 8;
  for (int k0 = 0; k0 < K; k0 += KS) {
    const int kn = min(KS, K - k0), per = kn >> 3;
    __syncthreads();                                        // the segment before has been read; mm_row is written
    for (int r = 0; r < nr; r++) {
      const __nv_bfloat16* ar = a + (size_t)mm_row[r] * lda + k0;
#pragma unroll 4
      for (int i = tid; i < per; i += MM_THREADS) *(uint4*)(rows + (size_t)r * LD + 8 * i) = *(const uint4*)(ar + 8 * i);
    }
    __syncthreads();
#pragma unroll 4
    for (int kb = 0; kb < kn; kb += 32) {
      const uint4 A0 = *(const uint4*)(wa + k0 + kb), A1 = *(const uint4*)(wb + k0 + kb);
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        // rows past nr hold whatever shared memory held: a row is a column of the MMA, and its sums are not stored
        const uint4 B = *(const uint4*)(rows + (size_t)(nt * 8 + g) * LD + kb + t * 8);
        mm_mma(acc[nt], A0.x, A1.x, A0.y, A1.y, B.x, B.y);
        mm_mma(acc[nt], A0.z, A1.z, A0.w, A1.w, B.z, B.w);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int r = nt * 8 + 2 * t + (i & 1), n = n0 + g + (i >> 1) * 8;
      if (r < nr && n < Nout) out[(size_t)(g0 + r) * Nout + n] = acc[nt][i];
    }
}

__global__ void __launch_bounds__(MM_THREADS) moe_grouped_mma_kernel(const __nv_bfloat16* __restrict__ a, long lda,
                                                                     const int* __restrict__ src, int top,
                                                                     const __nv_bfloat16* __restrict__ w,
                                                                     const int* __restrict__ offsets, float* __restrict__ out,
                                                                     int Nout, int K) {
  extern __shared__ __align__(16) unsigned char mx_raw[];
  __shared__ int mm_row[MM_ROWS];
  __nv_bfloat16* rows = (__nv_bfloat16*)mx_raw;             // [MM_ROWS][MM_LD], or half the rows of twice the k, or a quarter of four times
  hb_pdl_launch();
  hb_pdl_wait();
  const int e = blockIdx.y, lo = offsets[e], hi = offsets[e + 1];
  if (lo >= hi) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n0 = blockIdx.x * MM_TILE + warp * 16;
  const __nv_bfloat16* we = w + (size_t)e * Nout * K;
  for (int g0 = lo; g0 < hi; g0 += MM_ROWS) {
    const int nr = min(MM_ROWS, hi - g0);
    __syncthreads();                                        // the round before has read its row numbers
    if (tid < nr) mm_row[tid] = src ? src[g0 + tid] / top : g0 + tid;
    if (nr <= 8) mm_round<1>(a, lda, mm_row, nr, we, out, rows, g0, n0, Nout, K);
    else if (nr <= 16) mm_round<2>(a, lda, mm_row, nr, we, out, rows, g0, n0, Nout, K);
    else mm_round<4>(a, lda, mm_row, nr, we, out, rows, g0, n0, Nout, K);
  }
}

HB_EXPORT int hb_moe_grouped(const void* a, int a_dt, long lda, const int* src, int top, const void* w, int w_dt,
                             const int* offsets, float* out, int E, int Nout, int K, cudaStream_t s) {
  if (E <= 0 || Nout <= 0 || K <= 0) return 0;
  if (E > 65535) HB_FAIL("hb_moe_grouped: %d experts are too many for this kernel", E);
  if (a_dt == HB_BF16 && w_dt == HB_BF16 && K % 32 == 0 && lda % 8 == 0 && !(((uintptr_t)a | (uintptr_t)w) & 15)) {
    const size_t smem = (size_t)MM_ROWS * MM_LD * sizeof(__nv_bfloat16);
    cudaFuncSetAttribute(moe_grouped_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(moe_grouped_mma_kernel, dim3((Nout + MM_TILE - 1) / MM_TILE, E), dim3(MM_THREADS), smem, s,
              (const __nv_bfloat16*)a, lda, src, top, (const __nv_bfloat16*)w, offsets, out, Nout, K);
    HB_CHECK_LAUNCH("hb_moe_grouped");
    return 0;
  }
  const int esz = a_dt == HB_F32 ? 4 : 2;
  const int vec = (K % 4 == 0 && lda % 4 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0) ? 1 : 0;
  const int cap = (64 * 1024 / (MX_RB * esz)) & ~3;        // a segment's elements a row
  const int KS = K < cap ? ((K + 3) & ~3) : cap;
  const size_t smem = (size_t)MX_RB * KS * esz;
  dim3 grid((Nout + MX_TILE - 1) / MX_TILE, E);
  HB_DISPATCH_2(a_dt, w_dt, "hb_moe_grouped", do {
    auto kern = moe_grouped_kernel<TA, TB>;
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(kern, grid, dim3(MX_THREADS), smem, s, (const TA*)a, lda, src, top, (const TB*)w, offsets, out, Nout, K, KS, vec);
  } while (0));
  HB_CHECK_LAUNCH("hb_moe_grouped");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Many rows: the pairs sorted by expert.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int MS_THREADS = 1024;

// One block. Which sorted row a pair gets inside its expert's block depends on the order in which the threads arrive; a
// row's result does not depend on where it lies.
__global__ void __launch_bounds__(MS_THREADS) moe_sort_kernel(const int* __restrict__ expert, int* __restrict__ offsets,
                                                              int* __restrict__ pos, int* __restrict__ src, int pairs, int E) {
  extern __shared__ int ms_sm[];       // [E] counts, then cursors; [E] first sorted row of each expert
  int* count = ms_sm;
  int* base = ms_sm + E;
  hb_pdl_launch();
  hb_pdl_wait();
  for (int e = threadIdx.x; e < E; e += MS_THREADS) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += MS_THREADS) atomicAdd(&count[expert[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; e++) {
      base[e] = run;
      offsets[e] = run;
      run += count[e];
      count[e] = 0;
    }
    offsets[E] = run;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += MS_THREADS) {
    const int e = expert[p];
    const int r = base[e] + atomicAdd(&count[e], 1);
    pos[p] = r;
    src[r] = p;
  }
}

HB_EXPORT int hb_moe_sort(const int* expert, int* offsets, int* pos, int* src, int pairs, int E, cudaStream_t s) {
  if (pairs <= 0) return 0;
  const size_t smem = (size_t)2 * E * sizeof(int);
  if (smem > 40 * 1024) HB_FAIL("hb_moe_sort: %d experts are too many", E);
  hb_launch(moe_sort_kernel, dim3(1), dim3(MS_THREADS), smem, s, expert, offsets, pos, src, pairs, E);
  HB_CHECK_LAUNCH("hb_moe_sort");
  return 0;
}

template <typename TA>
__global__ void __launch_bounds__(128) moe_gather_kernel(const TA* __restrict__ xn, long ldx, const int* __restrict__ src,
                                                         TA* __restrict__ xs, int W, int top) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int r = blockIdx.x, t = src[r] / top;
  for (int i = threadIdx.x; i < W; i += 128) xs[(size_t)r * W + i] = xn[(size_t)t * ldx + i];
}

HB_EXPORT int hb_moe_gather(const void* xn, int x_dt, long ldx, const int* src, void* xs, int pairs, int W, int top,
                            cudaStream_t s) {
  if (pairs <= 0) return 0;
  HB_DISPATCH_1(x_dt, "hb_moe_gather",
                (hb_launch(moe_gather_kernel<TA>, dim3(pairs), dim3(128), 0, s, (const TA*)xn, ldx, src, (TA*)xs, W, top)));
  HB_CHECK_LAUNCH("hb_moe_gather");
  return 0;
}

// gu [rows][g (F) | u (F)] 32-bit, sorted rows; the pair's score enters here
template <typename TO>
__global__ void __launch_bounds__(256) moe_act_kernel(const float* __restrict__ gu, const int* __restrict__ src,
                                                      const float* __restrict__ weight, TO* __restrict__ act, long n, int F,
                                                      int at_output) {
  hb_pdl_launch();
  hb_pdl_wait();
  for (long idx = (long)blockIdx.x * 256 + threadIdx.x; idx < n; idx += (long)gridDim.x * 256) {
    const long r = idx / F;
    const int j = (int)(idx - r * F);
    const float sw = weight[src[r]];
    const float s = at_output ? 1.f : sw, so = at_output ? sw : 1.f;
    const float g = s * gu[r * 2 * F + j], u = s * gu[r * 2 * F + F + j];
    act[idx] = hb_from_float<TO>(g / (1.f + expf(-g)) * u * so);
  }
}

// Four columns a thread (F a multiple of four, aligned rows): the same values.
template <typename TO>
__global__ void __launch_bounds__(256) moe_act_vec_kernel(const float* __restrict__ gu, const int* __restrict__ src,
                                                          const float* __restrict__ weight, TO* __restrict__ act, long n4, int F,
                                                          int at_output) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int F4 = F >> 2;
  for (long idx = (long)blockIdx.x * 256 + threadIdx.x; idx < n4; idx += (long)gridDim.x * 256) {
    const long r = idx / F4;
    const int j = (int)(idx - r * F4) << 2;
    const float sw = weight[src[r]];
    const float s = at_output ? 1.f : sw, so = at_output ? sw : 1.f;
    const float4 gv = *(const float4*)(gu + r * 2 * F + j), uv = *(const float4*)(gu + r * 2 * F + F + j);
    const float g0 = s * gv.x, g1 = s * gv.y, g2 = s * gv.z, g3 = s * gv.w;
    hb_store4(act + r * F + j, make_float4(g0 / (1.f + expf(-g0)) * (s * uv.x) * so, g1 / (1.f + expf(-g1)) * (s * uv.y) * so,
                                           g2 / (1.f + expf(-g2)) * (s * uv.z) * so, g3 / (1.f + expf(-g3)) * (s * uv.w) * so));
  }
}

HB_EXPORT int hb_moe_act(const float* gu, const int* src, const float* weight, void* act, int o_dt, int pairs, int F,
                         int at_output, cudaStream_t s) {
  if (pairs <= 0) return 0;
  if (F % 4 == 0 && !(((uintptr_t)gu | (uintptr_t)act) & 15)) {
    const long n4 = (long)pairs * (F / 4);
    const int blocks4 = (int)((n4 + 255) / 256 < 148 * 16 ? (n4 + 255) / 256 : 148 * 16);
    HB_DISPATCH_1(o_dt, "hb_moe_act",
                  (hb_launch(moe_act_vec_kernel<TA>, dim3(blocks4), dim3(256), 0, s, gu, src, weight, (TA*)act, n4, F, at_output)));
    HB_CHECK_LAUNCH("hb_moe_act");
    return 0;
  }
  const long n = (long)pairs * F;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  HB_DISPATCH_1(o_dt, "hb_moe_act", (hb_launch(moe_act_kernel<TA>, dim3(blocks), dim3(256), 0, s, gu, src, weight, (TA*)act, n, F, at_output)));
  HB_CHECK_LAUNCH("hb_moe_act");
  return 0;
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ ys, const int* __restrict__ pos,
                                                          float* __restrict__ y, long ldy, long n, int W, int top) {
  hb_pdl_launch();
  hb_pdl_wait();
  for (long idx = (long)blockIdx.x * 256 + threadIdx.x; idx < n; idx += (long)gridDim.x * 256) {
    const long t = idx / W;
    const int c = (int)(idx - t * W);
    float acc = 0.f;
    for (int k = 0; k < top; k++) acc += ys[(size_t)pos[t * top + k] * W + c];
    y[t * ldy + c] += acc;
  }
}

HB_EXPORT int hb_moe_combine(const float* ys, const int* pos, float* y, long ldy, int T, int W, int top, cudaStream_t s) {
  if (T <= 0) return 0;
  const long n = (long)T * W;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  hb_launch(moe_combine_kernel, dim3(blocks), dim3(256), 0, s, ys, pos, y, ldy, n, W, top);
  HB_CHECK_LAUNCH("hb_moe_combine");
  return 0;
}
