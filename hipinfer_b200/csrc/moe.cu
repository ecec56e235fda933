// A routed feed-forward (mixture of experts): every token runs `top` of E small gated feed-forward layers.
//     z = Wr h (32-bit);  s = sigmoid(z);  the `top` largest s choose the experts (ties: the lower index)
//     out = sum over the chosen e of Wd_e (silu(Wg_e v) * (Wu_e v)),  v = s_e h
// The score multiplies the expert's INPUT. Experts have no biases, so Wg_e (s h) = s (Wg_e h): the products run on h and
// the score enters the activation in 32-bit, silu(s g) * (s u).
//
// moe_route_kernel          scores and the chosen experts of every row: expert [T][top], weight [T][top]
// Few rows (decoding): no sorting, nothing on the host
//   moe_gate_up_rows_kernel a block per ((row, choice), tile of the expert's hidden rows): act [T * top][F]
//   moe_down_rows_kernel    a block per (row, tile of output columns): the choices' results summed in their order
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
                                                               int* __restrict__ expert, float* __restrict__ weight, int W,
                                                               int E, int top) {
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
    if (lane == 0) sc[e] = 1.f / (1.f + expf(-acc));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 0; k < top; k++) {
      int best = 0;
      float bs = -2.f;
      for (int e = 0; e < E; e++)
        if (sc[e] > bs) {
          bs = sc[e];
          best = e;
        }
      expert[(size_t)t * top + k] = best;
      weight[(size_t)t * top + k] = bs;
      sc[best] = -1.f;                 // scores lie in [0, 1]: a taken expert is never the largest again
    }
  }
}

HB_EXPORT int hb_moe_route(const void* xn, int x_dt, long ldx, const void* router, int w_dt, int* expert, float* weight, int T,
                           int W, int E, int top, cudaStream_t s) {
  if (T <= 0) return 0;
  if (top < 1 || top > E) HB_FAIL("hb_moe_route: top %d of %d experts", top, E);
  const size_t smem = (size_t)(W + E) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_moe_route: a row of %d with %d experts does not fit shared memory", W, E);
  HB_DISPATCH_2(x_dt, w_dt, "hb_moe_route", do {
    auto kern = moe_route_kernel<TA, TB>;
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(kern, dim3(T), dim3(MR_THREADS), smem, s, (const TA*)xn, ldx, (const TB*)router, expert, weight, W, E, top);
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
                                                                      int W, int F, int top, int vec) {
  extern __shared__ __align__(16) float mg_row[];      // [W]
  hb_pdl_launch();
  hb_pdl_wait();
  const int pair = blockIdx.y, t = pair / top, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < W; i += MG_THREADS) mg_row[i] = hb_to_float(xn[(size_t)t * ldx + i]);
  __syncthreads();
  const int e = expert[pair];
  const float s = weight[pair];
  const TW* we = wgu + (size_t)e * 2 * F * W;          // [gate rows (F) | up rows (F)][W]
  const int j1 = min(F, (int)(blockIdx.x + 1) * MG_ROWS);
  for (int j = blockIdx.x * MG_ROWS + warp; j < j1; j += MG_THREADS / 32) {
    const float g = s * moe_warp_dot(we + (size_t)j * W, mg_row, W, lane, vec);
    const float u = s * moe_warp_dot(we + (size_t)(F + j) * W, mg_row, W, lane, vec);
    if (lane == 0) act[(size_t)pair * F + j] = hb_from_float<TO>(g / (1.f + expf(-g)) * u);
  }
}

HB_EXPORT int hb_moe_gate_up_rows(const void* xn, int x_dt, long ldx, const void* wgu, int w_dt, const int* expert,
                                  const float* weight, void* act, int T, int W, int F, int top, cudaStream_t s) {
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
    hb_launch(kern, grid, dim3(MG_THREADS), smem, s, (const TA*)xn, ldx, (const TB*)wgu, expert, weight, (TA*)act, W, F, top, vec);
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
                                                      const float* __restrict__ weight, TO* __restrict__ act, long n, int F) {
  hb_pdl_launch();
  hb_pdl_wait();
  for (long idx = (long)blockIdx.x * 256 + threadIdx.x; idx < n; idx += (long)gridDim.x * 256) {
    const long r = idx / F;
    const int j = (int)(idx - r * F);
    const float s = weight[src[r]];
    const float g = s * gu[r * 2 * F + j], u = s * gu[r * 2 * F + F + j];
    act[idx] = hb_from_float<TO>(g / (1.f + expf(-g)) * u);
  }
}

HB_EXPORT int hb_moe_act(const float* gu, const int* src, const float* weight, void* act, int o_dt, int pairs, int F,
                         cudaStream_t s) {
  if (pairs <= 0) return 0;
  const long n = (long)pairs * F;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  HB_DISPATCH_1(o_dt, "hb_moe_act", (hb_launch(moe_act_kernel<TA>, dim3(blocks), dim3(256), 0, s, gu, src, weight, (TA*)act, n, F)));
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
