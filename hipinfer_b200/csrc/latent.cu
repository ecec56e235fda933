// The helpers of latent attention: keys and values of all heads are functions of one latent vector per token, so that
// the cache keeps the latent (R wide) and one rotated key part (Dr wide, shared by all heads) per token, and attention
// runs in the latent's space: with k_h = Wuk_h c and v_h = Wuv_h c,
//     q_h . k_h = (Wuk_h^T q_h) . c          the query is taken into the latent's space, once per row
//     sum_j p_j v_hj = Wuv_h (sum_j p_j c_j)  the values are projected after the sum over keys, once per row
// so a row's attention is one pass over [c | kr] rows with queries R + Dr wide and values the first R columns.
//
// latent_prepare_kernel: from the 32-bit result of the first product (row = [.. cq_raw (Rq) .. c_raw (R) .. kr_raw (Dr) ..])
//   cq = cq_raw / rms(cq_raw) * wq      -> cq_out [T][Rq]
//   c  = c_raw / rms(c_raw) * wc        -> the token's cache row, columns [0, R)
//   kr = rotated(kr_raw)                -> the token's cache row, columns [R, R + Dr)   (pairs (2i, 2i + 1), i < rot / 2,
//                                          with pairing 1; pairs (i, i + rot / 2) with pairing 0)
//   root mean squares with eps inside the root, all 32-bit, rounded once.
// heads_linear_kernel: out[t, h, n] = sum_k a[t, h, k] Wt[h][k][n] (32-bit a, 32-bit sums), optionally times
//   sigmoid(gate[t, h, n]) (or of one number per head, gate[t, h]); and, where asked, the `tail` columns after a's K are
//   rotated the same way and copied behind out's N columns (the rotated part of a query).
#include "common.cuh"

template <typename TW, typename TO>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const float* __restrict__ proj, long ld, int cq_off, int c_off,
                                                             int kr_off, const TW* __restrict__ wq, const TW* __restrict__ wc,
                                                             const int* __restrict__ pos, const int* __restrict__ slot_map,
                                                             const float2* __restrict__ table, int rot, float eps,
                                                             TO* __restrict__ cq_out, TO* __restrict__ cache, int Rq, int R,
                                                             int Dr, int page_size, int pairing) {
  __shared__ float sh[32];
  hb_pdl_launch();
  hb_pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const float* row = proj + (size_t)t * ld;
  float ss = 0.f;
  for (int i = tid; i < Rq; i += 256) ss = fmaf(row[cq_off + i], row[cq_off + i], ss);
  const float fq = rsqrtf(hb_block_sum(ss, sh) / (float)Rq + eps);
  for (int i = tid; i < Rq; i += 256) cq_out[(size_t)t * Rq + i] = hb_from_float<TO>(row[cq_off + i] * fq * hb_to_float(wq[i]));
  const int slot = slot_map ? slot_map[t] : -1;
  if (slot < 0) return;
  ss = 0.f;
  for (int i = tid; i < R; i += 256) ss = fmaf(row[c_off + i], row[c_off + i], ss);
  const float fc = rsqrtf(hb_block_sum(ss, sh) / (float)R + eps);
  TO* dst = cache + (size_t)slot * (R + Dr);      // one head a page: the slot is the row
  for (int i = tid; i < R; i += 256) dst[i] = hb_from_float<TO>(row[c_off + i] * fc * hb_to_float(wc[i]));
  const int half = rot >> 1;
  const float2* cs = table + (size_t)pos[t] * half;
  for (int i = tid; i < half; i += 256) {
    const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
    const float u = row[kr_off + ia], v = row[kr_off + ib];
    const float2 c = cs[i];
    dst[R + ia] = hb_from_float<TO>(__fsub_rn(__fmul_rn(u, c.x), __fmul_rn(v, c.y)));
    dst[R + ib] = hb_from_float<TO>(__fadd_rn(__fmul_rn(v, c.x), __fmul_rn(u, c.y)));
  }
  for (int i = rot + tid; i < Dr; i += 256) dst[R + i] = hb_from_float<TO>(row[kr_off + i]);
}

HB_EXPORT int hb_latent_prepare(const float* proj, long ld, int cq_off, int c_off, int kr_off, const void* wq, const void* wc,
                                int w_dt, const int* pos, const int* slot_map, const void* table, int rot, float eps,
                                void* cq_out, void* cache, int o_dt, int T, int Rq, int R, int Dr, int page_size, int pairing,
                                cudaStream_t s) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > Dr || (rot & 1)) HB_FAIL("hb_latent_prepare: %d rotated dimensions of %d", rot, Dr);
  HB_DISPATCH_2(w_dt, o_dt, "hb_latent_prepare",
                (hb_launch(latent_prepare_kernel<TA, TB>, T, 256, 0, s, proj, ld, cq_off, c_off, kr_off, (const TA*)wq,
                           (const TA*)wc, pos, slot_map, (const float2*)table, rot, eps, (TB*)cq_out, (TB*)cache, Rq, R, Dr,
                           page_size, pairing)));
  HB_CHECK_LAUNCH("hb_latent_prepare");
  return 0;
}

constexpr int HL_TM = 8, HL_THREADS = 128, HL_TN = 32, HL_KZ = HL_THREADS / HL_TN;

// A block owns HL_TM rows, one head and HL_TN output columns; its threads are HL_TN columns x HL_KZ interleaved slices of
// k, summed in a fixed order (slice 0 .. HL_KZ - 1) through shared memory: few rows still fill the machine, and a
// thread's loads of the weight are independent of one another.
template <typename TW, typename TO>
__global__ void __launch_bounds__(HL_THREADS) heads_linear_kernel(const float* __restrict__ a, long lda, long a_head,
                                                                  const TW* __restrict__ wt, TO* __restrict__ out, long ldo,
                                                                  long o_head, int T, int K, int N,
                                                                  const float* __restrict__ gate, long ld_gate, int gate_off,
                                                                  int tail, int rot, const int* __restrict__ pos,
                                                                  const float2* __restrict__ table,
                                                                  const int* __restrict__ row_req,
                                                                  const int* __restrict__ q_len, int row_limit, int pairing,
                                                                  int gate_per_head) {
  extern __shared__ float hl_a[];      // [HL_TM][K + tail], then [HL_KZ][HL_TM][HL_TN] partial sums
  hb_pdl_launch();
  hb_pdl_wait();
  const int h = blockIdx.y, t0 = blockIdx.z * HL_TM, nl = threadIdx.x % HL_TN, kz = threadIdx.x / HL_TN;
  const int n = blockIdx.x * HL_TN + nl;
  const int KT_ = K + tail, rows = min(HL_TM, T - t0);
  float* red = hl_a + HL_TM * KT_;
  // rows of requests that bring row_limit rows or more belong to another path: a block all of whose rows do is idle
  unsigned skip = 0;
  if (q_len)
    for (int r = 0; r < rows; r++) skip |= (q_len[row_req[t0 + r]] >= row_limit ? 1u : 0u) << r;
  if (q_len && skip == (1u << rows) - 1u) return;
  for (int i = threadIdx.x; i < rows * KT_; i += HL_THREADS) {
    const int r = i / KT_, k = i - r * KT_;
    hl_a[r * KT_ + k] = a[(size_t)(t0 + r) * lda + (size_t)h * a_head + k];
  }
  __syncthreads();
  float acc[HL_TM];
#pragma unroll
  for (int r = 0; r < HL_TM; r++) acc[r] = 0.f;
  if (n < N) {
    const TW* w = wt + (size_t)h * K * N + n;
#pragma unroll 4
    for (int k = kz; k < K; k += HL_KZ) {
      const float wv = hb_to_float(w[(size_t)k * N]);
#pragma unroll
      for (int r = 0; r < HL_TM; r++) acc[r] = fmaf(hl_a[r * KT_ + k], wv, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < HL_TM; r++) red[(kz * HL_TM + r) * HL_TN + nl] = acc[r];
  __syncthreads();
  if (n < N) {
    // thread (nl, kz) finishes rows kz, kz + HL_KZ, ...
    for (int r = kz; r < rows; r += HL_KZ) {
      if (skip >> r & 1) continue;
      float o = 0.f;
#pragma unroll
      for (int z = 0; z < HL_KZ; z++) o += red[(z * HL_TM + r) * HL_TN + nl];
      if (gate) o *= 1.f / (1.f + expf(-gate[(size_t)(t0 + r) * ld_gate + gate_off + (gate_per_head ? (size_t)h : (size_t)h * N + n)]));
      out[(size_t)(t0 + r) * ldo + (size_t)h * o_head + n] = hb_from_float<TO>(o);
    }
  } else if (n < N + tail && kz == 0) {
    const int j = n - N, half = rot >> 1;
    for (int r = 0; r < rows; r++) {
      if (skip >> r & 1) continue;
      const float* src = hl_a + r * KT_ + K;
      float y = src[j];
      if (j < rot) {
        const int i = pairing ? j >> 1 : (j < half ? j : j - half);
        const bool second = pairing ? (j & 1) : (j >= half);
        const float2 c = table[(size_t)pos[t0 + r] * half + i];
        const float u = src[pairing ? 2 * i : i], v = src[pairing ? 2 * i + 1 : i + half];
        y = second ? __fadd_rn(__fmul_rn(v, c.x), __fmul_rn(u, c.y)) : __fsub_rn(__fmul_rn(u, c.x), __fmul_rn(v, c.y));
      }
      out[(size_t)(t0 + r) * ldo + (size_t)h * o_head + n] = hb_from_float<TO>(y);
    }
  }
}

// a float32 [T][lda], head h's K (+ tail) inputs at column h * a_head; wt [H][K][N]; out [T][ldo], head h's N (+ tail)
// outputs at column h * o_head.
HB_EXPORT int hb_heads_linear(const float* a, long lda, long a_head, const void* wt, int w_dt, void* out, int o_dt, long ldo,
                              long o_head, int T, int H, int K, int N, const float* gate, long ld_gate, int gate_off, int tail,
                              int rot, const int* pos, const void* table, const int* row_req, const int* q_len, int row_limit,
                              int pairing, int gate_per_head, cudaStream_t s) {
  if (T <= 0 || H <= 0) return 0;
  if (tail && (!pos || !table || rot > tail || (rot & 1))) HB_FAIL("hb_heads_linear: a rotated tail needs positions and a table");
  const size_t smem = ((size_t)HL_TM * (K + tail) + (size_t)HL_KZ * HL_TM * HL_TN) * sizeof(float);
  if (smem > 96 * 1024) HB_FAIL("hb_heads_linear: K = %d is too wide", K);
  if ((T + HL_TM - 1) / HL_TM > 65535 || H > 65535) HB_FAIL("hb_heads_linear: the grid is too large");
  dim3 grid((N + tail + HL_TN - 1) / HL_TN, H, (T + HL_TM - 1) / HL_TM);
#define HL_LAUNCH(TW, TO)                                                                                       \
  do {                                                                                                          \
    auto kern = heads_linear_kernel<TW, TO>;                                                                    \
    if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    hb_launch(kern, grid, dim3(HL_THREADS), smem, s, a, lda, a_head, (const TW*)wt, (TO*)out, ldo, o_head, T, K, N, gate,  \
              ld_gate, gate_off, tail, rot, pos, (const float2*)table, row_req, q_len, row_limit, pairing,     \
              gate_per_head);                                                                                   \
  } while (0)
  HB_DISPATCH_2(w_dt, o_dt, "hb_heads_linear", HL_LAUNCH(TA, TB));
#undef HL_LAUNCH
  HB_CHECK_LAUNCH("hb_heads_linear");
  return 0;
}

// The rows of one request's tokens [0, n) of a cache plane with one head ([page][1][page_size][W]) copied, in the
// order of their positions, into a contiguous buffer [n][W]: the input of a product over a request's whole context.
template <typename TC>
__global__ void __launch_bounds__(256) gather_rows_kernel(const TC* __restrict__ plane, const int* __restrict__ table,
                                                          TC* __restrict__ dst, int n, int W, int page_size) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int vec = 16 / sizeof(TC), cw = W / vec;
  for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < (long)n * cw; i += (long)gridDim.x * 256) {
    const int t = (int)(i / cw), c = (int)(i - (long)t * cw);
    const size_t row = (size_t)table[t / page_size] * page_size + t % page_size;
    ((uint4*)(dst + (size_t)t * W))[c] = ((const uint4*)(plane + row * W))[c];
  }
}

HB_EXPORT int hb_gather_rows(const void* plane, int dt, const int* table, void* dst, int n, int W, int page_size, cudaStream_t s) {
  if (n <= 0) return 0;
  const int esz = dt == HB_F32 ? 4 : 2;
  if ((W * esz) % 16 || (((uintptr_t)plane | (uintptr_t)dst) & 15)) HB_FAIL("hb_gather_rows: rows of %d elements are no whole 16-byte chunks", W);
  const long chunks = (long)n * (W * esz / 16);
  const int blocks = (int)((chunks + 255) / 256 < 2048 ? (chunks + 255) / 256 : 2048);
  HB_DISPATCH_1(dt, "hb_gather_rows", (hb_launch(gather_rows_kernel<TA>, blocks, 256, 0, s, (const TA*)plane, table, (TA*)dst, n, W, page_size)));
  HB_CHECK_LAUNCH("hb_gather_rows");
  return 0;
}
