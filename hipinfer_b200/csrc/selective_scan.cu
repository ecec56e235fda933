// The selective state-space recurrence with a decay per (channel, state) pair (the Mamba-1 form), and the sum that
// joins two side-by-side mixers.
//
// Per token, for every channel c of `inner` and state n of N, with the step's 32-bit inputs x [T][inner] (after the short
// convolution and silu), dt_raw [T][inner] (the step-size product without its bias), B and C [T][N] (shared by all
// channels) and the gate's pre-activation z [T][inner]:
//     dt = softplus(dt_raw + dt_bias_c);  A = -exp(A_log[c][n])
//     S[c][n] <- exp(dt A) S[c][n] + (dt x_c) B_n;   y_c = sum_n S[c][n] C_n + D_c x_c;   out_c = y_c * silu(z_c)
// The state S [inner][N] lives in 32-bit in the request's state slot and is carried from token to token and from step to
// step; step sizes, decays, the exponentials and the sums are 32-bit (expf, exp2f, log1pf; no fast-math), the result is
// rounded once. A block owns (a tile of channels, a request) and walks the request's rows of the step in order: KS threads share a
// channel, thread ks holds the states n = ks + i KS in registers, the KS partial sums of y are joined by shuffles. Tokens
// go by in chunks of SEL_CH: a chunk's rows are asked for a chunk ahead (cp.async, two buffers), the step sizes are
// finished in place, the chunk's results leave through shared memory in whole rows, where the gate multiplies them. Requests, lengths and state slots come
// from device arrays, so a decode-only step replays from a CUDA graph; a token's arithmetic does not depend on where a
// portion or a chunk starts.
//   Long portions run in three launches over pieces of L tokens instead, so that one long prompt fills the GPU: every piece
// from a zero state (what it adds itself, and the sum of its step sizes, whose exponential times the rate is the product
// of its decays), then the pieces' starting states one after another (selective_carry_kernel), then every piece again from
// its starting state for the results. The walk is the same code in all three; the two ways differ by rounding only.
#include "common.cuh"

constexpr int SEL_CH = 16;         // tokens a chunk
constexpr int SEL_THREADS = 64;

__device__ __forceinline__ void sel_cp4(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void sel_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void sel_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float sel_softplus(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }
// exp(dt * A) as 2^(dt * (A log2 e)): the rate comes multiplied by log2(e) once, a decay is one product and one exp2f
__device__ __forceinline__ float sel_decay(float dt, float rate2) { return exp2f(dt * rate2); }
constexpr float SEL_LOG2E = 1.4426950408889634f;

struct SelArgs {
  const float* x; long ldx;          // [T][inner] after convolution and silu
  const float* dt; long lddt;        // [T][inner] step-size product, no bias
  const float* bc; long ldbc;        // a row holds B [N] then C [N]
  const float* z; long ldz;          // [T][inner] gate pre-activation
  const void* dt_bias; const void* a_log; const void* d_skip;   // [inner], [inner][N], [inner]
  float* state;                      // [slots][inner][N]
  const int* q_start; const int* q_len; const int* slot;
  void* out; long ldo;               // [T][inner]
  int inner, N, KS;
  int L;                             // tokens a piece (the three-launch form)
  float* piece_state;                // [all requests' pieces][inner][N]
  float* piece_dt;                   // [all requests' pieces][inner]: the sum of a piece's step sizes
};

enum { SEL_WHOLE = 0, SEL_PIECE_LOCAL = 1, SEL_PIECE_OUT = 2 };

// The first piece of request r among all requests' pieces: every request before it has ceil(len / L) of them.
__device__ __forceinline__ int sel_piece_base(const int* q_len, int r, int L) {
  int base = 0;
  for (int i = 0; i < r; i++) base += (q_len[i] + L - 1) / L;
  return base;
}

// shared memory of a block: two buffers of a chunk's rows, each [SEL_CH][2N + 3 CPB]: B | C | dt | x | z (z becomes the result)
template <typename TW, typename TO, int NPT, int MODE>
__global__ void __launch_bounds__(SEL_THREADS) selective_scan_kernel(SelArgs A) {
  extern __shared__ float sel_sm[];
  hb_pdl_launch();
  const int KS = A.KS, CPB = SEL_THREADS / KS, N = A.N;
  const int cl = threadIdx.x / KS, ks = threadIdx.x % KS;
  const int c0 = blockIdx.x * CPB, c = c0 + cl, r = blockIdx.y;
  const bool live = c < A.inner;
  const int nch = min(CPB, A.inner - c0);
  const int row_w = 2 * N + 3 * CPB;
  float* buf[2] = {sel_sm, sel_sm + SEL_CH * row_w};
  // constants of the thread: its decays' rates, the skip weight and the bias (weights: before the wait)
  float rate[NPT], S[NPT];
  const TW* al = (const TW*)A.a_log;
#pragma unroll
  for (int i = 0; i < NPT; i++) {
    const int n = ks + i * KS;
    rate[i] = (live && n < N) ? -expf(hb_to_float(al[(size_t)c * N + n])) * SEL_LOG2E : 0.f;
  }
  const float dskip = live ? hb_to_float(((const TW*)A.d_skip)[c]) : 0.f;
  hb_pdl_wait();
  int len = A.q_len[r], t0 = A.q_start[r];
  float* st;
  size_t piece = 0;
  if (MODE == SEL_WHOLE) {
    if (len <= 0) return;
    st = A.state + ((size_t)A.slot[r] * A.inner + (live ? c : 0)) * N;
  } else {
    // this block's piece: tokens [z L, z L + L) of the request, the walk below sees them as a portion of their own
    const int j_first = blockIdx.z * A.L;
    if (j_first >= len) return;
    piece = (size_t)sel_piece_base(A.q_len, r, A.L) + blockIdx.z;
    st = A.piece_state + (piece * A.inner + (live ? c : 0)) * N;
    t0 += j_first;
    len = min(A.L, len - j_first);
  }
  float sum_dt = 0.f;
#pragma unroll
  for (int i = 0; i < NPT; i++) {
    const int n = ks + i * KS;
    S[i] = (MODE != SEL_PIECE_LOCAL && live && n < N) ? st[n] : 0.f;
  }
  if (MODE == SEL_WHOLE && len == 1) {
    // a single token (decoding): no staging; a thread asks for all it needs at once, beside its states above. The same
    // operations in the same order as the walk below: the same bits.
    const size_t t = (size_t)t0;
    float dtr = 0.f, xv = 0.f, zz = 0.f, Bn[NPT], Cn[NPT];
    if (live) {
      dtr = A.dt[t * A.lddt + c];
      xv = A.x[t * A.ldx + c];
      zz = A.z[t * A.ldz + c];
    }
#pragma unroll
    for (int i = 0; i < NPT; i++) {
      const int n = ks + i * KS;
      Bn[i] = n < N ? A.bc[t * A.ldbc + n] : 0.f;
      Cn[i] = n < N ? A.bc[t * A.ldbc + N + n] : 0.f;
    }
    const float dtv = sel_softplus(dtr + (live ? hb_to_float(((const TW*)A.dt_bias)[c]) : 0.f));
    const float dx = dtv * xv;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NPT; i++) {
      const int n = ks + i * KS;
      if (n < N) {
        S[i] = fmaf(sel_decay(dtv, rate[i]), S[i], dx * Bn[i]);
        acc = fmaf(S[i], Cn[i], acc);
      }
    }
    for (int o = KS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (live) {
      if (ks == 0) ((TO*)A.out)[t * A.ldo + c] = hb_from_float<TO>(fmaf(dskip, xv, acc) * (zz / (1.f + expf(-zz))));
#pragma unroll
      for (int i = 0; i < NPT; i++) {
        const int n = ks + i * KS;
        if (n < N) st[n] = S[i];
      }
    }
    return;
  }
  // how the block's threads tile a chunk's (token, channel) pairs: CPB is a power of two, so no division anywhere
  const int cshift = __ffs(CPB) - 1, kk = threadIdx.x & (CPB - 1), jj = threadIdx.x >> cshift, jstep = SEL_THREADS >> cshift;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  auto fetch = [&](int j0, float* b) {
    const int n = min(SEL_CH, len - j0);
    const int nbc = MODE == SEL_PIECE_LOCAL ? N : 2 * N;          // a piece from a zero state needs no C
    for (int j = wrp; j < n; j += SEL_THREADS / 32) {
      const float* src = A.bc + (size_t)(t0 + j0 + j) * A.ldbc;
      for (int k = lane; k < nbc; k += 32) sel_cp4(b + j * row_w + k, src + k);
    }
    if (kk < nch) {
      for (int j = jj; j < n; j += jstep) {
        const size_t t = (size_t)(t0 + j0 + j);
        float* row = b + j * row_w + 2 * N;
        sel_cp4(row + kk, A.dt + t * A.lddt + c0 + kk);
        sel_cp4(row + CPB + kk, A.x + t * A.ldx + c0 + kk);
        if (MODE != SEL_PIECE_LOCAL) sel_cp4(row + 2 * CPB + kk, A.z + t * A.ldz + c0 + kk);
      }
    }
    sel_commit();
  };
  fetch(0, buf[0]);
  const float my_bias = kk < nch ? hb_to_float(((const TW*)A.dt_bias)[c0 + kk]) : 0.f;
  int which = 0;
  for (int j0 = 0; j0 < len; j0 += SEL_CH, which ^= 1) {
    float* b = buf[which];
    const int n_tok = min(SEL_CH, len - j0);
    if (j0 + SEL_CH < len) {
      fetch(j0 + SEL_CH, buf[which ^ 1]);
      sel_wait<1>();
    } else {
      sel_wait<0>();
    }
    __syncthreads();
    // the step sizes, once per (token, channel)
    if (kk < nch) {
      for (int j = jj; j < n_tok; j += jstep) {
        float* p = b + j * row_w + 2 * N + kk;
        *p = sel_softplus(*p + my_bias);
      }
    }
    __syncthreads();
    for (int j = 0; j < n_tok; j++) {
      const float* row = b + j * row_w;
      const float dtv = row[2 * N + cl], xv = row[2 * N + CPB + cl];
      const float dx = dtv * xv;
      if (MODE == SEL_PIECE_LOCAL) sum_dt += dtv;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPT; i++) {
        const int n = ks + i * KS;
        if (n < N) {
          S[i] = fmaf(sel_decay(dtv, rate[i]), S[i], dx * row[n]);
          if (MODE != SEL_PIECE_LOCAL) acc = fmaf(S[i], row[N + n], acc);
        }
      }
      if (MODE != SEL_PIECE_LOCAL) {
        for (int o = KS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        // y takes the place of x (every lane of the channel has read x: the warp meets in between); the gate comes
        // in the pass below, where every thread has an element of its own
        __syncwarp();
        if (ks == 0) b[j * row_w + 2 * N + CPB + cl] = fmaf(dskip, xv, acc);
      }
    }
    __syncthreads();
    if (MODE != SEL_PIECE_LOCAL) {
      TO* out = (TO*)A.out;
      if (kk < nch) {
        for (int j = jj; j < n_tok; j += jstep) {
          const float* row = b + j * row_w + 2 * N;
          const float zz = row[2 * CPB + kk];
          out[(size_t)(t0 + j0 + j) * A.ldo + c0 + kk] = hb_from_float<TO>(row[CPB + kk] * (zz / (1.f + expf(-zz))));
        }
      }
      __syncthreads();     // the buffer is asked for again two chunks on
    }
  }
  if (MODE == SEL_PIECE_LOCAL && live && ks == 0) A.piece_dt[piece * A.inner + c] = sum_dt;
  if (MODE != SEL_PIECE_OUT && live) {
#pragma unroll
    for (int i = 0; i < NPT; i++) {
      const int n = ks + i * KS;
      if (n < N) st[n] = S[i];
    }
  }
}

// The pieces' starting states, one after another: an element (channel, state) of a request walks its pieces, leaves in each
// the state the piece starts from and carries exp(rate * the piece's summed step sizes) * state + the piece's own
// contribution on; the last goes to the request's slot.
template <typename TW>
__global__ void __launch_bounds__(256) selective_carry_kernel(SelArgs A) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int r = blockIdx.y, N = A.N;
  const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x, IN = (size_t)A.inner * N;
  if (e >= IN) return;
  const int len = A.q_len[r];
  if (len <= 0) return;
  const int c = (int)(e / N), pieces = (len + A.L - 1) / A.L;
  const float rate = -expf(hb_to_float(((const TW*)A.a_log)[e])) * SEL_LOG2E;
  float* slot = A.state + (size_t)A.slot[r] * IN + e;
  float carry = *slot;
  const size_t base = (size_t)sel_piece_base(A.q_len, r, A.L);
  float* ps = A.piece_state + base * IN + e;
  const float* pd = A.piece_dt + base * A.inner + c;
  for (int k0 = 0; k0 < pieces; k0 += 8) {                 // eight pieces' loads in flight, then their chain
    float own[8], dec[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const bool in = k0 + i < pieces;
      own[i] = in ? ps[(size_t)(k0 + i) * IN] : 0.f;
      dec[i] = in ? sel_decay(pd[(size_t)(k0 + i) * A.inner], rate) : 1.f;
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      if (k0 + i < pieces) {
        ps[(size_t)(k0 + i) * IN] = carry;
        carry = fmaf(dec[i], carry, own[i]);
      }
    }
  }
  *slot = carry;
}

// x, dt, z float32 [T][inner] (row strides ldx, lddt, ldz), bc float32 rows of B [N] | C [N] (stride ldbc); dt_bias [inner],
// a_log [inner][N], d_skip [inner] in the element type w_dt; state float32 [slots][inner][N]; out [T][inner] in o_dt.
// pieces > 0: the three-launch form over pieces of piece_len tokens, no request with more than `pieces` of them, with room
// for all requests' pieces (at most rows / piece_len + n_requests) in piece_state [.][inner][N] and piece_dt [.][inner].
HB_EXPORT int hb_selective_scan(const float* x, long ldx, const float* dt, long lddt, const float* bc, long ldbc, const float* z,
                                long ldz, const void* dt_bias, const void* a_log, const void* d_skip, int w_dt, float* state,
                                const int* q_start, const int* q_len, const int* slot, void* out, int o_dt, long ldo,
                                int n_requests, int inner, int N, int piece_len, int pieces, float* piece_state,
                                float* piece_dt, cudaStream_t s) {
  if (n_requests <= 0 || inner <= 0) return 0;
  if (pieces > 0 && (piece_len <= 0 || !piece_state || !piece_dt || pieces > 65535)) HB_FAIL("hb_selective_scan: %d pieces of %d", pieces, piece_len);
  if (N < 1 || N > 256) HB_FAIL("hb_selective_scan: %d states a channel (1 to 256 are supported)", N);
  int KS = 1;
  while (KS < 32 && (N + KS - 1) / KS > 4) KS <<= 1;
  const int npt = (N + KS - 1) / KS, CPB = SEL_THREADS / KS;
  SelArgs A = {x, ldx, dt, lddt, bc, ldbc, z, ldz, dt_bias, a_log, d_skip, state, q_start, q_len, slot, out, ldo, inner, N, KS,
               piece_len, piece_state, piece_dt};
  dim3 grid((inner + CPB - 1) / CPB, n_requests, pieces > 0 ? pieces : 1);
  if (grid.y > 65535) HB_FAIL("hb_selective_scan: the grid is too large");
  const size_t smem = (size_t)2 * SEL_CH * (2 * N + 3 * CPB) * sizeof(float);
#define SEL_LAUNCH_MODE(NPT, MODE)                                                                           \
  HB_DISPATCH_2(w_dt, o_dt, "hb_selective_scan", do {                                                        \
    auto kern = selective_scan_kernel<TA, TB, NPT, MODE>;                                                    \
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    hb_launch(kern, grid, dim3(SEL_THREADS), smem, s, A);                                                    \
  } while (0))
#define SEL_LAUNCH(MODE)                     \
  do {                                       \
    if (npt <= 1) SEL_LAUNCH_MODE(1, MODE);  \
    else if (npt <= 2) SEL_LAUNCH_MODE(2, MODE); \
    else if (npt <= 4) SEL_LAUNCH_MODE(4, MODE); \
    else SEL_LAUNCH_MODE(8, MODE);           \
  } while (0)
  if (pieces <= 0) {
    SEL_LAUNCH(SEL_WHOLE);
  } else {
    SEL_LAUNCH(SEL_PIECE_LOCAL);
    HB_CHECK_LAUNCH("hb_selective_scan");
    const size_t elems = (size_t)inner * N;
    HB_DISPATCH_1(w_dt, "hb_selective_scan",
                  (hb_launch(selective_carry_kernel<TA>, dim3((unsigned)((elems + 255) / 256), n_requests), dim3(256), 0, s, A)));
    HB_CHECK_LAUNCH("hb_selective_scan");
    SEL_LAUNCH(SEL_PIECE_OUT);
  }
#undef SEL_LAUNCH
#undef SEL_LAUNCH_MODE
  HB_CHECK_LAUNCH("hb_selective_scan");
  return 0;
}

// A 32-bit matrix as the sum of two bfloat16 matrices, hi = round(a) and lo = round(a - hi): two tensor-core products
// with them, added in 32-bit, carry 16 bits of a's mantissa instead of 8 (the low-rank step sizes into their product).
__global__ void __launch_bounds__(256) split_rounded_kernel(const float* __restrict__ a, long lda, __nv_bfloat16* __restrict__ hi,
                                                            __nv_bfloat16* __restrict__ lo, long n, int K) {
  hb_pdl_launch();
  hb_pdl_wait();
  for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long)gridDim.x * 256) {
    const long r = i / K;
    const float v = a[r * lda + (i - r * K)];
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
  }
}

// a float32 [M][K] with row stride lda; hi, lo bfloat16 [M][K] contiguous.
HB_EXPORT int hb_split_rounded(const float* a, long lda, void* hi, void* lo, int M, int K, cudaStream_t s) {
  if (M <= 0 || K <= 0) return 0;
  const long n = (long)M * K;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  hb_launch(split_rounded_kernel, dim3(blocks), dim3(256), 0, s, a, lda, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, n, K);
  HB_CHECK_LAUNCH("hb_split_rounded");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// The residual row after a sublayer, in one pass:
//     u = y                                                        a sublayer's plain result (or nothing)
//       + mix * (a / rms(a) * wa + b / rms(b) * wb)                two side-by-side results, each normed over the row first
//     v = alpha * x + u
//     x <- v / rms(v) * w       (w given: the norm AFTER the sum, its weight as stored, or as one plus what is stored;
//                                no w: x <- v)
// and, where asked, a copy of the new x in the compute element type for the products that read it next. Root mean squares
// with eps inside the root; everything 32-bit; one block a row, the row kept in shared memory between the passes.
// ---------------------------------------------------------------------------------------------------------------------
template <typename TW, typename TO>
__global__ void __launch_bounds__(256) residual_norm_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                            const float* __restrict__ a, const float* __restrict__ b,
                                                            const TW* __restrict__ wa, const TW* __restrict__ wb, float mix,
                                                            float pair_eps, float alpha, const float* __restrict__ w,
                                                            float eps, TO* __restrict__ xb, int W) {
  extern __shared__ float rn_row[];      // [W], then 32 floats for the sums, then (a pair) [W] and [W]
  float* red = rn_row + W;
  float* sa_row = red + 32;
  float* sb_row = sa_row + W;
  hb_pdl_launch();
  hb_pdl_wait();
  const size_t base = (size_t)blockIdx.x * W;
  float fa = 0.f, fb = 0.f;
  if (a) {
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < W; i += 256) {
      const float va = a[base + i], vb = b[base + i];
      sa_row[i] = va;
      sb_row[i] = vb;
      sa = fmaf(va, va, sa);
      sb = fmaf(vb, vb, sb);
    }
    fa = rsqrtf(hb_block_sum(sa, red) / (float)W + pair_eps);
    fb = rsqrtf(hb_block_sum(sb, red) / (float)W + pair_eps);
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += 256) {
    float u = y ? y[base + i] : 0.f;
    if (a) u += mix * (sa_row[i] * fa * hb_to_float(wa[i]) + sb_row[i] * fb * hb_to_float(wb[i]));
    const float v = fmaf(alpha, x[base + i], u);
    rn_row[i] = v;
    ss = fmaf(v, v, ss);
  }
  float f = 1.f;
  if (w) f = rsqrtf(hb_block_sum(ss, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += 256) {
    const float v = w ? rn_row[i] * f * w[i] : rn_row[i];
    x[base + i] = v;
    if (xb) xb[base + i] = hb_from_float<TO>(v);
  }
}

// x float32 [T][W] in place; y, a, b float32 [T][W] or null (a and b together); wa, wb [W] in pw_dt; w float32 [W] or null;
// xb [T][W] in xb_dt or null.
HB_EXPORT int hb_residual_norm(float* x, const float* y, const float* a, const float* b, const void* wa, const void* wb,
                               int pw_dt, float mix, float pair_eps, float alpha, const float* w, float eps, void* xb,
                               int xb_dt, int T, int W, cudaStream_t s) {
  if (T <= 0) return 0;
  if ((a != nullptr) != (b != nullptr) || (a && (!wa || !wb))) HB_FAIL("hb_residual_norm: a pair needs both rows and both weights");
  const size_t smem = (size_t)((a ? 3 : 1) * W + 32) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_residual_norm: a row of %d does not fit shared memory", W);
  if (!a) pw_dt = HB_F32;
  if (!xb) xb_dt = HB_F32;
  HB_DISPATCH_2(pw_dt, xb_dt, "hb_residual_norm", do {
    auto kern = residual_norm_kernel<TA, TB>;
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(kern, dim3(T), dim3(256), smem, s, x, y, a, b, (const TA*)wa, (const TA*)wb, mix, pair_eps, alpha, w, eps, (TB*)xb, W);
  } while (0));
  HB_CHECK_LAUNCH("hb_residual_norm");
  return 0;
}
