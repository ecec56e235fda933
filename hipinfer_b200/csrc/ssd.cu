// The state-space mixer with a scalar decay per head (state-space duality), in three kernels.
//
// From one 32-bit projection result per token, [z (H P) | x (H P) | B (G N) | C (G N) | dt (H)]:
//   ssd_conv_kernel       (x, B, C) <- silu(causal convolution over the token axis, K taps a channel, + bias); the last K - 1
//                         raw inputs of a request are carried in its state slot, zeros before the sequence
//   ssd_scan_kernel       per head h (group g = h / (H / G)), with a state S [N][P] carried in 32-bit from token to token:
//                             dt = softplus(dt_raw + dt_bias_h);  a = exp(-exp(A_log_h) dt)
//                             S <- a S + (dt B_g) x_h^T;  y = S^T C_g + D_h x_h
//   ssd_gate_norm_kernel  y <- y silu(z), then the row in `parts` equal parts, each divided by its own root mean square
//                         (eps inside the root) and multiplied by a weight; rounded once
//   Long portions run the recurrence in three launches instead, over pieces of L tokens: every piece from a zero state
//   (its own contribution and the product of its decays), then the pieces' starting states one after another
//   (ssd_carry_kernel), then every piece again from its starting state for y. The walk is the same code in all three.
// Everything here is 32-bit. Requests, lengths and state slots come from device arrays, so a decode step can be replayed
// from a CUDA graph; where a portion or a piece starts changes a token's result by rounding only.
#include "common.cuh"

constexpr int SC_TAPS_MAX = 16;    // most convolution taps (the kernel is built for up to 8 and for up to 16)
constexpr int SC_CHUNK = 64;       // tokens a block of the convolution walks
constexpr int SC_THREADS = 128;

// grid (channel tiles, requests, token chunks); a thread owns a channel and walks its chunk's tokens with the K - 1 raw
// inputs before them in registers. Only the block of a request's first chunk reads the carried inputs, and it alone writes
// the new ones, after it has read the old: nothing else in the launch touches them.
template <typename TW, int TAPS>
__global__ void __launch_bounds__(SC_THREADS) ssd_conv_kernel(const float* __restrict__ proj, long ld, int off,
                                                              const TW* __restrict__ w, const TW* __restrict__ bias,
                                                              float* __restrict__ carried, const int* __restrict__ q_start,
                                                              const int* __restrict__ q_len, const int* __restrict__ slot,
                                                              float* __restrict__ out, int C, int K) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int c = blockIdx.x * SC_THREADS + threadIdx.x, r = blockIdx.y;
  const int len = q_len[r], j0 = blockIdx.z * SC_CHUNK;
  if (c >= C || j0 >= len) return;
  const int t0 = q_start[r], K1 = K - 1;
  float* st = carried + (size_t)slot[r] * K1 * C + c;          // [K - 1][C], oldest first
  float wk[TAPS], hist[TAPS], old[TAPS];
#pragma unroll
  for (int k = 0; k < TAPS; k++) wk[k] = k < K ? hb_to_float(w[(size_t)c * K + k]) : 0.f;
  const float bs = hb_to_float(bias[c]);
  const float* in = proj + (size_t)t0 * ld + off + c;
  // hist[i]: the raw input i + 1 tokens before the current one
#pragma unroll
  for (int i = 0; i < TAPS - 1; i++) {
    old[i] = (blockIdx.z == 0 && i < K1) ? st[(size_t)i * C] : 0.f;
    hist[i] = 0.f;
  }
#pragma unroll
  for (int i = 0; i < TAPS - 1; i++) {
    if (i < K1) {
      const int j = j0 - 1 - i;
      if (j >= 0) hist[i] = in[(size_t)j * ld];
      else {
        float v = 0.f;                                         // old[K1 + j], a dynamic index kept out of local memory
#pragma unroll
        for (int q = 0; q < TAPS - 1; q++) v = (q == K1 + j) ? old[q] : v;
        hist[i] = v;
      }
    }
  }
  const int n = min(SC_CHUNK, len - j0);
  for (int j = 0; j < n; j++) {
    const float cur = in[(size_t)(j0 + j) * ld];
    float acc = bs;
#pragma unroll
    for (int i = TAPS - 2; i >= 0; i--)
      if (i < K1) acc = fmaf(wk[K1 - 1 - i], hist[i], acc);    // tap k multiplies the input K - 1 - k tokens back
    acc = fmaf(wk[K1], cur, acc);
    out[(size_t)(t0 + j0 + j) * C + c] = acc / (1.f + expf(-acc));
#pragma unroll
    for (int i = TAPS - 2; i > 0; i--) hist[i] = hist[i - 1];
    hist[0] = cur;
  }
  if (blockIdx.z == 0) {
    for (int k = 0; k < K1; k++) {
      const int j = len - K1 + k;                              // relative index of the input that becomes carried[k]
      float v;
      if (j >= 0) v = in[(size_t)j * ld];
      else {
        v = 0.f;
#pragma unroll
        for (int q = 0; q < TAPS - 1; q++) v = (q == K1 + j) ? old[q] : v;
      }
      st[(size_t)k * C] = v;
    }
  }
}

HB_EXPORT int hb_ssd_conv(const float* proj, long ld, int off, const void* w, const void* bias, int w_dt, float* carried,
                          const int* q_start, const int* q_len, const int* slot, float* out, int n_requests, int max_q_len,
                          int C, int K, cudaStream_t s) {
  if (n_requests <= 0 || max_q_len <= 0) return 0;
  if (K < 1 || K > SC_TAPS_MAX) HB_FAIL("hb_ssd_conv: %d taps (1 to %d are supported)", K, SC_TAPS_MAX);
  dim3 grid((C + SC_THREADS - 1) / SC_THREADS, n_requests, (max_q_len + SC_CHUNK - 1) / SC_CHUNK);
  if (grid.y > 65535 || grid.z > 65535) HB_FAIL("hb_ssd_conv: the grid is too large");
  if (K <= 8) {
    HB_DISPATCH_1(w_dt, "hb_ssd_conv",
                  (hb_launch(ssd_conv_kernel<TA, 8>, grid, dim3(SC_THREADS), 0, s, proj, ld, off, (const TA*)w, (const TA*)bias, carried,
                             q_start, q_len, slot, out, C, K)));
  } else {
    HB_DISPATCH_1(w_dt, "hb_ssd_conv",
                  (hb_launch(ssd_conv_kernel<TA, 16>, grid, dim3(SC_THREADS), 0, s, proj, ld, off, (const TA*)w, (const TA*)bias, carried,
                             q_start, q_len, slot, out, C, K)));
  }
  HB_CHECK_LAUNCH("hb_ssd_conv");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// The recurrence. A block owns (head, request) and walks the request's rows of the step in order, from and into its state
// slot. The state lives in registers: KS threads share a value channel p, thread ks holds the state channels n = i KS + ks.
// Tokens go by in chunks of SS_CH: a chunk's rows (x of the head, B and C of its group, dt) are asked for a chunk ahead
// (cp.async), what does not depend on the state (dt, the decay, dt B) is prepared in place, the walk reads it by
// broadcast.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int SS_CH = 16;

struct SsdArgs {
  const float* xbc; long ldx;            // after the convolution: [T][H P | G N | G N]
  const float* dt; long lddt;            // raw dt, [T][.. H ..] (already offset to its first column)
  const void* dt_bias; const void* a_log; const void* d_skip;   // [H] each
  float* state;                          // [slots][H][N][P]
  const int* q_start; const int* q_len; const int* slot;
  float* y;                              // [T][H P]
  int H, P, N, G, KS, vec4;
  float* piece_state;                    // pieces only: [all requests' pieces, request after request][H][N][P]
  float* piece_decay;                    // pieces only: [all requests' pieces][H]
  int L, pieces;                         // tokens a piece, most pieces a request
};

// The first piece of request r among all requests' pieces: requests lie one after another, each with as many pieces as
// its rows need, so a step of one long portion beside many single tokens holds few pieces.
__device__ __forceinline__ int ss_piece_base(const int* __restrict__ q_len, int r, int L) {
  int base = 0;
  for (int i = 0; i < r; i++) base += (q_len[i] + L - 1) / L;
  return base;
}

// MODE of the walk: whole portions from and into the state slot; a piece from zero (no y; leaves its state and the product
// of its decays); a piece from its starting state (y only).
enum { SS_WHOLE = 0, SS_PIECE_LOCAL = 1, SS_PIECE_OUT = 2 };

__device__ __forceinline__ void ss_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ss_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int DPT> struct SsdThreads { static constexpr int MAX = DPT <= 8 ? 1024 : DPT <= 32 ? 512 : 256; };

// FAST: N == DPT * KS with 16-byte aligned rows of multiples of four. A thread then holds the DPT CONTIGUOUS state channels
// ks * DPT .. of its value channel and reads their dt B and C four at a time (B and C lie in shared memory with 4 floats of
// padding after every DPT, so that the KS slices fall on different banks); no bounds are checked and every offset is a
// constant. Otherwise (any sizes) a thread holds every KS-th state channel.
template <int DPT, typename TW, int MODE, bool FAST>
__global__ void __launch_bounds__(SsdThreads<DPT>::MAX, 1) ssd_scan_kernel(SsdArgs A) {
  extern __shared__ __align__(16) float ssm[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
  const int H = A.H, P = A.P, N = A.N, KS = A.KS;
  const int g = h / (H / A.G);
  const int p = tid / KS, ks = tid - p * KS;
  const bool live = p < P;
  const int t0 = A.q_start[r];
  const int j_begin = MODE == SS_WHOLE ? 0 : (int)blockIdx.z * A.L;
  const int len = MODE == SS_WHOLE ? A.q_len[r] : min(A.q_len[r], j_begin + A.L);      // the walk ends here
  if (MODE != SS_WHOLE && j_begin >= len) return;
  float* S_g = MODE == SS_WHOLE ? A.state + ((size_t)A.slot[r] * H + h) * N * P
                                : A.piece_state + (((size_t)ss_piece_base(A.q_len, r, A.L) + blockIdx.z) * H + h) * N * P;
  // a token's row in shared memory: [B -> dt B (NQ) | C (NQ) | x (P) | dt_raw -> decay (1) | pad], two chunks deep
  const int NQ = FAST ? N + 4 * KS : N;
  const int RW = ((2 * NQ + P + 1 + 3) / 4) * 4;
  auto pidx = [&](int n) { return FAST ? n + (n / DPT) * 4 : n; };
  float S[DPT];
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int n = FAST ? ks * DPT + i : i * KS + ks;
    S[i] = (MODE != SS_PIECE_LOCAL && live && n < N) ? S_g[(size_t)n * P + p] : 0.f;
  }
  float decays = 1.f;
  const float dtb = hb_to_float(((const TW*)A.dt_bias)[h]);
  const float neg_a = -expf(hb_to_float(((const TW*)A.a_log)[h]));
  const float dsk = hb_to_float(((const TW*)A.d_skip)[h]);
  const int HP = H * P, GN = A.G * N;
  auto fetch = [&](int buf, int c0) {
    const int n = min(SS_CH, len - c0);
    float* st = ssm + buf * SS_CH * RW;
    if (A.vec4) {
      const int cn = N >> 2, cp = P >> 2, per = 2 * cn + cp;
      for (int i = tid; i < n * per; i += nthr) {
        const int j = i / per, c = i - j * per;
        const float* row = A.xbc + (size_t)(t0 + c0 + j) * A.ldx;
        if (c < cn) ss_cp16(st + j * RW + pidx(4 * c), row + HP + g * N + 4 * c);
        else if (c < 2 * cn) ss_cp16(st + j * RW + NQ + pidx(4 * (c - cn)), row + HP + GN + g * N + 4 * (c - cn));
        else ss_cp16(st + j * RW + 2 * NQ + 4 * (c - 2 * cn), row + h * P + 4 * (c - 2 * cn));
      }
    } else {
      const int per = 2 * N + P;
      for (int i = tid; i < n * per; i += nthr) {
        const int j = i / per, c = i - j * per;
        const float* row = A.xbc + (size_t)(t0 + c0 + j) * A.ldx;
        const float* src = c < N ? row + HP + g * N + c : c < 2 * N ? row + HP + GN + g * N + (c - N) : row + h * P + (c - 2 * N);
        ss_cp4(st + j * RW + c, src);
      }
    }
    for (int j = tid; j < n; j += nthr) ss_cp4(st + j * RW + 2 * NQ + P, A.dt + (size_t)(t0 + c0 + j) * A.lddt + h);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (len > j_begin) fetch(0, j_begin);
  int buf = 0;
  for (int c0 = j_begin; c0 < len; c0 += SS_CH, buf ^= 1) {
    const int n = min(SS_CH, len - c0);
    if (c0 + SS_CH < len) {
      fetch(buf ^ 1, c0 + SS_CH);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    float* st = ssm + buf * SS_CH * RW;
    // what does not depend on the state: the step size, dt B, and (last, by one thread a token) the decay in dt's place
    for (int i = tid; i < n * N; i += nthr) {
      const int j = i / N, c = i - j * N;
      float* row = st + j * RW;
      const float zz = row[2 * NQ + P] + dtb;
      const float dt = fmaxf(zz, 0.f) + log1pf(expf(-fabsf(zz)));
      row[pidx(c)] *= dt;
    }
    __syncthreads();
    for (int j = tid; j < n; j += nthr) {
      float* row = st + j * RW;
      const float zz = row[2 * NQ + P] + dtb;
      const float dt = fmaxf(zz, 0.f) + log1pf(expf(-fabsf(zz)));
      row[2 * NQ + P] = expf(neg_a * dt);
    }
    __syncthreads();
    for (int j = 0; j < n; j++) {
      const float* row = st + j * RW;
      const float xv = live ? row[2 * NQ + p] : 0.f;
      const float a = row[2 * NQ + P];
      const float* Bj = row;
      const float* Cj = row + NQ;
      if (MODE == SS_PIECE_LOCAL) {
        decays *= a;
        if constexpr (FAST) {
          const int sb = ks * (DPT + 4);
#pragma unroll
          for (int i = 0; i < DPT; i += 4) {
            const float4 b4 = *(const float4*)(Bj + sb + i);
            S[i] = fmaf(a, S[i], b4.x * xv);
            S[i + 1] = fmaf(a, S[i + 1], b4.y * xv);
            S[i + 2] = fmaf(a, S[i + 2], b4.z * xv);
            S[i + 3] = fmaf(a, S[i + 3], b4.w * xv);
          }
        } else {
#pragma unroll
          for (int i = 0; i < DPT; i++) {
            const int n0 = i * KS + ks;
            if (n0 < N) S[i] = fmaf(a, S[i], Bj[n0] * xv);
          }
        }
        continue;
      }
      float o = 0.f, o2 = 0.f;
      if constexpr (FAST) {
        const int sb = ks * (DPT + 4);
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 b4 = *(const float4*)(Bj + sb + i), c4 = *(const float4*)(Cj + sb + i);
          S[i] = fmaf(a, S[i], b4.x * xv);
          S[i + 1] = fmaf(a, S[i + 1], b4.y * xv);
          S[i + 2] = fmaf(a, S[i + 2], b4.z * xv);
          S[i + 3] = fmaf(a, S[i + 3], b4.w * xv);
          o = fmaf(S[i], c4.x, o);
          o2 = fmaf(S[i + 1], c4.y, o2);
          o = fmaf(S[i + 2], c4.z, o);
          o2 = fmaf(S[i + 3], c4.w, o2);
        }
      } else
#pragma unroll
      for (int i = 0; i < DPT; i += 2) {
        const int n0 = i * KS + ks, n1 = n0 + KS;
        if (n0 < N) {
          S[i] = fmaf(a, S[i], Bj[n0] * xv);
          o = fmaf(S[i], Cj[n0], o);
        }
        if (n1 < N) {
          S[i + 1] = fmaf(a, S[i + 1], Bj[n1] * xv);
          o2 = fmaf(S[i + 1], Cj[n1], o2);
        }
      }
      o += o2;
      for (int m = 1; m < KS; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (live && ks == 0) A.y[(size_t)(t0 + c0 + j) * HP + h * P + p] = fmaf(dsk, xv, o);
    }
    __syncthreads();             // the buffer is free for the chunk after the next
  }
  if (MODE == SS_PIECE_OUT) return;
#pragma unroll
  for (int i = 0; i < DPT; i++) {
    const int n = FAST ? ks * DPT + i : i * KS + ks;
    if (live && n < N) S_g[(size_t)n * P + p] = S[i];
  }
  if (MODE == SS_PIECE_LOCAL && tid == 0)
    A.piece_decay[((size_t)ss_piece_base(A.q_len, r, A.L) + blockIdx.z) * H + h] = decays;
}

// The pieces' starting states, one after another: an element of (request, head) walks its pieces, leaves in each the state
// the piece starts from and carries (decay product) * state + the piece's own contribution on; the last goes to the slot.
__global__ void __launch_bounds__(256) ssd_carry_kernel(SsdArgs A) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int r = blockIdx.y, NP = A.N * A.P;
  const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= (size_t)A.H * NP) return;
  const int h = (int)(e / NP), len = A.q_len[r];
  if (len <= 0) return;
  const int pieces = (len + A.L - 1) / A.L;
  float* slot = A.state + (size_t)A.slot[r] * A.H * NP + e;
  float carry = *slot;
  const size_t base = (size_t)ss_piece_base(A.q_len, r, A.L);
  float* ps = A.piece_state + base * A.H * NP + e;
  const float* pd = A.piece_decay + base * A.H + h;
  const size_t step = (size_t)A.H * NP;
  for (int c0 = 0; c0 < pieces; c0 += 8) {                 // eight pieces' loads in flight, then their chain
    float own[8], dec[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const bool in = c0 + i < pieces;
      own[i] = in ? ps[(size_t)(c0 + i) * step] : 0.f;
      dec[i] = in ? pd[(size_t)(c0 + i) * A.H] : 1.f;
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      if (c0 + i < pieces) {
        ps[(size_t)(c0 + i) * step] = carry;
        carry = fmaf(dec[i], carry, own[i]);
      }
    }
  }
  *slot = carry;
}

HB_EXPORT int hb_ssd_scan(const float* xbc, long ldx, const float* dt, long lddt, const void* dt_bias, const void* a_log,
                          const void* d_skip, int w_dt, float* state, const int* q_start, const int* q_len, const int* slot,
                          float* y, int n_requests, int H, int P, int N, int G, int piece_len, int pieces, float* piece_state,
                          float* piece_decay, cudaStream_t s) {
  // pieces > 0: the three-launch form over pieces of piece_len tokens, no request with more than `pieces` of them, with
  // room for all requests' pieces (at most rows / piece_len + n_requests) in piece_state [.][H][N][P] and piece_decay [.][H]
  if (n_requests <= 0) return 0;
  if (pieces > 0 && (piece_len <= 0 || !piece_state || !piece_decay || pieces > 65535)) HB_FAIL("hb_ssd_scan: %d pieces of %d", pieces, piece_len);
  if (P > 1024 || G <= 0 || H % G) HB_FAIL("hb_ssd_scan: %d heads of %d in %d groups", H, P, G);
  // threads a value channel (a power of two up to 32): the fewest that give the block 256 threads, else the most that fit
  int ks = 0;
  for (int c = 1; c <= 32; c *= 2) {
    const int per_c = (N + c - 1) / c, threads_c = ((P * c + 31) / 32) * 32;
    if (per_c > 64) continue;
    const int limit = per_c <= 8 ? 1024 : per_c <= 32 ? 512 : 256;
    if (threads_c > limit) break;
    ks = c;
    if (threads_c >= 256) break;
  }
  if (!ks) HB_FAIL("hb_ssd_scan: heads of %d x %d do not fit a block's registers", N, P);
  const int per = (N + ks - 1) / ks;
  SsdArgs A;
  A.xbc = xbc; A.ldx = ldx; A.dt = dt; A.lddt = lddt; A.dt_bias = dt_bias; A.a_log = a_log; A.d_skip = d_skip; A.state = state;
  A.q_start = q_start; A.q_len = q_len; A.slot = slot; A.y = y; A.H = H; A.P = P; A.N = N; A.G = G; A.KS = ks;
  A.vec4 = !((N | P) & 3) && !(ldx & 3) && !((uintptr_t)xbc & 15);
  A.piece_state = piece_state; A.piece_decay = piece_decay; A.L = piece_len; A.pieces = pieces;
  const int threads = ((P * ks + 31) / 32) * 32;
  const bool fast = A.vec4 && N == per * ks && (per == 8 || per == 16 || per == 32 || per == 64);
  const int NQ = fast ? N + 4 * ks : N;
  const int RW = ((2 * NQ + P + 1 + 3) / 4) * 4;
  const size_t smem = (size_t)2 * SS_CH * RW * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_ssd_scan: heads of %d x %d do not fit shared memory", N, P);
  if (n_requests > 65535) HB_FAIL("hb_ssd_scan: the grid is too large");
#define SS_LAUNCH_MODE(DPT, MODE, GRID)                                                                            \
  HB_DISPATCH_1(w_dt, "hb_ssd_scan", do {                                                                          \
    auto kern = fast ? ssd_scan_kernel<DPT, TA, MODE, true> : ssd_scan_kernel<DPT, TA, MODE, false>;               \
    if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    hb_launch(kern, GRID, dim3(threads), smem, s, A);                                                              \
  } while (0))
#define SS_LAUNCH(MODE, GRID)                                                                                      \
  do {                                                                                                             \
    if (per <= 8) SS_LAUNCH_MODE(8, MODE, GRID);                                                                   \
    else if (per <= 16) SS_LAUNCH_MODE(16, MODE, GRID);                                                            \
    else if (per <= 32) SS_LAUNCH_MODE(32, MODE, GRID);                                                            \
    else SS_LAUNCH_MODE(64, MODE, GRID);                                                                           \
  } while (0)
  if (pieces <= 0) {
    SS_LAUNCH(SS_WHOLE, dim3(H, n_requests));
  } else {
    const dim3 grid(H, n_requests, pieces);
    SS_LAUNCH(SS_PIECE_LOCAL, grid);
    HB_CHECK_LAUNCH("hb_ssd_scan");
    const size_t elems = (size_t)H * N * P;
    hb_launch(ssd_carry_kernel, dim3((unsigned)((elems + 255) / 256), n_requests), dim3(256), 0, s, A);
    HB_CHECK_LAUNCH("hb_ssd_scan");
    SS_LAUNCH(SS_PIECE_OUT, grid);
  }
#undef SS_LAUNCH
#undef SS_LAUNCH_MODE
  HB_CHECK_LAUNCH("hb_ssd_scan");
  return 0;
}

// One block a row: y silu(z), then every part of the row by its own root mean square, times the weight.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256) ssd_gate_norm_kernel(const float* __restrict__ y, const float* __restrict__ z, long ldz,
                                                            const TW* __restrict__ w, TO* __restrict__ out, int inner,
                                                            int parts, float eps) {
  __shared__ float sh[32];
  hb_pdl_launch();
  hb_pdl_wait();
  const int t = blockIdx.x, span = inner / parts;
  const float* yr = y + (size_t)t * inner;
  const float* zr = z + (size_t)t * ldz;
  for (int q = 0; q < parts; q++) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < span; i += 256) {
      const float zz = zr[q * span + i], v = yr[q * span + i] * (zz / (1.f + expf(-zz)));
      ss = fmaf(v, v, ss);
    }
    const float f = rsqrtf(hb_block_sum(ss, sh) / (float)span + eps);
    for (int i = threadIdx.x; i < span; i += 256) {
      const float zz = zr[q * span + i], v = yr[q * span + i] * (zz / (1.f + expf(-zz)));
      out[(size_t)t * inner + q * span + i] = hb_from_float<TO>(v * f * hb_to_float(w[q * span + i]));
    }
  }
}

HB_EXPORT int hb_ssd_gate_norm(const float* y, const float* z, long ldz, const void* w, int w_dt, void* out, int o_dt, int T,
                               int inner, int parts, float eps, cudaStream_t s) {
  if (T <= 0) return 0;
  if (parts <= 0 || inner % parts) HB_FAIL("hb_ssd_gate_norm: %d channels in %d parts", inner, parts);
  HB_DISPATCH_2(w_dt, o_dt, "hb_ssd_gate_norm",
                (hb_launch(ssd_gate_norm_kernel<TA, TB>, T, 256, 0, s, y, z, ldz, (const TA*)w, (TB*)out, inner, parts, eps)));
  HB_CHECK_LAUNCH("hb_ssd_gate_norm");
  return 0;
}
