// RG-LRU forward and backward kernels for sm_100a.
//
// Work decomposition.  A CTA owns CH (64 or 32) adjacent channels of one batch row and walks the whole
// sequence in chunks of LANES*TS time-steps.  Inside a chunk the time axis is split over LANES (16 or 32)
// time-lanes, each thread scanning TS = 4 steps of CV = 4 channels in registers (level one), after which a
// few threads per channel chain the lane aggregates and the carry from the previous chunk through shared
// memory (level two: one serial chain of 16 for the 64-channel shape, four segments of eight joined by a
// small exchange for the 32-lane shape) and every lane applies its incoming state.  Chunks are staged through
// shared memory by TMA (cp.async.bulk.tensor, 3-D tiles [1, rows, channels]) in a multi-stage mbarrier
// pipeline; results are written back into the stage in place and leave through TMA stores.  The bulk copies
// are issued either by a producer warp or, for the bf16 backward, by one compute thread (SELF_ISSUE: eight
// warps leave every thread the registers it wants).  The 64-byte rows of 32-channel bf16 tiles are staged two to a
// 128-byte line through 5-D tensor maps (PAIRED), which halves the forward's shared-memory bank conflicts.  A bounds-checked plain-load staging path with the same
// arithmetic covers shapes TMA cannot address (D * element size not a multiple of 16 bytes).
//
// What bounds them (ncu on B200, bf16, B = 8, T = 2048, D = 1024): DRAM traffic equals the algorithmic bytes;
// no pipe is more than 40 % busy and 0.4 instructions issue per scheduler and cycle: with one (backward) or two
// (forward) CTAs per SM the kernels are bound by dependent-instruction latency inside a warp and by what
// happens outside the chunk loop, so the channel arithmetic is written on float2 pairs (one issue slot per two
// fp32 operations), transcendental work is kept to three or four MUFU operations per element, and the
// prologue (first loads issued before the per-channel rates are worked out, the first chunk prefetched into
// L2 before the dependency wait) and the epilogue (row sums folded by the last CTA with all loads in flight
// at once) are kept short.  Sixteen-warp variants with two steps per thread measured 15 % slower.
//
// The gate epilogue follows griffin/griffin.py:237-258 of the reference, the scan :280-286, the backward is
// the closed form of autograd over those lines with the capped sqrt slope of :59-65.  All arithmetic is fp32.
//
// Template switches of the two kernels (each a separate instantiation, so the plain kernels pay nothing for
// them):
//   CONV    the width-4 causal conv in front of the layer (:474-486) is applied while a chunk is loaded, from
//           an x tile with a three-row halo;
//   MERGE   the block's GeLU-branch product (:464, :520) is formed in the store stage and differentiated in
//           the backward's load stage;
//   GROUPED both gate pre-activations come from one [B, T, 2 D] tensor written by a single grouped GEMM, the
//           gate biases are added here, and the backward also returns their gradient (column sums of du);
//   PLAIN   no token flags and a whole number of chunks: the masked arithmetic is not compiled in.
// The file also holds the raw affine scan operator (triton_scan.py:274-276), the TMA-staged kernels of the
// conv alone, and the self-test of the bounded wait.

#include <atomic>
#include <cstdlib>

#include "rglru_device.cuh"
#include "rglru_internal.h"

namespace rglru {

// Per-row multipliers that realise the reset / padding masks without branches.
struct RowMask {
  float keep;    // 0 at a reset, else 1          (a <- a * keep, gamma <- gamma * keep + (1 - keep))
  float live;    // 0 on padding, else 1          (a <- a * live + (1 - live), b <- b * live)
};

template <bool MASKED>
__device__ __forceinline__ RowMask row_mask(uint32_t packed, int st) {
  RowMask m{1.0f, 1.0f};
  if (MASKED) {
    const uint32_t byte = (packed >> (8 * (st & 3))) & 0xffu;
    m.keep = (byte & TOK_RESET) ? 0.0f : 1.0f;
    m.live = (byte & TOK_INACTIVE) ? 0.0f : 1.0f;
  }
  return m;
}

// Flag bytes of the TS steps a thread owns, packed four per word.  Steps at or
// beyond T are padding.
template <int TS>
__device__ __forceinline__ void load_flags(const uint8_t* tok, int b, int T, int t_first, uint32_t (&fl)[(TS + 3) / 4]) {
#pragma unroll
  for (int w = 0; w < (TS + 3) / 4; ++w) fl[w] = 0;
#pragma unroll
  for (int st = 0; st < TS; ++st) {
    const int t = t_first + st;
    uint32_t byte = TOK_INACTIVE;
    if (t < T) byte = tok ? tok[static_cast<size_t>(b) * T + t] : 0u;
    fl[st >> 2] |= byte << (8 * (st & 3));
  }
}

// Whether any of a thread's flag bytes is set.  Ordinary tokens have a zero byte, so a thread whose steps are
// all ordinary takes the mask-free arithmetic even when the caller passed a flag tensor.
template <int N>
__device__ __forceinline__ bool any_flag(const uint32_t (&fl)[N]) {
  uint32_t v = 0u;
#pragma unroll
  for (int i = 0; i < N; ++i) v |= fl[i];
  return v != 0u;
}

// The same for four steps, as one word when the four bytes are whole and 4-byte aligned (the byte of step st sits
// at bits 8 st).  Used by the conv kernels, whose per-element work is small enough for the byte loads to show;
// the scan kernels keep the byte loads (the word path perturbed their register allocation: +9 % backward time).
__device__ __forceinline__ void load_flags_word(const uint8_t* tok, int b, int T, int t_first, uint32_t (&fl)[1]) {
  if (tok && t_first + 4 <= T) {
    const uint8_t* p = tok + static_cast<size_t>(b) * T + t_first;
    if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) {
      fl[0] = *reinterpret_cast<const uint32_t*>(p);
      return;
    }
  }
  load_flags<4>(tok, b, T, t_first, fl);
}

// Plain-load staging of one [rows, CH] tile (zero-filled outside the tensor).
template <typename IO, int CH>
__device__ __forceinline__ void tile_load_plain(uint8_t* tile, const void* src, int b, int t0, int d0, int rows, int T, int D) {
  const IO* g = static_cast<const IO*>(src);
  IO* s = reinterpret_cast<IO*>(tile);
  for (int idx = threadIdx.x; idx < rows * CH; idx += blockDim.x) {
    const int row = idx / CH, col = idx % CH;
    const int t = t0 + row, d = d0 + col;
    IO v = Pack<IO>::from_float(0.0f);
    if (t >= 0 && t < T && d < D) v = g[(static_cast<size_t>(b) * T + t) * D + d];
    s[idx] = v;
  }
}
template <typename IO, int CH>
__device__ __forceinline__ void tile_store_plain(const uint8_t* tile, void* dst, int b, int t0, int d0, int rows, int T, int D) {
  IO* g = static_cast<IO*>(dst);
  const IO* s = reinterpret_cast<const IO*>(tile);
  for (int idx = threadIdx.x; idx < rows * CH; idx += blockDim.x) {
    const int row = idx / CH, col = idx % CH;
    const int t = t0 + row, d = d0 + col;
    if (t < T && d < D) g[(static_cast<size_t>(b) * T + t) * D + d] = s[idx];
  }
}

// Per-channel rate: -c * logsigmoid(Lambda) >= 0, and 0 for channels past D.
__device__ __forceinline__ float decay_rate(const float* lambda, int d, int D, float c) {
  if (d >= D) return 0.0f;
  const float lam = lambda[d];
  // softplus(-L) = -logsigmoid(L), evaluated without cancellation on either side.
  const float sp = lam >= 0.0f ? log1pf(expf(-lam)) : log1pf(expf(lam)) - lam;
  return c * sp;
}

template <int LANES, int CH>
struct ChainSmem {
  static constexpr int AGG = LANES * CH * 8;  // float2 per (lane, channel)
  static constexpr int EIN = LANES * CH * 4;  // float per (lane, channel)
};

// Grouped gate layout: both gate pre-activations come from ONE tensor [B, T, 2 D] written by a single
// grouped GEMM with the two weight blocks of a gate head stacked, i.e. per head of width bw the columns are
// [u_r (bw) | u_i (bw)].  The channel tile at d0 (which never straddles a head: bw is a multiple of the tile
// width) finds its u_r columns at (d0 / bw) * 2 bw + d0 % bw and its u_i columns bw further.  The gate biases
// (same column layout, fp32) are added in the kernel, pre-scaled for the sigmoid.
struct GateBias {
  float2 r[2], i[2];
};
__device__ __forceinline__ int grouped_col(int d0, int bw) { return (d0 / bw) * 2 * bw + d0 % bw; }
template <bool HALF_IO>
__device__ __forceinline__ void load_gate_bias(const float* bias, int rcol, int icol, GateBias& gb) {
  const float sc = gate_bias_scale<HALF_IO>();
  float4 br = make_float4(0.f, 0.f, 0.f, 0.f), bi = br;
  if (bias) {
    br = *reinterpret_cast<const float4*>(bias + rcol);
    bi = *reinterpret_cast<const float4*>(bias + icol);
  }
  gb.r[0] = make_float2(br.x * sc, br.y * sc); gb.r[1] = make_float2(br.z * sc, br.w * sc);
  gb.i[0] = make_float2(bi.x * sc, bi.y * sc); gb.i[1] = make_float2(bi.z * sc, bi.w * sc);
}

// Taps of the width-4 causal depthwise conv for the four channels a thread owns (column 3 of the
// [D, 4] weight multiplies the current token; griffin/griffin.py:474-486 of the reference).
struct ConvTaps {
  float2 w[4][2];
  float2 bias[2];
};

__device__ __forceinline__ void load_taps(const float* conv_w, const float* conv_b, int d, int D, ConvTaps& ct) {
  float w[4][4], bz[4];
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    const bool ok = d + ch < D;
    bz[ch] = (ok && conv_b) ? conv_b[d + ch] : 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k][ch] = ok ? conv_w[(d + ch) * 4 + k] : 0.0f;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) { ct.w[k][0] = make_float2(w[k][0], w[k][1]); ct.w[k][1] = make_float2(w[k][2], w[k][3]); }
  ct.bias[0] = make_float2(bz[0], bz[1]);
  ct.bias[1] = make_float2(bz[2], bz[3]);
}

// Conv folded into the load stage: the x tile carries three extra rows in front (times t0-3 .. t0-1), a
// thread reads the TS+3 rows ending at its last step and forms the TS conv outputs in registers.
// `hist` (non-null only for the first lane of the first chunk when a conv state is carried) replaces
// the three rows before t = 0.  Tap l is dropped when the token's flag byte says fewer than l earlier
// tokens belong to its document.
template <typename IO, int TS, int CH, bool MASKED>
__device__ __forceinline__ void conv_front(const uint8_t* tx, int off0, const ConvTaps& ct,
                                           const uint32_t (&fl)[(TS + 3) / 4], const float2 (*hist)[2],
                                           float2 (&xc)[TS][2]) {
  constexpr int ROWB = CH * sizeof(IO);
  float2 raw[TS + 3][2];
#pragma unroll
  for (int r = 0; r < TS + 3; ++r) Pack<IO>::unpack2(Pack<IO>::load(tx + off0 + r * ROWB), raw[r]);
  if (hist) {
#pragma unroll
    for (int r = 0; r < 3; ++r) { raw[r][0] = hist[r][0]; raw[r][1] = hist[r][1]; }
  }
#pragma unroll
  for (int st = 0; st < TS; ++st) {
    float m1 = 1.0f, m2 = 1.0f, m3 = 1.0f;
    if (MASKED) {
      const int reach = 3 - static_cast<int>((fl[st >> 2] >> (8 * (st & 3))) & TOK_CUT_MASK);
      m1 = reach >= 1 ? 1.0f : 0.0f;
      m2 = reach >= 2 ? 1.0f : 0.0f;
      m3 = reach >= 3 ? 1.0f : 0.0f;
    }
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
      float2 acc = fma2(ct.w[3][cp], raw[st + 3][cp], ct.bias[cp]);
      if (MASKED) {
        acc = fma2(mul2(ct.w[2][cp], f2(m1)), raw[st + 2][cp], acc);
        acc = fma2(mul2(ct.w[1][cp], f2(m2)), raw[st + 1][cp], acc);
        acc = fma2(mul2(ct.w[0][cp], f2(m3)), raw[st][cp], acc);
      } else {
        acc = fma2(ct.w[2][cp], raw[st + 2][cp], acc);
        acc = fma2(ct.w[1][cp], raw[st + 1][cp], acc);
        acc = fma2(ct.w[0][cp], raw[st][cp], acc);
      }
      xc[st][cp] = acc;
    }
  }
}

// The three inputs before t = 0 of one batch row, from the carried conv state [B, 3, D].
template <typename IO>
__device__ __forceinline__ void load_hist(const void* conv_state, int b, int d, int D, float2 (&hist)[3][2]) {
  const IO* st = static_cast<const IO*>(conv_state);
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    float v[4];
#pragma unroll
    for (int ch = 0; ch < 4; ++ch)
      v[ch] = (d + ch < D) ? Pack<IO>::to_float(st[(static_cast<size_t>(b) * 3 + r) * D + d + ch]) : 0.0f;
    hist[r][0] = make_float2(v[0], v[1]);
    hist[r][1] = make_float2(v[2], v[3]);
  }
}

// ======================================================================
// Forward
// ======================================================================

template <typename IO, int TS, int CH, bool MASKED, bool POLY, bool CONV, bool GROUPED, int RSTEP = CH * sizeof(IO)>
__device__ __forceinline__ void fwd_local(const uint8_t* tx, const uint8_t* tr, const uint8_t* ti, int off0,
                                          const float2 (&K)[2], const uint32_t (&fl)[(TS + 3) / 4],
                                          const ConvTaps& ct, const float2 (*hist)[2], const GateBias& gb,
                                          float2 (&P)[TS][2], float2 (&S)[TS][2]) {
  constexpr int ROWB = CH * sizeof(IO);
  float2 p[2] = {f2(1.0f), f2(1.0f)};
  float2 s[2] = {f2(0.0f), f2(0.0f)};
  float2 xc[CONV ? TS : 1][2];
  if (CONV) conv_front<IO, CONV ? TS : 1, CH, MASKED>(tx, off0, ct, fl, hist, xc);
#pragma unroll
  for (int st = 0; st < TS; ++st) {
    const int off = off0 + st * RSTEP;   // RSTEP: bytes between a thread's consecutive steps in the tile
    float2 xv[2], rv[2], iv[2];
    if (CONV) { xv[0] = xc[CONV ? st : 0][0]; xv[1] = xc[CONV ? st : 0][1]; }
    else Pack<IO>::unpack2(Pack<IO>::load(tx + off), xv);
    Pack<IO>::unpack2(Pack<IO>::load(tr + off), rv);
    Pack<IO>::unpack2(Pack<IO>::load(ti + off), iv);
    const RowMask m = row_mask<MASKED>(fl[st >> 2], st);
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
      float2 r, i;
      if (GROUPED) sigmoid_pair2_biased<sizeof(IO) == 2>(rv[cp], iv[cp], gb.r[cp], gb.i[cp], r, i);
      else sigmoid_pair2<sizeof(IO) == 2>(rv[cp], iv[cp], r, i);
      const float2 e = one_minus_exp_neg2<POLY, sizeof(IO) == 2>(mul2(r, K[cp]));   // 1 - a
      float2 a = fma2(e, f2(-1.0f), f2(1.0f));
      const float2 gsq = mul2(e, fma2(e, f2(-1.0f), f2(2.0f)));     // 1 - a^2
      // sqrt(gsq) as gsq * rsqrt(gsq): one MUFU operation; the offset keeps rsqrt finite (gamma error <= 1e-15)
      const float2 gq = add2(gsq, f2(1e-30f));
      float2 gam = mul2(gq, make_float2(rsqrt_approx(gq.x), rsqrt_approx(gq.y)));
      if (MASKED) {
        a = fma2(mul2(a, f2(m.keep)), f2(m.live), f2(1.0f - m.live));
        gam = mul2(fma2(gam, f2(m.keep), f2(1.0f - m.keep)), f2(m.live));
      }
      const float2 b = mul2(mul2(gam, i), xv[cp]);
      p[cp] = mul2(p[cp], a);
      s[cp] = fma2(a, s[cp], b);
      P[st][cp] = p[cp];
      S[st][cp] = s[cp];
    }
  }
}

template <typename IO, int TS, int LANES, int CH, int NSTAGE, bool CONV = false, bool MERGE = false>
struct FwdSmem {
  static constexpr int TC = LANES * TS;
  static constexpr int TILE = TC * CH * sizeof(IO);
  static constexpr int HALO = CONV ? 3 * CH * sizeof(IO) : 0;   // three rows in front of the x tile
  static constexpr int TILEX = TILE + HALO;
  static constexpr int OFF_G = TILEX + 2 * TILE;                // GeLU-branch tile of the merged variant
  static constexpr int STAGE = TILEX + 2 * TILE + (MERGE ? TILE : 0);
  static constexpr int OFF_AGG = NSTAGE * STAGE;
  static constexpr int OFF_EIN = OFF_AGG + ChainSmem<LANES, CH>::AGG;
  // The 32-lane shape splits a channel's chain over SEGS threads (segment totals: one float2 per segment and channel).
  static constexpr int SEGS = (LANES == 32 && CH == 32) ? 4 : 1;
  static constexpr int OFF_SEG = OFF_EIN + ChainSmem<LANES, CH>::EIN;
  static constexpr int OFF_BAR = OFF_SEG + SEGS * CH * 8;   // full[NSTAGE], ready[NSTAGE], dead flag
  static constexpr int BYTES = OFF_BAR + 2 * NSTAGE * 8 + 16;
};

// Threads [0, LANES*NCV) compute; with TMA one extra warp issues every bulk copy so that
// no compute warp ever waits on the copy engine's instruction latency.
// MERGE: the kernel also reads the pre-activation of the block's GeLU branch and writes
// h_t * gelu(branch_t) (griffin/griffin.py:464, 520 of the reference) instead of h_t.
template <typename IO, int TS, int LANES, int CH, int NSTAGE, bool USE_TMA, bool CONV, bool MERGE, bool GROUPED, bool PLAIN = false,
          bool CARRY = false, bool PAIRED = false>
__device__ __forceinline__ void rglru_fwd_body(const FwdMaps& maps, const ScanFwdArgs& p) {
  using SM = FwdSmem<IO, TS, LANES, CH, NSTAGE, CONV, MERGE>;
  static_assert(!CONV || (SM::HALO % 128 == 0), "the halo must keep the result rows 128-byte aligned for TMA");
  constexpr int NCV = CH / CV;
  constexpr int TC = SM::TC;
  constexpr int ROWB = CH * sizeof(IO);
  // PAIRED: 64-byte tile rows (32 bf16 channels) put the four time-lanes of a warp on the same sixteen banks.  The
  // tile is then staged through 5-D tensor maps that view time as (eighth, half, step), t = 8 q + 4 h + j, and lay
  // it out as [q][j][h][channels]: rows t and t + 4 share one 128-byte line, a thread's four steps are 128 bytes
  // apart, and two neighbouring time-lanes fill a line between them, so a warp's access touches every bank once.
  static_assert(!PAIRED || (USE_TMA && PLAIN && !CONV && !MERGE && !GROUPED && TS == 4 && ROWB == 64 && TC % 8 == 0),
                "paired rows: plain TMA-staged kernel on 64-byte rows only");
  constexpr int RSTEP = PAIRED ? 2 * ROWB : ROWB;
  constexpr int NCOMP = LANES * NCV;
  extern __shared__ __align__(128) uint8_t smem[];
  float2* agg = reinterpret_cast<float2*>(smem + SM::OFF_AGG);
  float* ein = reinterpret_cast<float*>(smem + SM::OFF_EIN);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
  uint64_t* ready = full + NSTAGE;
  volatile int* dead = reinterpret_cast<volatile int*>(ready + NSTAGE);

  const int tid = threadIdx.x;
  const int lane_t = tid / NCV;
  const int vec = tid % NCV;
  const int b = blockIdx.y;
  const int d0 = blockIdx.x * CH;
  const int nchunks = (p.T + TC - 1) / TC;
  const int nsave = (p.T + SAVE_EVERY - 1) / SAVE_EVERY;
  static_assert(!GROUPED || USE_TMA, "the grouped gate layout is staged by TMA only");
  const int rcol = GROUPED ? grouped_col(d0, p.gate_bw) : d0;   // first column of this tile's u_r / u_i
  const int icol = GROUPED ? rcol + p.gate_bw : d0;

  auto issue = [&](int k) {
    const int sidx = k % NSTAGE;
    uint8_t* st = smem + sidx * SM::STAGE;
    mbar_expect_tx(&full[sidx], SM::STAGE);
    if constexpr (PAIRED) {
      tma_load_5d(st, &maps.x, d0, 0, 0, k * (TC / 8), b, &full[sidx]);
      tma_load_5d(st + SM::TILEX, &maps.ur, d0, 0, 0, k * (TC / 8), b, &full[sidx]);
      tma_load_5d(st + SM::TILEX + SM::TILE, &maps.ui, d0, 0, 0, k * (TC / 8), b, &full[sidx]);
    } else {
      tma_load_3d(st, &maps.x, d0, k * TC - (CONV ? 3 : 0), b, &full[sidx]);   // rows before t = 0 read as zero
      tma_load_3d(st + SM::TILEX, &maps.ur, rcol, k * TC, b, &full[sidx]);
      tma_load_3d(st + SM::TILEX + SM::TILE, &maps.ui, icol, k * TC, b, &full[sidx]);
      if (MERGE) tma_load_3d(st + SM::OFF_G, &maps.g, d0, k * TC, b, &full[sidx]);
    }
  };
  // Set-up by the thread that will issue the bulk copies, published by one early CTA barrier; after it the
  // producer warp and the compute warps go their own ways (the compute warps vote among themselves), so the
  // first loads are issued while the per-channel rates are worked out and nobody waits for the issuing thread.
  pdl_launch_dependents();
  if (USE_TMA ? (tid == NCOMP) : (tid == 0)) {
    *dead = 0;
    if (USE_TMA) {
      for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full[s], 1); mbar_init(&ready[s], NCOMP / 32); }
      mbar_fence_init();
      prefetch_map(&maps.x); prefetch_map(&maps.ur); prefetch_map(&maps.ui); prefetch_map(&maps.y);
      if (MERGE) prefetch_map(&maps.g);
      // While the kernel in front of this one on the stream drains, pull the first chunk towards L2.
      if constexpr (PAIRED) {
        tma_prefetch_5d(&maps.x, d0, 0, 0, 0, b);
        tma_prefetch_5d(&maps.ur, d0, 0, 0, 0, b);
        tma_prefetch_5d(&maps.ui, d0, 0, 0, 0, b);
      } else {
        tma_prefetch_3d(&maps.x, d0, -(CONV ? 3 : 0), b);
        tma_prefetch_3d(&maps.ur, rcol, 0, b);
        tma_prefetch_3d(&maps.ui, icol, 0, b);
        if (MERGE) tma_prefetch_3d(&maps.g, d0, 0, b);
      }
    }
  }
  __syncthreads();
  pdl_wait();   // nothing above touches global memory; everything below may depend on the previous kernel

  if (USE_TMA && tid >= NCOMP) {
    // ---- producer warp: loads run NSTAGE-1 chunks ahead; a stage is refilled as soon as the
    // store of the results written into it has drained from shared memory.
    if (tid == NCOMP) {
      // Every CTA of the grid starts at once and asks for NSTAGE chunks; the first chunk is asked for alone and
      // the rest once it has landed, so that no CTA's first chunk queues behind other CTAs' later ones.
      issue(0);
      mbar_wait_or_flag(&full[0], 0, dead, p.status, DEV_TIMEOUT_LOAD);
      for (int k = 1; k < NSTAGE && k < nchunks; ++k) issue(k);
      for (int k = 0; k < nchunks; ++k) {
        const int sidx = k % NSTAGE;
        mbar_wait_or_flag(&ready[sidx], (k / NSTAGE) & 1, dead, p.status, DEV_TIMEOUT_STORE);
        if constexpr (PAIRED) tma_store_5d(&maps.y, smem + sidx * SM::STAGE, d0, 0, 0, k * (TC / 8), b);
        else if (!CARRY) tma_store_3d(&maps.y, smem + sidx * SM::STAGE + SM::HALO, d0, k * TC, b);
        tma_commit();
        if (k + NSTAGE < nchunks) {
          tma_wait_read<0>();
          issue(k + NSTAGE);
        }
      }
      tma_wait_all<0>();
    }
    return;
  }

  float2 K[2];
  {
    const int d = d0 + vec * CV;
    K[0] = make_float2(decay_rate(p.lambda, d, p.D, p.c), decay_rate(p.lambda, d + 1, p.D, p.c));
    K[1] = make_float2(decay_rate(p.lambda, d + 2, p.D, p.c), decay_rate(p.lambda, d + 3, p.D, p.c));
  }
  const bool poly = bar_compute_and(NCOMP, fmaxf(fmaxf(K[0].x, K[0].y), fmaxf(K[1].x, K[1].y)) <= -POLY_RANGE);

  if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0 && p.ticket) *p.ticket = 0u;   // consumed by the backward kernel

  ConvTaps ct;
  if (CONV) load_taps(p.conv_w, p.conv_b, d0 + vec * CV, p.D, ct);
  GateBias gb;
  if (GROUPED) load_gate_bias<sizeof(IO) == 2>(p.gate_bias, rcol + vec * CV, icol + vec * CV, gb);

  // Level-two chain: SEGS threads per channel (thread tid: channel d0 + tid % CH, lane segment tid / CH), each
  // of which carries the channel's state across chunks (identical copies).
  constexpr int SEGS = SM::SEGS, SEGL = LANES / SEGS;
  static_assert(SEGS * CH <= NCOMP && (SEGS * CH) % 32 == 0, "chain threads are whole warps of the compute group");
  float2* segtot = reinterpret_cast<float2*>(smem + SM::OFF_SEG);
  const bool chain_thread = tid < SEGS * CH;
  const int cch = tid % CH, seg = tid / CH;
  float carry = 0.0f;
  const int dch = d0 + cch;
  if (chain_thread && dch < p.D && p.h0) carry = p.h0[static_cast<size_t>(b) * p.D + dch];
  // Product of the decays over the sequence: with the final state it is the affine map h0 -> h_last of this
  // call, which is what a caller that splits one sequence over several calls (or GPUs) needs to chain them.
  const bool want_prod = p.decay_prod != nullptr;
  float prod_all = 1.0f;

  const int off0 = PAIRED ? ((lane_t >> 1) * TS) * RSTEP + (lane_t & 1) * ROWB + vec * Pack<IO>::BYTES
                          : (lane_t * TS) * ROWB + vec * Pack<IO>::BYTES;

  for (int k = 0; k < nchunks; ++k) {
    const int stage = USE_TMA ? (k % NSTAGE) : 0;
    uint8_t* tiles = smem + stage * SM::STAGE;
    const int t0 = k * TC;
    uint32_t fl[(TS + 3) / 4];
    const bool masked = !PLAIN && ((p.tok != nullptr) || (t0 + TC > p.T));
    if (masked) load_flags<TS>(p.tok, b, p.T, t0 + lane_t * TS, fl);

    if (USE_TMA) {
      mbar_wait_or_flag(&full[stage], (k / NSTAGE) & 1, dead, p.status, DEV_TIMEOUT_LOAD);
    } else {
      tile_load_plain<IO, CH>(tiles, p.x, b, t0 - (CONV ? 3 : 0), d0, TC + (CONV ? 3 : 0), p.T, p.D);
      tile_load_plain<IO, CH>(tiles + SM::TILEX, p.ur, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<IO, CH>(tiles + SM::TILEX + SM::TILE, p.ui, b, t0, d0, TC, p.T, p.D);
      if (MERGE) tile_load_plain<IO, CH>(tiles + SM::OFF_G, p.g, b, t0, d0, TC, p.T, p.D);
      bar_compute(NCOMP);
    }

    float2 P[TS][2], S[TS][2];
    const uint8_t* tx = tiles;
    const uint8_t* tr = tiles + SM::TILEX;
    const uint8_t* ti = tiles + SM::TILEX + SM::TILE;
    float2 hist_v[3][2];
    const float2 (*hist)[2] = nullptr;
    if (CONV && k == 0 && lane_t == 0 && p.conv_state) {   // history carried from an earlier call
      load_hist<IO>(p.conv_state, b, d0 + vec * CV, p.D, hist_v);
      hist = hist_v;
    }
    if (masked && any_flag(fl)) {
      if (poly) fwd_local<IO, TS, CH, true, true, CONV, GROUPED, RSTEP>(tx, tr, ti, off0, K, fl, ct, hist, gb, P, S);
      else fwd_local<IO, TS, CH, true, false, CONV, GROUPED, RSTEP>(tx, tr, ti, off0, K, fl, ct, hist, gb, P, S);
    } else {
      if (poly) fwd_local<IO, TS, CH, false, true, CONV, GROUPED, RSTEP>(tx, tr, ti, off0, K, fl, ct, hist, gb, P, S);
      else fwd_local<IO, TS, CH, false, false, CONV, GROUPED, RSTEP>(tx, tr, ti, off0, K, fl, ct, hist, gb, P, S);
    }
    {
      float4* dst = reinterpret_cast<float4*>(agg + lane_t * CH + vec * CV);
      dst[0] = make_float4(P[TS - 1][0].x, S[TS - 1][0].x, P[TS - 1][0].y, S[TS - 1][0].y);
      dst[1] = make_float4(P[TS - 1][1].x, S[TS - 1][1].x, P[TS - 1][1].y, S[TS - 1][1].y);
    }
    bar_compute(NCOMP);

    if (chain_thread) {
      float2 ag[SEGL];
#pragma unroll
      for (int j = 0; j < SEGL; ++j) ag[j] = agg[(seg * SEGL + j) * CH + cch];
      auto emit = [&](int lane, float e) {       // state entering a lane; every SAVE_EVERY steps also kept for the backward
        if (((lane * TS) % SAVE_EVERY) == 0) {
          const int t = t0 + lane * TS;
          if (p.states && t < p.T && dch < p.D)
            p.states[(static_cast<size_t>(b) * nsave + t / SAVE_EVERY) * p.D + dch] = e;
        }
        ein[lane * CH + cch] = e;
      };
      if (SEGS == 1) {
        float e = carry;
#pragma unroll
        for (int j = 0; j < LANES; ++j) {
          emit(j, e);
          e = fmaf(ag[j].x, e, ag[j].y);
        }
        carry = e;
        if (want_prod) {
#pragma unroll
          for (int j = 0; j < LANES; ++j) prod_all *= ag[j].x;
        }
      } else {
        // Each thread composes its segment from the identity, keeping the map (pp, sp) that takes the state
        // entering the segment to the state entering each of its lanes; the segment totals are exchanged through
        // shared memory and every thread chains the few totals in front of it.
        float pp[SEGL], sp[SEGL];
        float pa = 1.0f, sa = 0.0f;
#pragma unroll
        for (int j = 0; j < SEGL; ++j) {
          pp[j] = pa;
          sp[j] = sa;
          sa = fmaf(ag[j].x, sa, ag[j].y);
          pa *= ag[j].x;
        }
        segtot[seg * CH + cch] = make_float2(pa, sa);
        bar_chain(SEGS * CH);
        float e = carry, enter = carry;
#pragma unroll
        for (int sgm = 0; sgm < SEGS; ++sgm) {
          const float2 tot = segtot[sgm * CH + cch];
          if (sgm == seg) enter = e;
          e = fmaf(tot.x, e, tot.y);
          prod_all *= tot.x;
        }
        carry = e;
#pragma unroll
        for (int j = 0; j < SEGL; ++j) emit(seg * SEGL + j, fmaf(pp[j], enter, sp[j]));
      }
    }
    bar_compute(NCOMP);

    {
      const float4 e4 = *reinterpret_cast<const float4*>(ein + lane_t * CH + vec * CV);
      const float2 e[2] = {make_float2(e4.x, e4.y), make_float2(e4.z, e4.w)};
      uint8_t* ty = tiles + SM::HALO;  // y overwrites the x tile in place (past its halo rows)
#pragma unroll
      for (int st = 0; st < TS; ++st) {
        float2 yv[2];
#pragma unroll
        for (int cp = 0; cp < 2; ++cp) yv[cp] = fma2(P[st][cp], e[cp], S[st][cp]);
        if (MERGE) {
          float2 gv[2];
          Pack<IO>::unpack2(Pack<IO>::load(tiles + SM::OFF_G + off0 + st * RSTEP), gv);
#pragma unroll
          for (int cp = 0; cp < 2; ++cp) yv[cp] = mul2(yv[cp], mul2(gv[cp], gelu_sigmoid2<sizeof(IO) == 2>(gv[cp])));
        }
        Pack<IO>::store2(ty + off0 + st * RSTEP, yv);
      }
    }
    if (USE_TMA) {
      fence_async_smem();        // make this thread's results visible to the bulk store
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(&ready[stage]);   // one arrival per warp
    } else {
      bar_compute(NCOMP);
      if (!CARRY) tile_store_plain<IO, CH>(tiles + SM::HALO, p.y, b, t0, d0, TC, p.T, p.D);
      bar_compute(NCOMP);
    }
  }
  if (tid < CH && dch < p.D && p.h_last) p.h_last[static_cast<size_t>(b) * p.D + dch] = carry;   // segment 0's copy
  if (tid < CH && dch < p.D && want_prod) p.decay_prod[static_cast<size_t>(b) * p.D + dch] = prod_all;
}

// PLAIN: no token flags and a whole number of chunks, so the masked arithmetic is not compiled in.
// CARRY: the carry-only pass of a time-split sequence: no output tensor, nothing is stored but h_last and decay_prod.
// PAIRED: 64-byte tile rows staged two to a 128-byte line through 5-D tensor maps (see rglru_fwd_body).
template <typename IO, int TS, int LANES, int CH, int NSTAGE, bool USE_TMA, bool CONV, bool MERGE, bool GROUPED, bool PLAIN = false,
          bool CARRY = false, bool PAIRED = false>
__global__ void __launch_bounds__(LANES*(CH / CV) + (USE_TMA ? 32 : 0))
    rglru_fwd_kernel(const __grid_constant__ FwdMaps maps, const ScanFwdArgs p) {
  rglru_fwd_body<IO, TS, LANES, CH, NSTAGE, USE_TMA, CONV, MERGE, GROUPED, PLAIN, CARRY, PAIRED>(maps, p);
}
// The same kernel capped at 96 registers, which lets two 9-warp CTAs share an SM's register files (five warps
// on one scheduler partition).  Used for the merged / grouped variants, which otherwise take about 112.
template <typename IO, int TS, int LANES, int CH, int NSTAGE, bool USE_TMA, bool CONV, bool MERGE, bool GROUPED>
__global__ void __maxnreg__(96)
    rglru_fwd_kernel_capped(const __grid_constant__ FwdMaps maps, const ScanFwdArgs p) {
  rglru_fwd_body<IO, TS, LANES, CH, NSTAGE, USE_TMA, CONV, MERGE, GROUPED>(maps, p);
}

// ======================================================================
// Backward
// ======================================================================

template <typename IO, int TS>
struct BwdRegs {
  float2 am[TS][2];  // decay after masking
  float2 hb[TS][2];  // drive b, later the state entering the step
  float2 ar[TS][2];  // unmasked decay, zeroed where the decay receives no gradient
  float2 c1[TS][2];  // d x      = g * c1
  float2 c2[TS][2];  // d u_i    = g * c2
  float2 c3[TS][2];  // d log a  = g * (h_prev * ar + c3)   (c3 <= 0 side of the sqrt slope term)
  float2 rr[TS][2];  // recurrence gate r
  typename Pack<IO>::Raw dy[TS];
};

// Level one of the backward chunk: gate math, coefficients for the second pass, and the
// lane aggregates: prod a, the local state, and the local reverse carry,
// where the reverse carry is a_t g_t flowing from step t to step t-1.
// MERGE: the incoming gradient is that of h * gelu(branch).  This pass turns it into the gradient of h
// (kept, rounded to the I/O type, where the incoming gradient was) and leaves d_out * gelu'(branch) in the
// branch tile; the second pass multiplies that by h_t to get the branch gradient.
template <typename IO, int TS, int CH, bool MASKED, bool POLY, bool CONV, bool MERGE, bool GROUPED>
__device__ __forceinline__ void bwd_local(uint8_t* tdy, uint8_t* tg, const uint8_t* tx, const uint8_t* tr, const uint8_t* ti,
                                          int off0, const float2 (&K)[2], const uint32_t (&fl)[(TS + 3) / 4],
                                          const ConvTaps& ct, const float2 (*hist)[2], const GateBias& gb,
                                          BwdRegs<IO, TS>& R, float2 (&prod)[2], float2 (&sfwd)[2],
                                          float2 (&crev)[2]) {
  constexpr int ROWB = CH * sizeof(IO);
  float2 p[2] = {f2(1.0f), f2(1.0f)};
  float2 s[2] = {f2(0.0f), f2(0.0f)};
  float2 xc[CONV ? TS : 1][2];
  if (CONV) conv_front<IO, CONV ? TS : 1, CH, MASKED>(tx, off0, ct, fl, hist, xc);
#pragma unroll
  for (int st = 0; st < TS; ++st) {
    const int off = off0 + st * ROWB;
    float2 xv[2], rv[2], iv[2];
    if (CONV) { xv[0] = xc[CONV ? st : 0][0]; xv[1] = xc[CONV ? st : 0][1]; }
    else Pack<IO>::unpack2(Pack<IO>::load(tx + off), xv);
    Pack<IO>::unpack2(Pack<IO>::load(tr + off), rv);
    Pack<IO>::unpack2(Pack<IO>::load(ti + off), iv);
    R.dy[st] = Pack<IO>::load(tdy + off);
    if (MERGE) {
      float2 dm[2], gv[2], q[2];
      Pack<IO>::unpack2(R.dy[st], dm);
      Pack<IO>::unpack2(Pack<IO>::load(tg + off), gv);
#pragma unroll
      for (int cp = 0; cp < 2; ++cp) {
        const float2 sg = gelu_sigmoid2<sizeof(IO) == 2>(gv[cp]);
        q[cp] = mul2(dm[cp], gelu_slope2(gv[cp], sg));
        dm[cp] = mul2(dm[cp], mul2(gv[cp], sg));
      }
      R.dy[st] = Pack<IO>::pack2(dm);
      Pack<IO>::store2(tg + off, q);
    }
    const RowMask m = row_mask<MASKED>(fl[st >> 2], st);
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
      float2 r, i;
      if (GROUPED) sigmoid_pair2_biased<sizeof(IO) == 2>(rv[cp], iv[cp], gb.r[cp], gb.i[cp], r, i);
      else sigmoid_pair2<sizeof(IO) == 2>(rv[cp], iv[cp], r, i);
      const float2 e = one_minus_exp_neg2<POLY, sizeof(IO) == 2>(mul2(r, K[cp]));       // 1 - a
      const float2 a = fma2(e, f2(-1.0f), f2(1.0f));
      float2 gsq = mul2(e, fma2(e, f2(-1.0f), f2(2.0f)));               // 1 - a^2
      // The offset keeps rsqrt finite; it changes gamma by at most 1e-15.
      gsq = add2(gsq, f2(1e-30f));
      const float2 rs = make_float2(rsqrt_approx(gsq.x), rsqrt_approx(gsq.y));
      float2 gam = mul2(gsq, rs);                                       // sqrt(gsq)
      // -2 * slope, slope = 1 / sqrt(max(4 gsq, 1e-6)) = min(rs / 2, 1000); the sign rides on the min for free
      const float2 nrs2 = make_float2(-fminf(rs.x, 2.0f * SLOPE_CAP), -fminf(rs.y, 2.0f * SLOPE_CAP));
      const float2 ix = mul2(i, xv[cp]);
      float2 am = a, ar = a;
      // slope term of d log a, stored negated: -2 a^2 slope i x.  Unmasked, one factor a is left to the second
      // pass, which has a g at hand as the reverse carry.
      float2 c3 = MASKED ? mul2(mul2(a, a), mul2(nrs2, ix)) : mul2(a, mul2(nrs2, ix));
      if (MASKED) {
        const float kl = m.keep * m.live;
        am = fma2(mul2(a, f2(m.keep)), f2(m.live), f2(1.0f - m.live));
        ar = mul2(a, f2(kl));
        c3 = mul2(c3, f2(kl));
        gam = mul2(fma2(gam, f2(m.keep), f2(1.0f - m.keep)), f2(m.live));
      }
      const float2 c1 = mul2(gam, i);
      const float2 bb = mul2(gam, ix);
      R.am[st][cp] = am;
      if (MASKED) R.ar[st][cp] = ar;
      R.c1[st][cp] = c1;
      R.c2[st][cp] = mul2(bb, fma2(i, f2(-1.0f), f2(1.0f)));
      R.c3[st][cp] = c3;
      R.rr[st][cp] = r;
      R.hb[st][cp] = bb;
      p[cp] = mul2(p[cp], am);
      s[cp] = fma2(am, s[cp], bb);
    }
  }
  float2 c[2] = {f2(0.0f), f2(0.0f)};
#pragma unroll
  for (int st = TS - 1; st >= 0; --st) {
    float2 dyv[2];
    Pack<IO>::unpack2(R.dy[st], dyv);
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) c[cp] = mul2(R.am[st][cp], add2(dyv[cp], c[cp]));
  }
#pragma unroll
  for (int cp = 0; cp < 2; ++cp) { prod[cp] = p[cp]; sfwd[cp] = s[cp]; crev[cp] = c[cp]; }
}

// Second pass of the backward chunk: with the state `hin` entering the thread's first step and the reverse
// carry `cin` entering its last, rebuild the states, run the reverse recurrence and write dx, du_r, du_i (and,
// merged, the branch gradient) over the input tiles.  MASKED = false is the path of a thread whose tokens are
// all ordinary: the decay that takes the gradient is the decay itself, so R.ar is not read.  The incoming
// gradient is read back from its tile unless the merged variant replaced it in registers.
// SUMS: also accumulate the sums over time of du_r and du_i (the gate-bias gradient of the grouped layout).
template <typename IO, int TS, int CH, bool MASKED, bool CONV, bool MERGE, bool SUMS>
__device__ __forceinline__ void bwd_apply(uint8_t* tiles, int off_dx, int off_dr, int off_di, int off_g, int off0,
                                          const float2 (&K)[2], const float2 (&hin)[2], const float2 (&cin)[2],
                                          BwdRegs<IO, TS>& R, float2 (&dlam)[2], float2 (&dsr)[2], float2 (&dsi)[2]) {
  constexpr int ROWB = CH * sizeof(IO);
  float2 h[2] = {hin[0], hin[1]};
  float2 c[2] = {cin[0], cin[1]};
  // States entering each step, rebuilt forward in time.
#pragma unroll
  for (int st = 0; st < TS; ++st) {
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
      const float2 hprev = h[cp];
      h[cp] = fma2(R.am[st][cp], hprev, R.hb[st][cp]);
      R.hb[st][cp] = hprev;
    }
    if (MERGE) {   // d branch_t = d_out_t * gelu'(branch_t) * h_t, the first two factors left by the first pass
      uint8_t* tq = tiles + off_g + off0 + st * ROWB;
      float2 q[2];
      Pack<IO>::unpack2(Pack<IO>::load(tq), q);
      q[0] = mul2(q[0], h[0]);
      q[1] = mul2(q[1], h[1]);
      Pack<IO>::store2(tq, q);
    }
  }
  uint8_t* tdx = tiles + off_dx;   // over x (past its halo rows)
  uint8_t* tdr = tiles + off_dr;   // over u_r
  uint8_t* tdi = tiles + off_di;   // over u_i
  const float2 nK[2] = {mul2(K[0], f2(-1.0f)), mul2(K[1], f2(-1.0f))};
#pragma unroll
  for (int st = TS - 1; st >= 0; --st) {
    const int off = off0 + st * ROWB;
    float2 dyv[2], dxv[2], drv[2], div[2];
    if (MERGE) Pack<IO>::unpack2(R.dy[st], dyv);
    else Pack<IO>::unpack2(Pack<IO>::load(tiles + off), dyv);
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
      const float2 g = add2(dyv[cp], c[cp]);
      c[cp] = mul2(R.am[st][cp], g);
      dxv[cp] = mul2(g, R.c1[st][cp]);
      div[cp] = mul2(g, R.c2[st][cp]);
      // d log a = g a (h_prev + c3 / a); unmasked, g a is the reverse carry just formed and c3 came divided by a
      const float2 dl = MASKED ? mul2(g, fma2(R.hb[st][cp], R.ar[st][cp], R.c3[st][cp]))
                               : mul2(c[cp], add2(R.hb[st][cp], R.c3[st][cp]));
      const float2 w = mul2(dl, R.rr[st][cp]);
      dlam[cp] = add2(dlam[cp], w);
      // d u_r = dl * d(log a)/d u_r = dl * (-K) r (1 - r) with K = -c logsigmoid(Lambda) >= 0
      drv[cp] = mul2(w, fma2(K[cp], R.rr[st][cp], nK[cp]));
      if (SUMS) {
        dsr[cp] = add2(dsr[cp], drv[cp]);
        dsi[cp] = add2(dsi[cp], div[cp]);
      }
    }
    Pack<IO>::store2(tdx + off, dxv);
    Pack<IO>::store2(tdr + off, drv);
    Pack<IO>::store2(tdi + off, div);
  }
}

template <typename IO, int TS, int LANES, int CH, int NSTAGE, bool CONV = false, bool MERGE = false>
struct BwdSmem {
  static constexpr int TC = LANES * TS;
  static constexpr int TILE = TC * CH * sizeof(IO);
  static constexpr int HALO = CONV ? 3 * CH * sizeof(IO) : 0;   // three rows in front of the x tile
  static constexpr int TILEX = TILE + HALO;
  static constexpr int OFF_X = TILE, OFF_UR = TILE + TILEX, OFF_UI = 2 * TILE + TILEX;   // after the dy tile
  static constexpr int OFF_G = 3 * TILE + TILEX;                // GeLU-branch tile of the merged variant
  static constexpr int STAGE = 3 * TILE + TILEX + (MERGE ? TILE : 0);
  // Lane aggregates as three float planes [LANES][CH]: decay product, local state, local reverse carry.
  static constexpr int PLANE = LANES * CH * 4;
  static constexpr int OFF_AGGP = NSTAGE * STAGE;
  static constexpr int OFF_AGGS = OFF_AGGP + PLANE;
  static constexpr int OFF_AGGC = OFF_AGGS + PLANE;
  static constexpr int OFF_EINF = OFF_AGGC + PLANE;
  static constexpr int OFF_EINR = OFF_EINF + PLANE;
  static constexpr int OFF_BAR = OFF_EINR + PLANE;   // full[NSTAGE], ready[NSTAGE], dead flag
  static constexpr int BYTES = OFF_BAR + 2 * NSTAGE * 8 + 16;
};

// SELF_ISSUE: no producer warp.  One thread of the last compute warp (not a chain thread) issues the bulk
// copies right after the first barrier of a chunk: by then every thread has finished, and fenced, the results
// of the chunk before, so that chunk's tiles can leave and the stage of the chunk before it, whose store has
// been read out of shared memory by now, can be refilled.  No barrier is added; loads run NSTAGE - 2 chunks
// ahead.  A whole number of warps per scheduler partition leaves every thread 128 registers at 512 threads.
// PLAIN: the caller passed no token flags and the sequence is a whole number of chunks, so no step is ever
// masked; the masked arithmetic is not compiled in (half the code, and registers allotted for this path alone).
// CARRY: the carry-only pass of a time-split sequence: no gradient tensors, nothing is stored but dh0.
template <typename IO, int TS, int LANES, int CH, int NSTAGE, bool USE_TMA, bool CONV, bool MERGE, bool GROUPED,
          bool SELF_ISSUE = false, bool PLAIN = false, bool CARRY = false>
__global__ void __launch_bounds__(LANES*(CH / CV) + ((USE_TMA && !SELF_ISSUE) ? 32 : 0),
                                  (SELF_ISSUE && CH == 32) ? 2 : 1)
    rglru_bwd_kernel(const __grid_constant__ BwdMaps maps, const ScanBwdArgs p) {
  using SM = BwdSmem<IO, TS, LANES, CH, NSTAGE, CONV, MERGE>;
  static_assert(!CONV || (SM::HALO % 128 == 0), "the halo must keep the result rows 128-byte aligned for TMA");
  constexpr int NCV = CH / CV;
  constexpr int TC = SM::TC;
  static_assert(TC % SAVE_EVERY == 0, "backward chunks must start on a saved state");
  static_assert(!SELF_ISSUE || !USE_TMA || NSTAGE >= 3, "without a producer warp a stage is refilled two chunks after its use");
  constexpr int ROWB = CH * sizeof(IO);
  constexpr int NCOMP = LANES * NCV;
  extern __shared__ __align__(128) uint8_t smem[];
  float* aggP = reinterpret_cast<float*>(smem + SM::OFF_AGGP);
  float* aggS = reinterpret_cast<float*>(smem + SM::OFF_AGGS);
  float* aggC = reinterpret_cast<float*>(smem + SM::OFF_AGGC);
  float* einF = reinterpret_cast<float*>(smem + SM::OFF_EINF);
  float* einR = reinterpret_cast<float*>(smem + SM::OFF_EINR);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
  uint64_t* ready = full + NSTAGE;
  volatile int* dead = reinterpret_cast<volatile int*>(ready + NSTAGE);

  const int tid = threadIdx.x;
  const int lane_t = tid / NCV;
  const int vec = tid % NCV;
  const int b = blockIdx.y;
  const int d0 = blockIdx.x * CH;
  const int nchunks = (p.T + TC - 1) / TC;
  const int nsave = (p.T + SAVE_EVERY - 1) / SAVE_EVERY;
  static_assert(!GROUPED || USE_TMA, "the grouped gate layout is staged by TMA only");
  const int rcol = GROUPED ? grouped_col(d0, p.gate_bw) : d0;   // first column of this tile's u_r / u_i (and du_r / du_i)
  const int icol = GROUPED ? rcol + p.gate_bw : d0;

  auto issue = [&](int q) {  // q-th chunk in processing order == chunk nchunks-1-q in time
    const int k = nchunks - 1 - q;
    const int sidx = q % NSTAGE;
    uint8_t* st = smem + sidx * SM::STAGE;
    mbar_expect_tx(&full[sidx], SM::STAGE);
    tma_load_3d(st, &maps.dy, d0, k * TC, b, &full[sidx]);
    tma_load_3d(st + SM::OFF_X, &maps.x, d0, k * TC - (CONV ? 3 : 0), b, &full[sidx]);
    tma_load_3d(st + SM::OFF_UR, &maps.ur, rcol, k * TC, b, &full[sidx]);
    tma_load_3d(st + SM::OFF_UI, &maps.ui, icol, k * TC, b, &full[sidx]);
    if (MERGE) tma_load_3d(st + SM::OFF_G, &maps.g, d0, k * TC, b, &full[sidx]);
  };
  auto store = [&](int q) {
    const int k = nchunks - 1 - q;
    uint8_t* st = smem + (q % NSTAGE) * SM::STAGE;
    if (!CARRY) {
      tma_store_3d(&maps.dx, st + SM::OFF_X + SM::HALO, d0, k * TC, b);
      tma_store_3d(&maps.dur, st + SM::OFF_UR, rcol, k * TC, b);
      tma_store_3d(&maps.dui, st + SM::OFF_UI, icol, k * TC, b);
      if (MERGE) tma_store_3d(&maps.dg, st + SM::OFF_G, d0, k * TC, b);
    }
    tma_commit();
  };
  // Set-up by the thread that will issue the bulk copies (the producer warp's first lane, or with SELF_ISSUE
  // the first lane of the last compute warp), published by one early CTA barrier; after it the producer warp
  // and the compute warps go their own ways (the compute warps vote among themselves), so the first loads are
  // issued while the per-channel rates are worked out.
  const bool issuer = USE_TMA && tid == (SELF_ISSUE ? NCOMP - 32 : NCOMP);
  const bool self_issuer = SELF_ISSUE && issuer;
  pdl_launch_dependents();
  if (USE_TMA ? issuer : (tid == 0)) {
    *dead = 0;
    if (USE_TMA) {
      for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full[s], 1); mbar_init(&ready[s], NCOMP / 32); }
      mbar_fence_init();
      prefetch_map(&maps.dy); prefetch_map(&maps.x); prefetch_map(&maps.ur); prefetch_map(&maps.ui);
      prefetch_map(&maps.dx); prefetch_map(&maps.dur); prefetch_map(&maps.dui);
      if (MERGE) { prefetch_map(&maps.g); prefetch_map(&maps.dg); }
      // While the kernel in front of this one on the stream drains, pull the first chunk (the last in time)
      // towards L2.
      const int kl = nchunks - 1;
      tma_prefetch_3d(&maps.dy, d0, kl * TC, b);
      tma_prefetch_3d(&maps.x, d0, kl * TC - (CONV ? 3 : 0), b);
      tma_prefetch_3d(&maps.ur, rcol, kl * TC, b);
      tma_prefetch_3d(&maps.ui, icol, kl * TC, b);
      if (MERGE) tma_prefetch_3d(&maps.g, d0, kl * TC, b);
    }
  }
  __syncthreads();
  pdl_wait();   // nothing above touches global memory; everything below may depend on the previous kernel

  if (USE_TMA && !SELF_ISSUE && tid >= NCOMP) {
    // ---- producer warp (chunks are walked from the end of the sequence to its start)
    if (tid == NCOMP) {
      // the first chunk is asked for alone, the rest once it has landed (see the forward kernel)
      issue(0);
      mbar_wait_or_flag(&full[0], 0, dead, p.status, DEV_TIMEOUT_LOAD);
      for (int q = 1; q < NSTAGE && q < nchunks; ++q) issue(q);
      for (int q = 0; q < nchunks; ++q) {
        const int sidx = q % NSTAGE;
        mbar_wait_or_flag(&ready[sidx], (q / NSTAGE) & 1, dead, p.status, DEV_TIMEOUT_STORE);
        store(q);
        if (q + NSTAGE < nchunks) {
          tma_wait_read<0>();
          issue(q + NSTAGE);
        }
      }
      tma_wait_all<0>();
    }
    return;
  }

  if (self_issuer) issue(0);    // the first chunk before this thread's share of the prologue, the rest after it
  float2 K[2];
  {
    const int d = d0 + vec * CV;
    K[0] = make_float2(decay_rate(p.lambda, d, p.D, p.c), decay_rate(p.lambda, d + 1, p.D, p.c));
    K[1] = make_float2(decay_rate(p.lambda, d + 2, p.D, p.c), decay_rate(p.lambda, d + 3, p.D, p.c));
  }
  const bool poly = bar_compute_and(NCOMP, fmaxf(fmaxf(K[0].x, K[0].y), fmaxf(K[1].x, K[1].y)) <= -POLY_RANGE);

  // Threads 0..63 chain the forward lane aggregates, threads 64..127 the reverse ones.
  const int cch = tid & (CH - 1);
  const int dch = d0 + cch;
  const bool fwd_chain = tid < CH;
  const bool rev_chain = tid >= CH && tid < 2 * CH;
  float carry_rev = 0.0f;
  if (rev_chain && dch < p.D && p.dh_last) carry_rev = p.dh_last[static_cast<size_t>(b) * p.D + dch];

  ConvTaps ct;
  if (CONV) load_taps(p.conv_w, p.conv_b, d0 + vec * CV, p.D, ct);
  GateBias gb;
  if (GROUPED) load_gate_bias<sizeof(IO) == 2>(p.gate_bias, rcol + vec * CV, icol + vec * CV, gb);

  float2 dlam[2] = {f2(0.0f), f2(0.0f)};
  float2 dsr[2] = {f2(0.0f), f2(0.0f)}, dsi[2] = {f2(0.0f), f2(0.0f)};   // grouped layout: sums over time of du_r, du_i
  const int off0 = (lane_t * TS) * ROWB + vec * Pack<IO>::BYTES;

  for (int q = 0; q < nchunks; ++q) {
    const int k = nchunks - 1 - q;
    const int stage = USE_TMA ? (q % NSTAGE) : 0;
    uint8_t* tiles = smem + stage * SM::STAGE;
    const int t0 = k * TC;
    uint32_t fl[(TS + 3) / 4];
    const bool masked = !PLAIN && ((p.tok != nullptr) || (t0 + TC > p.T));
    if (masked) load_flags<TS>(p.tok, b, p.T, t0 + lane_t * TS, fl);

    // State entering this chunk (saved by the forward kernel; chunk 0 starts from h0).
    float enter = 0.0f;
    if (fwd_chain && dch < p.D) {
      if (k == 0) enter = p.h0 ? p.h0[static_cast<size_t>(b) * p.D + dch] : 0.0f;
      else enter = p.states[(static_cast<size_t>(b) * nsave + t0 / SAVE_EVERY) * p.D + dch];
    }

    if (USE_TMA) {
      mbar_wait_or_flag(&full[stage], (q / NSTAGE) & 1, dead, p.status, DEV_TIMEOUT_LOAD);
      if (self_issuer && q == 0)      // the first chunk was asked for alone; now that it has landed, the rest
        for (int qq = 1; qq < NSTAGE && qq < nchunks; ++qq) issue(qq);
    } else {
      tile_load_plain<IO, CH>(tiles, p.dy, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<IO, CH>(tiles + SM::OFF_X, p.x, b, t0 - (CONV ? 3 : 0), d0, TC + (CONV ? 3 : 0), p.T, p.D);
      tile_load_plain<IO, CH>(tiles + SM::OFF_UR, p.ur, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<IO, CH>(tiles + SM::OFF_UI, p.ui, b, t0, d0, TC, p.T, p.D);
      if (MERGE) tile_load_plain<IO, CH>(tiles + SM::OFF_G, p.g, b, t0, d0, TC, p.T, p.D);
      bar_compute(NCOMP);
    }

    BwdRegs<IO, TS> R;
    float2 prod[2], sfwd[2], crev[2];
    const bool flagged = masked && any_flag(fl);
    {
      uint8_t* tdy = tiles;
      uint8_t* tg = tiles + SM::OFF_G;
      const uint8_t* tx = tiles + SM::OFF_X;
      const uint8_t* tr = tiles + SM::OFF_UR;
      const uint8_t* ti = tiles + SM::OFF_UI;
      float2 hist_v[3][2];
      const float2 (*hist)[2] = nullptr;
      if (CONV && k == 0 && lane_t == 0 && p.conv_state) {
        load_hist<IO>(p.conv_state, b, d0 + vec * CV, p.D, hist_v);
        hist = hist_v;
      }
      if (flagged) {
        if (poly) bwd_local<IO, TS, CH, true, true, CONV, MERGE, GROUPED>(tdy, tg, tx, tr, ti, off0, K, fl, ct, hist, gb, R, prod, sfwd, crev);
        else bwd_local<IO, TS, CH, true, false, CONV, MERGE, GROUPED>(tdy, tg, tx, tr, ti, off0, K, fl, ct, hist, gb, R, prod, sfwd, crev);
      } else {
        if (poly) bwd_local<IO, TS, CH, false, true, CONV, MERGE, GROUPED>(tdy, tg, tx, tr, ti, off0, K, fl, ct, hist, gb, R, prod, sfwd, crev);
        else bwd_local<IO, TS, CH, false, false, CONV, MERGE, GROUPED>(tdy, tg, tx, tr, ti, off0, K, fl, ct, hist, gb, R, prod, sfwd, crev);
      }
    }
    {
      const int ao = lane_t * CH + vec * CV;
      *reinterpret_cast<float4*>(aggP + ao) = make_float4(prod[0].x, prod[0].y, prod[1].x, prod[1].y);
      *reinterpret_cast<float4*>(aggS + ao) = make_float4(sfwd[0].x, sfwd[0].y, sfwd[1].x, sfwd[1].y);
      *reinterpret_cast<float4*>(aggC + ao) = make_float4(crev[0].x, crev[0].y, crev[1].x, crev[1].y);
    }
    bar_compute(NCOMP);
    if (self_issuer && q >= 1) {
      store(q - 1);
      if (q >= 2 && q - 2 + NSTAGE < nchunks) {
        tma_wait_read<1>();      // all but the store just committed have been read out: the stage of chunk q-2 is free
        issue(q - 2 + NSTAGE);
      }
    }

    if (fwd_chain || rev_chain) {
      const float* plane = fwd_chain ? aggS : aggC;
      float* ein = fwd_chain ? einF : einR;
      float ap[LANES], as[LANES];
#pragma unroll
      for (int j = 0; j < LANES; ++j) { ap[j] = aggP[j * CH + cch]; as[j] = plane[j * CH + cch]; }
      if (fwd_chain) {
        float e = enter;
#pragma unroll
        for (int j = 0; j < LANES; ++j) {
          ein[j * CH + cch] = e;
          e = fmaf(ap[j], e, as[j]);
        }
      } else {
        float e = carry_rev;
#pragma unroll
        for (int j = LANES - 1; j >= 0; --j) {
          ein[j * CH + cch] = e;
          e = fmaf(ap[j], e, as[j]);
        }
        carry_rev = e;
      }
    }
    bar_compute(NCOMP);

    {
      const float4 f4 = *reinterpret_cast<const float4*>(einF + lane_t * CH + vec * CV);
      const float4 r4 = *reinterpret_cast<const float4*>(einR + lane_t * CH + vec * CV);
      const float2 hin[2] = {make_float2(f4.x, f4.y), make_float2(f4.z, f4.w)};
      const float2 cin[2] = {make_float2(r4.x, r4.y), make_float2(r4.z, r4.w)};
      if (flagged) bwd_apply<IO, TS, CH, true, CONV, MERGE, GROUPED>(tiles, SM::OFF_X + SM::HALO, SM::OFF_UR, SM::OFF_UI, SM::OFF_G, off0, K, hin, cin, R, dlam, dsr, dsi);
      else bwd_apply<IO, TS, CH, false, CONV, MERGE, GROUPED>(tiles, SM::OFF_X + SM::HALO, SM::OFF_UR, SM::OFF_UI, SM::OFF_G, off0, K, hin, cin, R, dlam, dsr, dsi);
    }
    if (USE_TMA && SELF_ISSUE) {
      fence_async_smem();          // the stage leaves after the next barrier all threads pass
    } else if (USE_TMA) {
      fence_async_smem();
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(&ready[stage]);   // one arrival per warp
    } else {
      bar_compute(NCOMP);
      if (!CARRY) {
        tile_store_plain<IO, CH>(tiles + SM::OFF_X + SM::HALO, p.dx, b, t0, d0, TC, p.T, p.D);
        tile_store_plain<IO, CH>(tiles + SM::OFF_UR, p.dur, b, t0, d0, TC, p.T, p.D);
        tile_store_plain<IO, CH>(tiles + SM::OFF_UI, p.dui, b, t0, d0, TC, p.T, p.D);
        if (MERGE) tile_store_plain<IO, CH>(tiles + SM::OFF_G, p.dg, b, t0, d0, TC, p.T, p.D);
      }
      bar_compute(NCOMP);
    }
  }

  if (rev_chain && dch < p.D && p.dh0) p.dh0[static_cast<size_t>(b) * p.D + dch] = carry_rev;

  // Per-row partial of sum_t dl * r: fold the time-lanes in a fixed order.
  bar_compute(NCOMP);
  if (self_issuer) store(nchunks - 1);     // the last chunk's results; the issuing thread drains its stores on its way out
  auto drain = [&]() { if (USE_TMA && SELF_ISSUE && self_issuer) tma_wait_all<0>(); };
  *reinterpret_cast<float4*>(einF + lane_t * CH + vec * CV) = make_float4(dlam[0].x, dlam[0].y, dlam[1].x, dlam[1].y);
  if (GROUPED) {   // the chain planes are free now: the two gate sums go through them the same way
    *reinterpret_cast<float4*>(einR + lane_t * CH + vec * CV) = make_float4(dsr[0].x, dsr[0].y, dsr[1].x, dsr[1].y);
    *reinterpret_cast<float4*>(aggP + lane_t * CH + vec * CV) = make_float4(dsi[0].x, dsi[0].y, dsi[1].x, dsi[1].y);
  }
  bar_compute(NCOMP);
  static_assert(!GROUPED || NCOMP >= 3 * CH, "one thread per channel and sum");
  if (tid < (GROUPED ? 3 * CH : CH) && dch < p.D) {
    const int which = tid / CH;                       // 0: dLambda partial, 1: sum du_r, 2: sum du_i
    const float* plane = which == 0 ? einF : (which == 1 ? einR : aggP);
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < LANES; ++j) acc += plane[j * CH + cch];
    if (which == 0) p.dlam_part[static_cast<size_t>(b) * p.D + dch] = acc;
    else if (p.dgate_part) p.dgate_part[static_cast<size_t>(b) * 2 * p.D + (which == 1 ? rcol : icol) + cch] = acc;
  }
  if (!p.ticket) { drain(); return; }   // the caller folds the rows with rglru_dlambda_kernel

  // The CTA that finishes last folds the per-row partials into dLambda (rows in index order, so the
  // result does not depend on which CTA that is) and re-arms the ticket for the next backward call.
  // The ticket is one acquire-release atomic by one thread between two CTA barriers: the barrier in front makes
  // the partial rows every thread of this CTA stored part of what the release publishes, the barrier behind makes
  // what the acquire saw (the other CTAs' rows) visible to every thread that goes on to read them, past L1.
  __shared__ int s_last;
  bar_compute(NCOMP);
  if (tid == 0) {
    const unsigned total = gridDim.x * gridDim.y;
    unsigned before;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(before) : "l"(p.ticket), "r"(1u) : "memory");
    s_last = (before == total - 1u) ? 1 : 0;
  }
  bar_compute(NCOMP);
  if (!s_last) { drain(); return; }
  // Rows are added in index order whatever the load order; loads go out eight rows at a time so that the
  // fold costs a few round trips to L2, not one per row.
  if ((p.D & 3) == 0) {
    for (int d = tid * 4; d < p.D; d += NCOMP * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r0 = 0; r0 < p.B; r0 += 8) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[j] = (r0 + j < p.B) ? __ldcg(reinterpret_cast<const float4*>(p.dlam_part + static_cast<size_t>(r0 + j) * p.D + d))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
      }
      const float4 lam = *reinterpret_cast<const float4*>(p.lambda + d);
      float4 out;
      out.x = (1.0f / (1.0f + expf(lam.x))) * p.c * acc.x;
      out.y = (1.0f / (1.0f + expf(lam.y))) * p.c * acc.y;
      out.z = (1.0f / (1.0f + expf(lam.z))) * p.c * acc.z;
      out.w = (1.0f / (1.0f + expf(lam.w))) * p.c * acc.w;
      *reinterpret_cast<float4*>(p.dlambda + d) = out;
    }
  } else {
    for (int d = tid; d < p.D; d += NCOMP) {
      float acc = 0.0f;
      for (int r = 0; r < p.B; ++r) acc += __ldcg(p.dlam_part + static_cast<size_t>(r) * p.D + d);
      const float lam = p.lambda[d];
      p.dlambda[d] = (1.0f / (1.0f + expf(lam))) * p.c * acc;
    }
  }
  if (GROUPED && p.dgate && p.dgate_part) {     // gate-bias gradient: column sums of du over the batch rows
    const int N2 = 2 * p.D;                     // a multiple of 4: the grouped layout needs 64-channel gate heads
    for (int d = tid * 4; d < N2; d += NCOMP * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r0 = 0; r0 < p.B; r0 += 8) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[j] = (r0 + j < p.B) ? __ldcg(reinterpret_cast<const float4*>(p.dgate_part + static_cast<size_t>(r0 + j) * N2 + d))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
      }
      *reinterpret_cast<float4*>(p.dgate + d) = acc;
    }
  }
  if (tid == 0) *p.ticket = 0u;
  drain();
}

// out[n] = sum_b part[b, n], rows added in index order (gate-bias gradient when the batch is too large for the
// backward kernel's own fold).
__global__ void rglru_colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int B, int N) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float acc = 0.0f;
  for (int b = 0; b < B; ++b) acc += part[static_cast<size_t>(b) * N + n];
  out[n] = acc;
}

// dLambda[d] = d/dLambda of sum dl * r * c * logsigmoid(Lambda) = sigmoid(-Lambda_d) * c * sum_b partial[b, d],
// rows added in index order.
__global__ void rglru_dlambda_kernel(const float* __restrict__ part, const float* __restrict__ lambda,
                                     float* __restrict__ dlambda, int B, int D, float c) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float acc = 0.0f;
  for (int b = 0; b < B; ++b) acc += part[static_cast<size_t>(b) * D + d];
  const float lam = lambda[d];
  const float sig_neg = 1.0f / (1.0f + expf(lam));
  dlambda[d] = sig_neg * c * acc;
}

// ======================================================================
// Raw affine scan h_t = a_t h_{t-1} + b_t on fp32 tensors (operator-level drop-in
// for griffin/triton_scan.py:274-276).  Same two-level structure, no gate math.
// ======================================================================

constexpr int CH = 64;
constexpr int NCV = CH / CV;
constexpr int RAW_TS = 4;
constexpr int RAW_LANES = 16;
constexpr int RAW_NT = RAW_LANES * NCV;
constexpr int RAW_TC = RAW_LANES * RAW_TS;
constexpr int RAW_TILE = RAW_TC * CH * 4;

template <int NSTAGE>
struct RawSmem {
  static constexpr int NTILE = 3;
  static constexpr int STAGE = NTILE * RAW_TILE;
  static constexpr int OFF_AGG = NSTAGE * STAGE;
  static constexpr int OFF_EIN = OFF_AGG + ChainSmem<RAW_LANES, CH>::AGG;
  static constexpr int OFF_BAR = OFF_EIN + ChainSmem<RAW_LANES, CH>::EIN;
  static constexpr int BYTES = OFF_BAR + NSTAGE * 8 + 16;
};

template <int NSTAGE, bool USE_TMA>
__global__ void __launch_bounds__(RAW_NT) rawscan_fwd_kernel(const __grid_constant__ RawFwdMaps maps, const RawScanArgs p) {
  using SM = RawSmem<NSTAGE>;
  constexpr int TS = RAW_TS, TC = RAW_TC, ROWB = CH * 4, LANES = RAW_LANES;
  extern __shared__ __align__(128) uint8_t smem[];
  float2* agg = reinterpret_cast<float2*>(smem + SM::OFF_AGG);
  float* ein = reinterpret_cast<float*>(smem + SM::OFF_EIN);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
  const int tid = threadIdx.x, lane_t = tid / NCV, vec = tid % NCV;
  const int b = blockIdx.y, d0 = blockIdx.x * CH;
  const int nchunks = (p.T + TC - 1) / TC;

  auto issue = [&](int k) {
    const int sidx = k % NSTAGE;
    uint8_t* st = smem + sidx * SM::STAGE;
    mbar_expect_tx(&bars[sidx], 2 * RAW_TILE);
    tma_load_3d(st, &maps.drive, d0, k * TC, b, &bars[sidx]);
    tma_load_3d(st + RAW_TILE, &maps.decay, d0, k * TC, b, &bars[sidx]);
  };
  if (USE_TMA) {
    if (tid == 0) {
      for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[s], 1);
      mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0)
      for (int k = 0; k < NSTAGE && k < nchunks; ++k) issue(k);
  }
  float carry = 0.0f;
  const int dch = d0 + tid;
  if (tid < CH && dch < p.D && p.h0) carry = p.h0[static_cast<size_t>(b) * p.D + dch];
  const int off0 = (lane_t * TS) * ROWB + vec * 16;
  bool alive = true;

  for (int k = 0; k < nchunks; ++k) {
    const int stage = USE_TMA ? (k % NSTAGE) : 0;
    uint8_t* tiles = smem + stage * SM::STAGE;
    const int t0 = k * TC;
    if (USE_TMA) {
      alive = mbar_wait_bounded(&bars[stage], (k / NSTAGE) & 1);
    } else {
      tile_load_plain<float, CH>(tiles, p.drive, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<float, CH>(tiles + RAW_TILE, p.decay, b, t0, d0, TC, p.T, p.D);
      __syncthreads();
    }
    float2 P[TS][2], S[TS][2];
    {
      float2 pp[2] = {f2(1.0f), f2(1.0f)}, ss[2] = {f2(0.0f), f2(0.0f)};
#pragma unroll
      for (int st = 0; st < TS; ++st) {
        float2 bv[2], av[2];
        Pack<float>::unpack2(Pack<float>::load(tiles + off0 + st * ROWB), bv);
        Pack<float>::unpack2(Pack<float>::load(tiles + RAW_TILE + off0 + st * ROWB), av);
        const float live = (t0 + lane_t * TS + st < p.T) ? 1.0f : 0.0f;  // steps past T carry the state through
#pragma unroll
        for (int cp = 0; cp < 2; ++cp) {
          const float2 a = fma2(av[cp], f2(live), f2(1.0f - live));
          const float2 bb = mul2(bv[cp], f2(live));
          pp[cp] = mul2(pp[cp], a);
          ss[cp] = fma2(a, ss[cp], bb);
          P[st][cp] = pp[cp];
          S[st][cp] = ss[cp];
        }
      }
    }
    {
      float4* dst = reinterpret_cast<float4*>(agg + lane_t * CH + vec * CV);
      dst[0] = make_float4(P[TS - 1][0].x, S[TS - 1][0].x, P[TS - 1][0].y, S[TS - 1][0].y);
      dst[1] = make_float4(P[TS - 1][1].x, S[TS - 1][1].x, P[TS - 1][1].y, S[TS - 1][1].y);
    }
    alive = __syncthreads_and(alive);
    if (!alive) break;
    if (tid < CH) {
      float2 ag[LANES];
#pragma unroll
      for (int j = 0; j < LANES; ++j) ag[j] = agg[j * CH + tid];
      float e = carry;
#pragma unroll
      for (int j = 0; j < LANES; ++j) {
        ein[j * CH + tid] = e;
        e = fmaf(ag[j].x, e, ag[j].y);
      }
      carry = e;
    }
    __syncthreads();
    {
      const float4 e4 = *reinterpret_cast<const float4*>(ein + lane_t * CH + vec * CV);
      const float2 e[2] = {make_float2(e4.x, e4.y), make_float2(e4.z, e4.w)};
#pragma unroll
      for (int st = 0; st < TS; ++st) {
        float2 yv[2];
#pragma unroll
        for (int cp = 0; cp < 2; ++cp) yv[cp] = fma2(P[st][cp], e[cp], S[st][cp]);
        Pack<float>::store2(tiles + off0 + st * ROWB, yv);
      }
    }
    if (USE_TMA) {
      fence_async_smem();
      __syncthreads();
      if (tid == 0) {
        tma_store_3d(&maps.out, tiles, d0, t0, b);
        tma_commit();
        const int kp = k - 1;
        if (kp >= 0 && kp + NSTAGE < nchunks) {
          tma_wait_read<1>();
          issue(kp + NSTAGE);
        }
      }
    } else {
      __syncthreads();
      tile_store_plain<float, CH>(tiles, p.out, b, t0, d0, TC, p.T, p.D);
      __syncthreads();
    }
  }
  if (USE_TMA && tid == 0) {
    tma_wait_all<0>();
    if (!alive) atomicExch(p.status, DEV_TIMEOUT_LOAD);
  }
}

// Backward of the raw scan.  Tiles per chunk: d_out, decay, and the forward output
// shifted one step back in time (row t holds h_{t-1}; the row before t = 0 is h0).
template <int NSTAGE, bool USE_TMA>
__global__ void __launch_bounds__(RAW_NT) rawscan_bwd_kernel(const __grid_constant__ RawBwdMaps maps, const RawScanArgs p) {
  using SM = RawSmem<NSTAGE>;
  constexpr int TS = RAW_TS, TC = RAW_TC, ROWB = CH * 4, LANES = RAW_LANES;
  extern __shared__ __align__(128) uint8_t smem[];
  float2* agg = reinterpret_cast<float2*>(smem + SM::OFF_AGG);
  float* ein = reinterpret_cast<float*>(smem + SM::OFF_EIN);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
  const int tid = threadIdx.x, lane_t = tid / NCV, vec = tid % NCV;
  const int b = blockIdx.y, d0 = blockIdx.x * CH;
  const int nchunks = (p.T + TC - 1) / TC;

  auto issue = [&](int q) {
    const int k = nchunks - 1 - q;
    const int sidx = q % NSTAGE;
    uint8_t* st = smem + sidx * SM::STAGE;
    mbar_expect_tx(&bars[sidx], 3 * RAW_TILE);
    tma_load_3d(st, &maps.dout, d0, k * TC, b, &bars[sidx]);
    tma_load_3d(st + RAW_TILE, &maps.decay, d0, k * TC, b, &bars[sidx]);
    tma_load_3d(st + 2 * RAW_TILE, &maps.out, d0, k * TC - 1, b, &bars[sidx]);
  };
  if (USE_TMA) {
    if (tid == 0) {
      for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[s], 1);
      mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0)
      for (int q = 0; q < NSTAGE && q < nchunks; ++q) issue(q);
  }
  float carry = 0.0f;  // a_t g_t flowing towards earlier steps
  const int dch = d0 + tid;
  const int off0 = (lane_t * TS) * ROWB + vec * 16;
  bool alive = true;

  for (int q = 0; q < nchunks; ++q) {
    const int k = nchunks - 1 - q;
    const int stage = USE_TMA ? (q % NSTAGE) : 0;
    uint8_t* tiles = smem + stage * SM::STAGE;
    const int t0 = k * TC;
    if (USE_TMA) {
      alive = mbar_wait_bounded(&bars[stage], (q / NSTAGE) & 1);
    } else {
      tile_load_plain<float, CH>(tiles, p.dout, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<float, CH>(tiles + RAW_TILE, p.decay, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<float, CH>(tiles + 2 * RAW_TILE, p.out_in, b, t0 - 1, d0, TC, p.T, p.D);
      __syncthreads();
    }
    float2 av[TS][2], gv[TS][2], hv[TS][2];
    float2 qq[2] = {f2(1.0f), f2(1.0f)}, cc[2] = {f2(0.0f), f2(0.0f)};
#pragma unroll
    for (int st = 0; st < TS; ++st) {
      Pack<float>::unpack2(Pack<float>::load(tiles + off0 + st * ROWB), gv[st]);
      Pack<float>::unpack2(Pack<float>::load(tiles + RAW_TILE + off0 + st * ROWB), av[st]);
      Pack<float>::unpack2(Pack<float>::load(tiles + 2 * RAW_TILE + off0 + st * ROWB), hv[st]);
    }
    if (k == 0 && lane_t == 0) {  // the state entering t = 0
      float h0v[CV];
#pragma unroll
      for (int ch = 0; ch < CV; ++ch) {
        const int d = d0 + vec * CV + ch;
        h0v[ch] = (p.h0 && d < p.D) ? p.h0[static_cast<size_t>(b) * p.D + d] : 0.0f;
      }
      hv[0][0] = make_float2(h0v[0], h0v[1]);
      hv[0][1] = make_float2(h0v[2], h0v[3]);
    }
#pragma unroll
    for (int st = TS - 1; st >= 0; --st)
#pragma unroll
      for (int cp = 0; cp < 2; ++cp) {
        cc[cp] = mul2(av[st][cp], add2(gv[st][cp], cc[cp]));
        qq[cp] = mul2(qq[cp], av[st][cp]);
      }
    {
      float4* dst = reinterpret_cast<float4*>(agg + lane_t * CH + vec * CV);
      dst[0] = make_float4(qq[0].x, cc[0].x, qq[0].y, cc[0].y);
      dst[1] = make_float4(qq[1].x, cc[1].x, qq[1].y, cc[1].y);
    }
    alive = __syncthreads_and(alive);
    if (!alive) break;
    if (tid < CH) {
      float2 ag[LANES];
#pragma unroll
      for (int j = 0; j < LANES; ++j) ag[j] = agg[j * CH + tid];
      float e = carry;
#pragma unroll
      for (int j = LANES - 1; j >= 0; --j) {
        ein[j * CH + tid] = e;
        e = fmaf(ag[j].x, e, ag[j].y);
      }
      carry = e;
    }
    __syncthreads();
    {
      const float4 e4 = *reinterpret_cast<const float4*>(ein + lane_t * CH + vec * CV);
      float2 c[2] = {make_float2(e4.x, e4.y), make_float2(e4.z, e4.w)};
#pragma unroll
      for (int st = TS - 1; st >= 0; --st) {
        float2 da[2], db[2];
#pragma unroll
        for (int cp = 0; cp < 2; ++cp) {
          const float2 g = add2(gv[st][cp], c[cp]);
          c[cp] = mul2(av[st][cp], g);
          db[cp] = g;
          da[cp] = mul2(g, hv[st][cp]);
        }
        Pack<float>::store2(tiles + off0 + st * ROWB, db);
        Pack<float>::store2(tiles + RAW_TILE + off0 + st * ROWB, da);
      }
    }
    if (USE_TMA) {
      fence_async_smem();
      __syncthreads();
      if (tid == 0) {
        tma_store_3d(&maps.ddrive, tiles, d0, t0, b);
        tma_store_3d(&maps.ddecay, tiles + RAW_TILE, d0, t0, b);
        tma_commit();
        const int qp = q - 1;
        if (qp >= 0 && qp + NSTAGE < nchunks) {
          tma_wait_read<1>();
          issue(qp + NSTAGE);
        }
      }
    } else {
      __syncthreads();
      tile_store_plain<float, CH>(tiles, p.ddrive, b, t0, d0, TC, p.T, p.D);
      tile_store_plain<float, CH>(tiles + RAW_TILE, p.ddecay, b, t0, d0, TC, p.T, p.D);
      __syncthreads();
    }
  }
  if (USE_TMA && tid == 0) {
    tma_wait_all<0>();
    if (!alive) atomicExch(p.status, DEV_TIMEOUT_LOAD);
  }
  if (alive && tid < CH && dch < p.D && p.dh0) p.dh0[static_cast<size_t>(b) * p.D + dch] = carry;
}

// ======================================================================
// The conv alone (griffin/griffin.py:474-487 of the reference), staged like the scan:
// a CTA owns 64 channels of one batch row and walks the sequence in 64-step chunks
// that a producer warp moves through shared memory with TMA; there is no cross-thread
// dependence, so the only synchronisation is the mbarrier pipeline itself.
// Used when B * ceil(D / 64) CTAs fill the machine; otherwise the per-run kernels of
// rglru_conv.cu, which also split the time axis, are the better fit.
// ======================================================================

template <typename IO, int NSTAGE>
struct ConvFwdSmem {
  static constexpr int TS = 4, LANES = 16, CH = 64, TC = LANES * TS;
  static constexpr int TILE = TC * CH * sizeof(IO);
  static constexpr int HALO = 3 * CH * sizeof(IO);
  static constexpr int TILEX = TILE + HALO;     // input rows t0-3 .. t0+TC-1
  static constexpr int STAGE = TILEX + TILE;    // + the result tile
  static constexpr int OFF_BAR = NSTAGE * STAGE;
  static constexpr int BYTES = OFF_BAR + 2 * NSTAGE * 8 + 16;
};

template <typename IO, int NSTAGE>
__global__ void __launch_bounds__(288) conv_tma_fwd_kernel(const __grid_constant__ ConvMaps maps, const ConvTmaArgs p) {
  using SM = ConvFwdSmem<IO, NSTAGE>;
  constexpr int TS = SM::TS, CH = SM::CH, TC = SM::TC, NCV = CH / CV, NCOMP = SM::LANES * NCV;
  constexpr int ROWB = CH * sizeof(IO);
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
  uint64_t* ready = full + NSTAGE;
  volatile int* dead = reinterpret_cast<volatile int*>(ready + NSTAGE);
  const int tid = threadIdx.x, lane_t = tid / NCV, vec = tid % NCV;
  const int b = blockIdx.y, d0 = blockIdx.x * CH;
  const int nchunks = (p.T + TC - 1) / TC;

  if (tid == 0) {
    *dead = 0;
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full[s], 1); mbar_init(&ready[s], NCOMP / 32); }
    mbar_fence_init();
  }
  __syncthreads();

  if (tid >= NCOMP) {
    if (tid == NCOMP) {
      prefetch_map(&maps.in0); prefetch_map(&maps.out0);
      auto issue = [&](int k) {
        const int sidx = k % NSTAGE;
        mbar_expect_tx(&full[sidx], SM::TILEX);
        tma_load_3d(smem + sidx * SM::STAGE, &maps.in0, d0, k * TC - 3, b, &full[sidx]);   // rows before t = 0 read as zero
      };
      for (int k = 0; k < NSTAGE && k < nchunks; ++k) issue(k);
      for (int k = 0; k < nchunks; ++k) {
        const int sidx = k % NSTAGE;
        mbar_wait_or_flag(&ready[sidx], (k / NSTAGE) & 1, dead, p.status, DEV_TIMEOUT_STORE);
        tma_store_3d(&maps.out0, smem + sidx * SM::STAGE + SM::TILEX, d0, k * TC, b);
        tma_commit();
        if (k + NSTAGE < nchunks) {
          tma_wait_read<0>();
          issue(k + NSTAGE);
        }
      }
      tma_wait_all<0>();
    }
    return;
  }

  ConvTaps ct;
  load_taps(p.w, p.bias, d0 + vec * CV, p.D, ct);
  const int off0 = (lane_t * TS) * ROWB + vec * Pack<IO>::BYTES;

  for (int k = 0; k < nchunks; ++k) {
    const int stage = k % NSTAGE;
    uint8_t* tiles = smem + stage * SM::STAGE;
    const int t0 = k * TC;
    uint32_t fl[1];
    const bool masked = (p.tok != nullptr) || (t0 + TC > p.T);
    if (masked) load_flags_word(p.tok, b, p.T, t0 + lane_t * TS, fl);
    float2 hist_v[3][2];
    const float2 (*hist)[2] = nullptr;
    if (k == 0 && lane_t == 0 && p.state) {
      load_hist<IO>(p.state, b, d0 + vec * CV, p.D, hist_v);
      hist = hist_v;
    }
    mbar_wait_or_flag(&full[stage], (k / NSTAGE) & 1, dead, p.status, DEV_TIMEOUT_LOAD);
    float2 xc[TS][2];
    const bool flagged = masked && any_flag(fl);
    if (flagged) conv_front<IO, TS, CH, true>(tiles, off0, ct, fl, hist, xc);
    else conv_front<IO, TS, CH, false>(tiles, off0, ct, fl, hist, xc);
    uint8_t* to = tiles + SM::TILEX;
#pragma unroll
    for (int st = 0; st < TS; ++st) {
      if (flagged && ((fl[0] >> (8 * st)) & TOK_INACTIVE)) { xc[st][0] = f2(0.0f); xc[st][1] = f2(0.0f); }   // padding emits zero
      Pack<IO>::store2(to + off0 + st * ROWB, xc[st]);
    }
    fence_async_smem();
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(&ready[stage]);
  }
}

// The TS steps of one thread in the conv backward.  Two sliding four-row windows: ga = upstream gradient of
// tokens (step .. step+3), xa = input at times (step-3 .. step); each step loads one new row of each.
// `fb` holds the flag bytes of the TS + 3 tokens whose gradient is read; `dstate` (first lane of the first
// chunk only) receives the gradient of the carried history, whose rows only tokens 0 .. 2 reach.
template <typename IO, int TS, int CH, bool MASKED>
__device__ __forceinline__ void conv_bwd_steps(const uint8_t* tg, const uint8_t* tx, uint8_t* tdx, int off0,
                                               const ConvTaps& ct, const uint32_t (&fb)[TS + 3], const float2 (*hist)[2],
                                               IO* dstate, int D, int channels_left, float2 (&gw)[5][2]) {
  constexpr int ROWB = CH * sizeof(IO);
  auto grad_row = [&](int j, float2 (&v)[2]) {
    Pack<IO>::unpack2(Pack<IO>::load(tg + off0 + j * ROWB), v);
    if (MASKED && (fb[j] & TOK_INACTIVE)) { v[0] = f2(0.0f); v[1] = f2(0.0f); }
  };
  auto reach_of = [&](int j) { return MASKED ? 3 - static_cast<int>(fb[j] & TOK_CUT_MASK) : 3; };
  float2 ga[4][2], xa[4][2];
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    grad_row(j, ga[j]);
    Pack<IO>::unpack2(Pack<IO>::load(tx + off0 + j * ROWB), xa[j]);
    if (hist) { xa[j][0] = hist[j][0]; xa[j][1] = hist[j][1]; }
  }
  if (dstate) {
#pragma unroll
    for (int slot = 0; slot < 3; ++slot) {
      float2 acc[2] = {f2(0.0f), f2(0.0f)};
#pragma unroll
      for (int u = 0; u <= slot; ++u) {               // token u reads time slot-3 with lag u + 3 - slot
        const int lag = u + 3 - slot;
        const float m = reach_of(u) >= lag ? 1.0f : 0.0f;
#pragma unroll
        for (int cp = 0; cp < 2; ++cp) acc[cp] = fma2(mul2(ct.w[3 - lag][cp], f2(m)), ga[u][cp], acc[cp]);
      }
      const float v4[4] = {acc[0].x, acc[0].y, acc[1].x, acc[1].y};
#pragma unroll
      for (int ch = 0; ch < 4; ++ch)
        if (ch < channels_left) dstate[static_cast<size_t>(slot) * D + ch] = Pack<IO>::from_float(v4[ch]);
    }
  }
#pragma unroll
  for (int st = 0; st < TS; ++st) {
    grad_row(st + 3, ga[3]);
    Pack<IO>::unpack2(Pack<IO>::load(tx + off0 + (st + 3) * ROWB), xa[3]);   // input at the step's own time
    float2 dx[2];
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
      if (MASKED) {
        float2 a = mul2(ct.w[3][cp], ga[0][cp]);
        a = fma2(mul2(ct.w[2][cp], f2(reach_of(st + 1) >= 1 ? 1.0f : 0.0f)), ga[1][cp], a);
        a = fma2(mul2(ct.w[1][cp], f2(reach_of(st + 2) >= 2 ? 1.0f : 0.0f)), ga[2][cp], a);
        dx[cp] = fma2(mul2(ct.w[0][cp], f2(reach_of(st + 3) >= 3 ? 1.0f : 0.0f)), ga[3][cp], a);
      } else {
        float2 a = mul2(ct.w[3][cp], ga[0][cp]);
        a = fma2(ct.w[2][cp], ga[1][cp], a);
        a = fma2(ct.w[1][cp], ga[2][cp], a);
        dx[cp] = fma2(ct.w[0][cp], ga[3][cp], a);
      }
    }
    Pack<IO>::store2(tdx + off0 + st * ROWB, dx);
    // tap gradients of the step's own token (its flag decides how far back it reaches)
    const int reach = reach_of(st);
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
      const float2 g0 = ga[0][cp];
      gw[4][cp] = add2(gw[4][cp], g0);
      gw[3][cp] = fma2(g0, xa[3][cp], gw[3][cp]);
      if (MASKED) {
        gw[2][cp] = fma2(mul2(g0, f2(reach >= 1 ? 1.0f : 0.0f)), xa[2][cp], gw[2][cp]);
        gw[1][cp] = fma2(mul2(g0, f2(reach >= 2 ? 1.0f : 0.0f)), xa[1][cp], gw[1][cp]);
        gw[0][cp] = fma2(mul2(g0, f2(reach >= 3 ? 1.0f : 0.0f)), xa[0][cp], gw[0][cp]);
      } else {
        gw[2][cp] = fma2(g0, xa[2][cp], gw[2][cp]);
        gw[1][cp] = fma2(g0, xa[1][cp], gw[1][cp]);
        gw[0][cp] = fma2(g0, xa[0][cp], gw[0][cp]);
      }
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      ga[j][0] = ga[j + 1][0]; ga[j][1] = ga[j + 1][1];
      xa[j][0] = xa[j + 1][0]; xa[j][1] = xa[j + 1][1];
    }
  }
}

// Backward of the conv.  Per chunk: the upstream gradient rows t0 .. t0+TC+2 (three rows of look-ahead, zero
// past T), the input rows t0-3 .. t0+TC-1, and the result tile.
//   dx[t]     = sum_lag w[3-lag] g[t+lag] [token t+lag reaches back lag steps]
//   dw[3-lag] += g[t] x[t-lag] [token t reaches back lag steps],   db += g[t]
// with g zero on padding.  The tap gradients stay in registers over the whole sequence and are folded
// across the CTA's time-lanes in a fixed order at the end: one partial row [5, D] per batch row.
template <typename IO, int NSTAGE>
struct ConvBwdSmem {
  static constexpr int TS = 4, LANES = 16, CH = 64, TC = LANES * TS;
  static constexpr int TILE = TC * CH * sizeof(IO);
  static constexpr int HALO = 3 * CH * sizeof(IO);
  static constexpr int TILEX = TILE + HALO;
  static constexpr int OFF_X = TILEX, OFF_DX = 2 * TILEX;
  static constexpr int STAGE = 2 * TILEX + TILE;
  static constexpr int OFF_BAR = NSTAGE * STAGE;
  static constexpr int BYTES = OFF_BAR + 2 * NSTAGE * 8 + 16;
  static_assert(NSTAGE * STAGE >= LANES * 5 * CH * 4, "the final fold reuses the stage memory");
};

template <typename IO, int NSTAGE>
__global__ void __maxnreg__(96) conv_tma_bwd_kernel(const __grid_constant__ ConvMaps maps, const ConvTmaArgs p) {
  using SM = ConvBwdSmem<IO, NSTAGE>;
  constexpr int TS = SM::TS, CH = SM::CH, TC = SM::TC, NCV = CH / CV, NCOMP = SM::LANES * NCV, LANES = SM::LANES;
  constexpr int ROWB = CH * sizeof(IO);
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
  uint64_t* ready = full + NSTAGE;
  volatile int* dead = reinterpret_cast<volatile int*>(ready + NSTAGE);
  const int tid = threadIdx.x, lane_t = tid / NCV, vec = tid % NCV;
  const int b = blockIdx.y, d0 = blockIdx.x * CH;
  const int nchunks = (p.T + TC - 1) / TC;

  if (tid == 0) {
    *dead = 0;
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full[s], 1); mbar_init(&ready[s], NCOMP / 32); }
    mbar_fence_init();
  }
  __syncthreads();

  if (tid >= NCOMP) {
    if (tid == NCOMP) {
      prefetch_map(&maps.in0); prefetch_map(&maps.in1); prefetch_map(&maps.out0);
      auto issue = [&](int k) {
        const int sidx = k % NSTAGE;
        uint8_t* st = smem + sidx * SM::STAGE;
        mbar_expect_tx(&full[sidx], 2 * SM::TILEX);
        tma_load_3d(st, &maps.in0, d0, k * TC, b, &full[sidx]);                   // gradient, rows past T read as zero
        tma_load_3d(st + SM::OFF_X, &maps.in1, d0, k * TC - 3, b, &full[sidx]);   // input, rows before 0 read as zero
      };
      for (int k = 0; k < NSTAGE && k < nchunks; ++k) issue(k);
      for (int k = 0; k < nchunks; ++k) {
        const int sidx = k % NSTAGE;
        mbar_wait_or_flag(&ready[sidx], (k / NSTAGE) & 1, dead, p.status, DEV_TIMEOUT_STORE);
        tma_store_3d(&maps.out0, smem + sidx * SM::STAGE + SM::OFF_DX, d0, k * TC, b);
        tma_commit();
        if (k + NSTAGE < nchunks) {
          tma_wait_read<0>();
          issue(k + NSTAGE);
        }
      }
      tma_wait_all<0>();
    }
    bar_all(NCOMP + 32);   // the final fold below reuses stage memory: every bulk store has left it
    return;
  }

  ConvTaps ct;
  load_taps(p.w, nullptr, d0 + vec * CV, p.D, ct);
  float2 gw[5][2];
#pragma unroll
  for (int q = 0; q < 5; ++q) { gw[q][0] = f2(0.0f); gw[q][1] = f2(0.0f); }
  const int off0 = (lane_t * TS) * ROWB + vec * Pack<IO>::BYTES;

  for (int k = 0; k < nchunks; ++k) {
    const int stage = k % NSTAGE;
    uint8_t* tiles = smem + stage * SM::STAGE;
    const int t0 = k * TC;
    // flag bytes of the TS + 3 tokens whose gradient this thread reads (steps at or past T count as padding)
    uint32_t fb[TS + 3];
    const bool masked = (p.tok != nullptr) || (t0 + TC + 3 > p.T);
    {
      const int t_first = t0 + lane_t * TS;
      const uint8_t* fp = p.tok ? p.tok + static_cast<size_t>(b) * p.T + t_first : nullptr;
      if (masked && fp && t_first + 8 <= p.T && (reinterpret_cast<uintptr_t>(fp) & 3u) == 0) {
        const uint32_t w0 = *reinterpret_cast<const uint32_t*>(fp);       // two aligned words cover the seven tokens
        const uint32_t w1 = *reinterpret_cast<const uint32_t*>(fp + 4);
#pragma unroll
        for (int j = 0; j < TS + 3; ++j) fb[j] = ((j < 4 ? w0 : w1) >> (8 * (j & 3))) & 0xffu;
      } else {
#pragma unroll
        for (int j = 0; j < TS + 3; ++j) {
          fb[j] = 0u;
          if (masked) {
            const int t = t_first + j;
            fb[j] = t < p.T ? (p.tok ? p.tok[static_cast<size_t>(b) * p.T + t] : 0u) : TOK_INACTIVE;
          }
        }
      }
    }
    float2 hist_v[3][2];
    const bool use_hist = (k == 0 && lane_t == 0 && p.state != nullptr);
    if (use_hist) load_hist<IO>(p.state, b, d0 + vec * CV, p.D, hist_v);
    mbar_wait_or_flag(&full[stage], (k / NSTAGE) & 1, dead, p.status, DEV_TIMEOUT_LOAD);

    IO* dstate = nullptr;
    if (k == 0 && lane_t == 0 && p.d_state)
      dstate = static_cast<IO*>(p.d_state) + static_cast<size_t>(b) * 3 * p.D + d0 + vec * CV;
    const float2 (*hist)[2] = use_hist ? hist_v : nullptr;
    if (masked && any_flag(fb)) conv_bwd_steps<IO, TS, CH, true>(tiles, tiles + SM::OFF_X, tiles + SM::OFF_DX, off0, ct, fb, hist, dstate,
                                                 p.D, p.D - (d0 + vec * CV), gw);
    else conv_bwd_steps<IO, TS, CH, false>(tiles, tiles + SM::OFF_X, tiles + SM::OFF_DX, off0, ct, fb, hist, dstate,
                                           p.D, p.D - (d0 + vec * CV), gw);
    fence_async_smem();
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(&ready[stage]);
  }

  // Fold the time-lanes in index order; the stage memory is free once the producer has drained its stores.
  bar_all(NCOMP + 32);
  float* red = reinterpret_cast<float*>(smem);          // [LANES][5][CH]
#pragma unroll
  for (int q = 0; q < 5; ++q)
    *reinterpret_cast<float4*>(red + (lane_t * 5 + q) * CH + vec * CV) = make_float4(gw[q][0].x, gw[q][0].y, gw[q][1].x, gw[q][1].y);
  bar_compute(NCOMP);
  for (int idx = tid; idx < 5 * CH; idx += NCOMP) {
    const int q = idx / CH, cc = idx % CH;
    if (d0 + cc >= p.D) continue;
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < LANES; ++j) acc += red[(j * 5 + q) * CH + cc];
    p.part[(static_cast<size_t>(b) * 5 + q) * p.D + d0 + cc] = acc;
  }
}

// ======================================================================
// Self-test of the bounded wait: one CTA waits on an mbarrier that nothing ever completes, with a limit of
// `limit` SM cycles.  The wait must give up, set the device status word, and let every thread reach the
// barrier and the final store below -- the behaviour the pipelined kernels rely on when a copy never lands.
// ======================================================================
__global__ void __launch_bounds__(64) wait_selftest_kernel(int* status, int* finished, long long limit) {
  __shared__ uint64_t bar;
  __shared__ int dead_flag;
  volatile int* dead = &dead_flag;
  if (threadIdx.x == 0) {
    dead_flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  mbar_wait_or_flag(&bar, 0, dead, status, DEV_TIMEOUT_SELFTEST, limit);
  __syncthreads();                       // every thread gets here: barriers stay matched after a timeout
  if (threadIdx.x == 0 && finished) *finished = 1;
}
cudaError_t launch_wait_selftest(int* status, int* finished, long long limit_cycles, cudaStream_t s) {
  wait_selftest_kernel<<<1, 64, 0, s>>>(status, finished, limit_cycles);
  return cudaGetLastError();
}

// ======================================================================
// Launchers
// ======================================================================

// CTA shapes.  CH channels x (LANES * TS) time-steps per chunk, LANES * CH / 4 compute threads.
//   64 x 64  : the default; grids large enough to put two or more forward CTAs on every SM.
//   32 x 128 : half-width forward tiles double the number of CTAs for small grids, so that two CTAs
//              (two independent barrier domains) still share an SM and overlap their phases.
struct Shape64x16x4 { static constexpr int CH = 64, LANES = 16, TS = 4; };
struct Shape32x32x4 { static constexpr int CH = 32, LANES = 32, TS = 4; };

// Kernel variants.  Forward: 0 = 64 x 64 tiles, 2 = 32 x 128 tiles.  Backward: 0 = 64 x 64 tiles with a
// producer warp, 3 = the same tiles with the bulk copies issued by a compute thread (SELF_ISSUE).  The numbers
// are what RGLRU_FWD_VARIANT / RGLRU_BWD_VARIANT accept (they force one variant for a whole process; the
// test-suite uses them to run every variant over the parity cases); anything else means "choose by shape".
static bool fwd_variant_exists(int v) { return v == 0 || v == 2; }
static bool bwd_variant_exists(int v) { return v == 0 || v == 3; }

// Whether a forward call takes the paired-row tile layout: the 32-channel shape on bf16 tensors without token
// flags over a whole number of 128-step chunks.  The API encodes 5-D tensor maps exactly when this says so.
bool scan_fwd_paired(int variant, bool bf16, const void* tok, int T) {
  return variant == 2 && bf16 && tok == nullptr && T % 128 == 0;
}
int scan_fwd_box_rows(int v) { return v == 2 ? 128 : 64; }
int scan_fwd_box_cols(int v) { return v == 2 ? 32 : 64; }
int scan_bwd_box_rows(int) { return 64; }
int scan_bwd_box_cols(int) { return 64; }

static int env_override(const char* name) {
  const char* v = getenv(name);
  return (v && v[0] >= '0' && v[0] <= '9' && v[1] == 0) ? (v[0] - '0') : -1;
}

// Measured on B200 (bf16, T = 2048, D = 1024): half-width forward tiles win while 64-channel tiles cannot fill
// the 148 SMs (B = 8, 128 tiles: 31 us against 50 us) and lose once they can (B = 16: 58 us against 52 us); for
// fp32 the 64-channel shape is faster throughout.  The backward runs one CTA per SM either way; without the
// producer warp it is 1 to 2 % faster for bf16 tensors (eight warps leave every thread its registers).
int scan_fwd_variant(int B, int T, int D, bool bf16) {
  static const int forced = env_override("RGLRU_FWD_VARIANT");
  if (fwd_variant_exists(forced)) return forced;
  const long long tiles = static_cast<long long>(B) * ((D + 63) / 64);
  return (bf16 && tiles <= 160 && T >= 256) ? 2 : 0;
}
int scan_bwd_variant(int B, int T, int D, bool bf16) {
  static const int forced = env_override("RGLRU_BWD_VARIANT");
  if (bwd_variant_exists(forced)) return forced;
  (void)B; (void)T; (void)D;
  return bf16 ? 3 : 0;
}

// Launch with programmatic stream serialization, so that this kernel's launch and prologue may overlap
// the tail of the kernel before it on the stream (the kernels call pdl_wait before touching memory).
template <typename Kern, typename Maps, typename Args>
static cudaError_t launch_pdl(Kern kern, dim3 grid, int threads, int bytes, cudaStream_t s, const Maps& maps, const Args& a) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, maps, a);
}

// Shared-memory attributes of one kernel: the largest carveout, so that occupancy is set by the kernel's own
// footprint and not by the default L1 / shared split, and the dynamic size.  They are per device and do not
// change, so each call site (one per kernel instantiation, told apart by TAG) sets them once per device.
template <typename TAG, typename Kern>
static cudaError_t set_smem(Kern kern, int bytes) {
  static std::atomic<unsigned long long> done{0ull};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long bit = (dev >= 0 && dev < 64) ? (1ull << dev) : 0ull;
  if (bit && (done.load(std::memory_order_acquire) & bit)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && bit) done.fetch_or(bit, std::memory_order_release);
  return e;
}
template <typename... Ts> struct KernelTag {};
template <int... Vs> struct IntTag {};

template <typename IO, typename V, int STAGES, bool USE_TMA, bool CONV = false, bool MERGE = false, bool GROUPED = false,
          bool PLAIN = false, bool CARRY = false, bool PAIRED = false>
static cudaError_t launch_fwd_t(const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  constexpr int ST = USE_TMA ? STAGES : 1;
  constexpr bool CAPPED = USE_TMA && !CONV && (MERGE || GROUPED);
  void (*kern)(FwdMaps, ScanFwdArgs);
  if constexpr (CAPPED) kern = rglru_fwd_kernel_capped<IO, V::TS, V::LANES, V::CH, ST, USE_TMA, CONV, MERGE, GROUPED>;
  else kern = rglru_fwd_kernel<IO, V::TS, V::LANES, V::CH, ST, USE_TMA, CONV, MERGE, GROUPED, PLAIN, CARRY, PAIRED>;
  constexpr int bytes = FwdSmem<IO, V::TS, V::LANES, V::CH, ST, CONV, MERGE>::BYTES;
  static_assert(bytes <= 232448, "shared memory of one CTA");
  cudaError_t e = set_smem<KernelTag<FwdMaps, IO, V, IntTag<ST, USE_TMA, CONV, MERGE, GROUPED, PLAIN, CARRY, PAIRED>>>(kern, bytes);
  if (e != cudaSuccess) return e;
  dim3 grid((a.D + V::CH - 1) / V::CH, a.B);
  return launch_pdl(kern, grid, V::LANES * (V::CH / CV) + (USE_TMA ? 32 : 0), bytes, s, maps, a);
}

template <typename IO>
static cudaError_t launch_fwd_io(bool use_tma, int variant, const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  constexpr bool H = sizeof(IO) == 2;
  if (a.y == nullptr)   // carry-only pass: one shape, masked arithmetic
    return use_tma ? launch_fwd_t<IO, Shape64x16x4, H ? 4 : 3, true, false, false, false, false, true>(maps, a, s)
                   : launch_fwd_t<IO, Shape64x16x4, 1, false, false, false, false, false, true>(maps, a, s);
  if (!use_tma) return launch_fwd_t<IO, Shape64x16x4, 1, false>(maps, a, s);
  const bool plain = a.tok == nullptr && a.T % 128 == 0;   // no step of any chunk is masked
  if (plain && variant == 0) return launch_fwd_t<IO, Shape64x16x4, H ? 4 : 3, true, false, false, false, true>(maps, a, s);
  if (plain && variant == 2) {
    if constexpr (H) {   // 64-byte rows: the paired-row layout when the caller could encode its 5-D maps
      if (a.paired) return launch_fwd_t<IO, Shape32x32x4, 4, true, false, false, false, true, false, true>(maps, a, s);
    }
    return launch_fwd_t<IO, Shape32x32x4, H ? 4 : 3, true, false, false, false, true>(maps, a, s);
  }
  if (variant == 2) return launch_fwd_t<IO, Shape32x32x4, H ? 4 : 3, true>(maps, a, s);
  return launch_fwd_t<IO, Shape64x16x4, H ? 4 : 3, true>(maps, a, s);
}

cudaError_t launch_scan_fwd(bool bf16, bool use_tma, int variant, const FwdMaps& maps, const ScanFwdArgs& a,
                            cudaStream_t s) {
  return bf16 ? launch_fwd_io<__nv_bfloat16>(use_tma, variant, maps, a, s) : launch_fwd_io<float>(use_tma, variant, maps, a, s);
}

template <typename IO, typename V, int STAGES, bool USE_TMA, bool CONV = false, bool MERGE = false, bool GROUPED = false,
          bool SELF_ISSUE = false, bool PLAIN = false, bool CARRY = false>
static cudaError_t launch_bwd_t(const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  constexpr int ST = USE_TMA ? STAGES : 1;
  auto kern = rglru_bwd_kernel<IO, V::TS, V::LANES, V::CH, ST, USE_TMA, CONV, MERGE, GROUPED, SELF_ISSUE, PLAIN, CARRY>;
  constexpr int bytes = BwdSmem<IO, V::TS, V::LANES, V::CH, ST, CONV, MERGE>::BYTES;
  static_assert(bytes <= 232448, "shared memory of one CTA");
  cudaError_t e = set_smem<KernelTag<BwdMaps, IO, V, IntTag<ST, USE_TMA, CONV, MERGE, GROUPED, SELF_ISSUE, PLAIN, CARRY>>>(kern, bytes);
  if (e != cudaSuccess) return e;
  dim3 grid((a.D + V::CH - 1) / V::CH, a.B);
  e = launch_pdl(kern, grid, V::LANES * (V::CH / CV) + ((USE_TMA && !SELF_ISSUE) ? 32 : 0), bytes, s, maps, a);
  if (e != cudaSuccess || a.ticket || !a.dlambda) return e;
  rglru_dlambda_kernel<<<(a.D + 255) / 256, 256, 0, s>>>(a.dlam_part, a.lambda, a.dlambda, a.B, a.D, a.c);
  if (GROUPED && a.dgate && a.dgate_part)
    rglru_colsum_kernel<<<(2 * a.D + 255) / 256, 256, 0, s>>>(a.dgate_part, a.dgate, a.B, 2 * a.D);
  return cudaGetLastError();
}

template <typename IO>
static cudaError_t launch_bwd_io(bool use_tma, int variant, const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  constexpr bool H = sizeof(IO) == 2;
  if (a.dx == nullptr)   // carry-only pass: producer-warp shape, masked arithmetic
    return use_tma ? launch_bwd_t<IO, Shape64x16x4, H ? 4 : 3, true, false, false, false, false, false, true>(maps, a, s)
                   : launch_bwd_t<IO, Shape64x16x4, 1, false, false, false, false, false, false, true>(maps, a, s);
  if (!use_tma) return launch_bwd_t<IO, Shape64x16x4, 1, false>(maps, a, s);
  const bool plain = a.tok == nullptr && a.T % 64 == 0;   // no step of any chunk is masked
  if (variant == 3) {   // bulk copies issued by a compute thread: loads run NSTAGE - 2 chunks ahead, so one more stage
    if (plain) return launch_bwd_t<IO, Shape64x16x4, H ? 5 : 3, true, false, false, false, true, true>(maps, a, s);
    return launch_bwd_t<IO, Shape64x16x4, H ? 5 : 3, true, false, false, false, true>(maps, a, s);
  }
  if (plain) return launch_bwd_t<IO, Shape64x16x4, H ? 4 : 3, true, false, false, false, false, true>(maps, a, s);
  return launch_bwd_t<IO, Shape64x16x4, H ? 4 : 3, true>(maps, a, s);
}

cudaError_t launch_scan_bwd(bool bf16, bool use_tma, int variant, const BwdMaps& maps, const ScanBwdArgs& a,
                            cudaStream_t s) {
  return bf16 ? launch_bwd_io<__nv_bfloat16>(use_tma, variant, maps, a, s) : launch_bwd_io<float>(use_tma, variant, maps, a, s);
}

// Conv folded into the load stage: one shape (64 channels x 64 steps); the x map's box has three more rows.
cudaError_t launch_conv_scan_fwd(bool bf16, bool use_tma, const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  if (bf16)
    return use_tma ? launch_fwd_t<__nv_bfloat16, Shape64x16x4, 4, true, true>(maps, a, s)
                   : launch_fwd_t<__nv_bfloat16, Shape64x16x4, 1, false, true>(maps, a, s);
  return use_tma ? launch_fwd_t<float, Shape64x16x4, 3, true, true>(maps, a, s)
                 : launch_fwd_t<float, Shape64x16x4, 1, false, true>(maps, a, s);
}
cudaError_t launch_conv_scan_bwd(bool bf16, bool use_tma, const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  if (bf16)
    return use_tma ? launch_bwd_t<__nv_bfloat16, Shape64x16x4, 4, true, true, false, false, true>(maps, a, s)
                   : launch_bwd_t<__nv_bfloat16, Shape64x16x4, 1, false, true>(maps, a, s);
  return use_tma ? launch_bwd_t<float, Shape64x16x4, 3, true, true>(maps, a, s)
                 : launch_bwd_t<float, Shape64x16x4, 1, false, true>(maps, a, s);
}

// Branch merge folded into the store stage (forward) and the load stage (backward), with or without the
// conv fold: one shape (64 channels x 64 steps).  One more tile per stage, so fp32 backward keeps two stages.
template <typename IO, bool CONV>
static cudaError_t launch_merge_fwd_t(bool use_tma, const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  constexpr bool H = sizeof(IO) == 2;
  return use_tma ? launch_fwd_t<IO, Shape64x16x4, H ? (CONV ? 4 : 3) : 3, true, CONV, true>(maps, a, s)
                 : launch_fwd_t<IO, Shape64x16x4, 1, false, CONV, true>(maps, a, s);
}
template <typename IO, bool CONV>
static cudaError_t launch_merge_bwd_t(bool use_tma, const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  constexpr bool H = sizeof(IO) == 2;
  if (!use_tma) return launch_bwd_t<IO, Shape64x16x4, 1, false, CONV, true>(maps, a, s);
  // bf16: four stages without a producer warp (eight warps leave these variants the registers they need);
  // fp32 fits two stages only, which the producer warp needs to keep a load ahead
  if constexpr (H) return launch_bwd_t<IO, Shape64x16x4, 4, true, CONV, true, false, true>(maps, a, s);
  else return launch_bwd_t<IO, Shape64x16x4, 2, true, CONV, true>(maps, a, s);
}
cudaError_t launch_merge_fwd(bool bf16, bool use_tma, bool conv, const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  if (bf16) return conv ? launch_merge_fwd_t<__nv_bfloat16, true>(use_tma, maps, a, s)
                        : launch_merge_fwd_t<__nv_bfloat16, false>(use_tma, maps, a, s);
  return conv ? launch_merge_fwd_t<float, true>(use_tma, maps, a, s) : launch_merge_fwd_t<float, false>(use_tma, maps, a, s);
}
cudaError_t launch_merge_bwd(bool bf16, bool use_tma, bool conv, const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  if (bf16) return conv ? launch_merge_bwd_t<__nv_bfloat16, true>(use_tma, maps, a, s)
                        : launch_merge_bwd_t<__nv_bfloat16, false>(use_tma, maps, a, s);
  return conv ? launch_merge_bwd_t<float, true>(use_tma, maps, a, s) : launch_merge_bwd_t<float, false>(use_tma, maps, a, s);
}

// Grouped gate layout (one [B, T, 2 D] gate tensor, biases added in the kernel), with or without the
// branch merge; TMA staging only, one shape (64 channels x 64 steps).
template <typename IO, bool MERGE>
static cudaError_t launch_grouped_fwd_t(const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  constexpr bool H = sizeof(IO) == 2;
  return launch_fwd_t<IO, Shape64x16x4, H ? (MERGE ? 3 : 4) : 3, true, false, MERGE, true>(maps, a, s);
}
template <typename IO, bool MERGE>
static cudaError_t launch_grouped_bwd_t(const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  constexpr bool H = sizeof(IO) == 2;
  // Measured on B200 at B = 16, T = 2048, D = 1024 bf16: with the branch merge (five loads and four stores per
  // chunk) the producer warp wins although the kernel then spills a little at its 168-register limit (162 us
  // against 169 us with the copies issued by a compute thread); without the merge the compute-thread variant does.
  if constexpr (H && !MERGE) return launch_bwd_t<IO, Shape64x16x4, 5, true, false, false, true, true>(maps, a, s);
  else return launch_bwd_t<IO, Shape64x16x4, H ? 4 : (MERGE ? 2 : 3), true, false, MERGE, true>(maps, a, s);
}
cudaError_t launch_grouped_fwd(bool bf16, bool merge, const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  if (bf16) return merge ? launch_grouped_fwd_t<__nv_bfloat16, true>(maps, a, s) : launch_grouped_fwd_t<__nv_bfloat16, false>(maps, a, s);
  return merge ? launch_grouped_fwd_t<float, true>(maps, a, s) : launch_grouped_fwd_t<float, false>(maps, a, s);
}
cudaError_t launch_grouped_bwd(bool bf16, bool merge, const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  if (bf16) return merge ? launch_grouped_bwd_t<__nv_bfloat16, true>(maps, a, s) : launch_grouped_bwd_t<__nv_bfloat16, false>(maps, a, s);
  return merge ? launch_grouped_bwd_t<float, true>(maps, a, s) : launch_grouped_bwd_t<float, false>(maps, a, s);
}
int grouped_box_cols() { return Shape64x16x4::CH; }

int raw_box_rows() { return RAW_TC; }
int raw_box_cols() { return CH; }

template <int NSTAGE, bool USE_TMA>
static cudaError_t launch_raw_fwd_t(const RawFwdMaps& maps, const RawScanArgs& a, cudaStream_t s) {
  auto kern = rawscan_fwd_kernel<NSTAGE, USE_TMA>;
  constexpr int bytes = RawSmem<NSTAGE>::BYTES;
  cudaError_t e = set_smem<KernelTag<RawFwdMaps, IntTag<NSTAGE, USE_TMA>>>(kern, bytes);
  if (e != cudaSuccess) return e;
  dim3 grid((a.D + CH - 1) / CH, a.B);
  kern<<<grid, RAW_NT, bytes, s>>>(maps, a);
  return cudaGetLastError();
}
cudaError_t launch_raw_fwd(bool use_tma, const RawFwdMaps& maps, const RawScanArgs& a, cudaStream_t s) {
  return use_tma ? launch_raw_fwd_t<3, true>(maps, a, s) : launch_raw_fwd_t<1, false>(maps, a, s);
}
template <int NSTAGE, bool USE_TMA>
static cudaError_t launch_raw_bwd_t(const RawBwdMaps& maps, const RawScanArgs& a, cudaStream_t s) {
  auto kern = rawscan_bwd_kernel<NSTAGE, USE_TMA>;
  constexpr int bytes = RawSmem<NSTAGE>::BYTES;
  cudaError_t e = set_smem<KernelTag<RawBwdMaps, IntTag<NSTAGE, USE_TMA>>>(kern, bytes);
  if (e != cudaSuccess) return e;
  dim3 grid((a.D + CH - 1) / CH, a.B);
  kern<<<grid, RAW_NT, bytes, s>>>(maps, a);
  return cudaGetLastError();
}
cudaError_t launch_raw_bwd(bool use_tma, const RawBwdMaps& maps, const RawScanArgs& a, cudaStream_t s) {
  return use_tma ? launch_raw_bwd_t<3, true>(maps, a, s) : launch_raw_bwd_t<1, false>(maps, a, s);
}

int conv_tma_box_rows() { return 64 + 3; }
int conv_tma_box_cols() { return 64; }

template <typename IO>
static cudaError_t conv_tma_fwd_t(const ConvMaps& maps, const ConvTmaArgs& a, cudaStream_t s) {
  constexpr int ST = sizeof(IO) == 2 ? 4 : 3;
  auto kern = conv_tma_fwd_kernel<IO, ST>;
  constexpr int bytes = ConvFwdSmem<IO, ST>::BYTES;
  cudaError_t e = set_smem<KernelTag<ConvFwdSmem<IO, ST>>>(kern, bytes);
  if (e != cudaSuccess) return e;
  kern<<<dim3((a.D + 63) / 64, a.B), 288, bytes, s>>>(maps, a);
  return cudaGetLastError();
}
cudaError_t launch_conv_tma_fwd(bool bf16, const ConvMaps& maps, const ConvTmaArgs& a, cudaStream_t s) {
  return bf16 ? conv_tma_fwd_t<__nv_bfloat16>(maps, a, s) : conv_tma_fwd_t<float>(maps, a, s);
}
template <typename IO>
static cudaError_t conv_tma_bwd_t(const ConvMaps& maps, const ConvTmaArgs& a, cudaStream_t s) {
  constexpr int ST = sizeof(IO) == 2 ? 4 : 2;   // about 100 KB either way: two CTAs per SM
  auto kern = conv_tma_bwd_kernel<IO, ST>;
  constexpr int bytes = ConvBwdSmem<IO, ST>::BYTES;
  static_assert(bytes <= 232448, "shared memory of one CTA");
  cudaError_t e = set_smem<KernelTag<ConvBwdSmem<IO, ST>>>(kern, bytes);
  if (e != cudaSuccess) return e;
  kern<<<dim3((a.D + 63) / 64, a.B), 288, bytes, s>>>(maps, a);
  return cudaGetLastError();
}
cudaError_t launch_conv_tma_bwd(bool bf16, const ConvMaps& maps, const ConvTmaArgs& a, cudaStream_t s) {
  return bf16 ? conv_tma_bwd_t<__nv_bfloat16>(maps, a, s) : conv_tma_bwd_t<float>(maps, a, s);
}

}  // namespace rglru
