// RG-LRU forward and backward kernels for sm_100a.
//
// Work decomposition.  A CTA owns CH = 64 adjacent channels of one batch row and
// walks the whole sequence in chunks of LANES*TS time-steps.  Inside a chunk the
// time axis is split over LANES = 16 time-lanes, each thread scanning TS steps of
// CV = 4 channels in registers (level one), after which one thread per channel
// chains the 16 lane aggregates and the carry from the previous chunk (level two)
// and every lane applies its incoming state.  Chunks are staged through shared
// memory by TMA (cp.async.bulk.tensor, 3-D tiles [1, rows, 64 channels]) in a
// multi-stage mbarrier pipeline; results are written back into the stage in
// place and leave through TMA stores.  A bounds-checked plain-load staging path
// with the same arithmetic covers shapes TMA cannot address (D*elem % 16 != 0).
//
// The gate epilogue follows griffin/griffin.py:237-258 of the reference, the
// scan :280-286, the backward is the closed form of autograd over those lines
// with the capped sqrt slope of :59-65.  All arithmetic is fp32.

#include "rglru_device.cuh"
#include "rglru_internal.h"

namespace rglru {

struct ElemFlags {
  bool reset;
  bool inactive;
};

template <bool MASKED>
__device__ __forceinline__ ElemFlags elem_flags(uint32_t packed, int st) {
  ElemFlags f{false, false};
  if (MASKED) {
    const uint32_t byte = (packed >> (8 * (st & 3))) & 0xffu;
    f.reset = (byte & TOK_RESET) != 0;
    f.inactive = (byte & TOK_INACTIVE) != 0;
  }
  return f;
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

// Plain-load staging of one [rows, CH] tile (zero-filled outside the tensor).
template <typename IO>
__device__ __forceinline__ void tile_load_plain(uint8_t* tile, const void* src, int b, int t0, int d0, int rows, int T, int D) {
  const IO* g = static_cast<const IO*>(src);
  IO* s = reinterpret_cast<IO*>(tile);
  for (int idx = threadIdx.x; idx < rows * CH; idx += NT) {
    const int row = idx / CH, col = idx % CH;
    const int t = t0 + row, d = d0 + col;
    IO v = Pack<IO>::from_float(0.0f);
    if (t >= 0 && t < T && d < D) v = g[(static_cast<size_t>(b) * T + t) * D + d];
    s[idx] = v;
  }
}
template <typename IO>
__device__ __forceinline__ void tile_store_plain(const uint8_t* tile, void* dst, int b, int t0, int d0, int rows, int T, int D) {
  IO* g = static_cast<IO*>(dst);
  const IO* s = reinterpret_cast<const IO*>(tile);
  for (int idx = threadIdx.x; idx < rows * CH; idx += NT) {
    const int row = idx / CH, col = idx % CH;
    const int t = t0 + row, d = d0 + col;
    if (t < T && d < D) g[(static_cast<size_t>(b) * T + t) * D + d] = s[idx];
  }
}

// Per-channel constants: K = c * logsigmoid(Lambda), 0 for channels past D.
__device__ __forceinline__ float decay_rate(const float* lambda, int d, int D, float c) {
  if (d >= D) return 0.0f;
  const float lam = lambda[d];
  // logsigmoid(L) = -softplus(-L), evaluated without cancellation on either side.
  const float ls = lam >= 0.0f ? -log1pf(expf(-lam)) : lam - log1pf(expf(lam));
  return c * ls;
}

// ======================================================================
// Forward
// ======================================================================

template <typename IO, int TS, bool MASKED, bool POLY>
__device__ __forceinline__ void fwd_local(const uint8_t* tx, const uint8_t* tr, const uint8_t* ti, int off0,
                                          const float (&K)[CV], const uint32_t (&fl)[(TS + 3) / 4],
                                          float (&P)[TS][CV], float (&S)[TS][CV]) {
  constexpr int ROWB = CH * sizeof(IO);
  float p[CV], s[CV];
#pragma unroll
  for (int ch = 0; ch < CV; ++ch) { p[ch] = 1.0f; s[ch] = 0.0f; }
#pragma unroll
  for (int st = 0; st < TS; ++st) {
    const int off = off0 + st * ROWB;
    float xv[CV], rv[CV], iv[CV];
    Pack<IO>::unpack(Pack<IO>::load(tx + off), xv);
    Pack<IO>::unpack(Pack<IO>::load(tr + off), rv);
    Pack<IO>::unpack(Pack<IO>::load(ti + off), iv);
    const ElemFlags f = elem_flags<MASKED>(fl[st >> 2], st);
#pragma unroll
    for (int ch = 0; ch < CV; ++ch) {
      float r, i;
      sigmoid_pair(rv[ch], iv[ch], r, i);
      const float em = expm1_nonpos<POLY>(r * K[ch]);
      float a = 1.0f + em;
      const float gsq = fmaxf(-em * (2.0f + em), 0.0f);
      float b = sqrt_approx(gsq) * i * xv[ch];
      if (MASKED) {
        if (f.reset) { a = 0.0f; b = i * xv[ch]; }
        if (f.inactive) { a = 1.0f; b = 0.0f; }
      }
      p[ch] *= a;
      s[ch] = fmaf(a, s[ch], b);
      P[st][ch] = p[ch];
      S[st][ch] = s[ch];
    }
  }
}

template <typename IO, int TS, int NSTAGE>
struct FwdSmem {
  static constexpr int TC = LANES * TS;
  static constexpr int TILE = TC * CH * sizeof(IO);
  static constexpr int STAGE = 3 * TILE;
  static constexpr int OFF_AGG = NSTAGE * STAGE;
  static constexpr int OFF_EIN = OFF_AGG + LANES * CH * 8;
  static constexpr int OFF_BAR = OFF_EIN + LANES * CH * 4;
  static constexpr int BYTES = OFF_BAR + NSTAGE * 8 + 16;
};

template <typename IO, int TS, int NSTAGE, bool USE_TMA>
__global__ void __launch_bounds__(NT) rglru_fwd_kernel(const __grid_constant__ FwdMaps maps, const ScanFwdArgs p) {
  using SM = FwdSmem<IO, TS, NSTAGE>;
  constexpr int TC = SM::TC;
  constexpr int ROWB = CH * sizeof(IO);
  extern __shared__ __align__(128) uint8_t smem[];
  float2* agg = reinterpret_cast<float2*>(smem + SM::OFF_AGG);
  float* ein = reinterpret_cast<float*>(smem + SM::OFF_EIN);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);

  const int tid = threadIdx.x;
  const int lane_t = tid / NCV;
  const int vec = tid % NCV;
  const int b = blockIdx.y;
  const int d0 = blockIdx.x * CH;
  const int nchunks = (p.T + TC - 1) / TC;
  const int nsave = (p.T + SAVE_EVERY - 1) / SAVE_EVERY;

  float K[CV];
  bool poly_ok = true;
#pragma unroll
  for (int ch = 0; ch < CV; ++ch) {
    K[ch] = decay_rate(p.lambda, d0 + vec * CV + ch, p.D, p.c);
    poly_ok = poly_ok && (K[ch] >= POLY_RANGE);
  }
  const bool poly = __syncthreads_and(poly_ok);

  if (USE_TMA) {
    if (tid == 0) {
      prefetch_map(&maps.x); prefetch_map(&maps.ur); prefetch_map(&maps.ui); prefetch_map(&maps.y);
      for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[s], 1);
      mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {
      for (int k = 0; k < NSTAGE && k < nchunks; ++k) {
        uint8_t* st = smem + k * SM::STAGE;
        mbar_expect_tx(&bars[k], SM::STAGE);
        tma_load_3d(st, &maps.x, d0, k * TC, b, &bars[k]);
        tma_load_3d(st + SM::TILE, &maps.ur, d0, k * TC, b, &bars[k]);
        tma_load_3d(st + 2 * SM::TILE, &maps.ui, d0, k * TC, b, &bars[k]);
      }
    }
  }

  // Level-two chain state: thread `tid` < CH carries channel d0 + tid across chunks.
  float carry = 0.0f;
  const int dch = d0 + tid;
  if (tid < CH && dch < p.D && p.h0) carry = p.h0[static_cast<size_t>(b) * p.D + dch];

  const int off0 = (lane_t * TS) * ROWB + vec * Pack<IO>::BYTES;
  bool alive = true;

  for (int k = 0; k < nchunks; ++k) {
    const int stage = USE_TMA ? (k % NSTAGE) : 0;
    uint8_t* tiles = smem + stage * SM::STAGE;
    const int t0 = k * TC;
    uint32_t fl[(TS + 3) / 4];
    const bool masked = (p.tok != nullptr) || (t0 + TC > p.T);
    if (masked) load_flags<TS>(p.tok, b, p.T, t0 + lane_t * TS, fl);

    if (USE_TMA) {
      alive = mbar_wait_bounded(&bars[stage], (k / NSTAGE) & 1);
    } else {
      tile_load_plain<IO>(tiles, p.x, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<IO>(tiles + SM::TILE, p.ur, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<IO>(tiles + 2 * SM::TILE, p.ui, b, t0, d0, TC, p.T, p.D);
      __syncthreads();
    }

    float P[TS][CV], S[TS][CV];
    const uint8_t* tx = tiles;
    const uint8_t* tr = tiles + SM::TILE;
    const uint8_t* ti = tiles + 2 * SM::TILE;
    if (masked) {
      if (poly) fwd_local<IO, TS, true, true>(tx, tr, ti, off0, K, fl, P, S);
      else fwd_local<IO, TS, true, false>(tx, tr, ti, off0, K, fl, P, S);
    } else {
      if (poly) fwd_local<IO, TS, false, true>(tx, tr, ti, off0, K, fl, P, S);
      else fwd_local<IO, TS, false, false>(tx, tr, ti, off0, K, fl, P, S);
    }
    {
      float4* dst = reinterpret_cast<float4*>(agg + lane_t * CH + vec * CV);
      dst[0] = make_float4(P[TS - 1][0], S[TS - 1][0], P[TS - 1][1], S[TS - 1][1]);
      dst[1] = make_float4(P[TS - 1][2], S[TS - 1][2], P[TS - 1][3], S[TS - 1][3]);
    }
    alive = __syncthreads_and(alive);
    if (!alive) break;  // a load never arrived: leave without touching the stage

    if (tid < CH) {
      float2 ag[LANES];
#pragma unroll
      for (int j = 0; j < LANES; ++j) ag[j] = agg[j * CH + tid];
      float e = carry;
#pragma unroll
      for (int j = 0; j < LANES; ++j) {
        if (((j * TS) % SAVE_EVERY) == 0) {
          const int t = t0 + j * TS;
          if (p.states && t < p.T && dch < p.D)
            p.states[(static_cast<size_t>(b) * nsave + t / SAVE_EVERY) * p.D + dch] = e;
        }
        ein[j * CH + tid] = e;
        e = fmaf(ag[j].x, e, ag[j].y);
      }
      carry = e;
    }
    __syncthreads();

    {
      const float4 e4 = *reinterpret_cast<const float4*>(ein + lane_t * CH + vec * CV);
      const float e[CV] = {e4.x, e4.y, e4.z, e4.w};
      uint8_t* ty = tiles;  // y overwrites the x tile in place
#pragma unroll
      for (int st = 0; st < TS; ++st) {
        float yv[CV];
#pragma unroll
        for (int ch = 0; ch < CV; ++ch) yv[ch] = fmaf(P[st][ch], e[ch], S[st][ch]);
        Pack<IO>::store(ty + off0 + st * ROWB, yv);
      }
    }
    if (USE_TMA) {
      fence_async_smem();
      __syncthreads();
      if (tid == 0) {
        tma_store_3d(&maps.y, tiles, d0, t0, b);
        tma_commit();
        // Refill the stage of the previous chunk once its store has drained from shared memory.
        const int kp = k - 1;
        if (kp >= 0 && kp + NSTAGE < nchunks) {
          tma_wait_read<1>();
          const int sp = kp % NSTAGE;
          uint8_t* st = smem + sp * SM::STAGE;
          const int kn = kp + NSTAGE;
          mbar_expect_tx(&bars[sp], SM::STAGE);
          tma_load_3d(st, &maps.x, d0, kn * TC, b, &bars[sp]);
          tma_load_3d(st + SM::TILE, &maps.ur, d0, kn * TC, b, &bars[sp]);
          tma_load_3d(st + 2 * SM::TILE, &maps.ui, d0, kn * TC, b, &bars[sp]);
        }
      }
    } else {
      __syncthreads();
      tile_store_plain<IO>(tiles, p.y, b, t0, d0, TC, p.T, p.D);
      __syncthreads();
    }
  }

  if (USE_TMA && tid == 0) {
    tma_wait_all<0>();
    if (!alive) atomicExch(p.status, DEV_TIMEOUT_LOAD);
  }
  if (alive && tid < CH && dch < p.D && p.h_last) p.h_last[static_cast<size_t>(b) * p.D + dch] = carry;
}

// ======================================================================
// Backward
// ======================================================================

template <typename IO, int TS>
struct BwdRegs {
  float am[TS][CV];  // decay after masking
  float hb[TS][CV];  // drive b, later the state entering the step
  float ar[TS][CV];  // unmasked decay, zeroed where the decay receives no gradient
  float c1[TS][CV];  // d x      = g * c1
  float c2[TS][CV];  // d u_i    = g * c2
  float c3[TS][CV];  // d log a  = g * (h_prev * ar - c3)
  float rr[TS][CV];  // recurrence gate r
  typename Pack<IO>::Raw dy[TS];
};

template <typename IO, int TS, bool MASKED, bool POLY>
__device__ __forceinline__ void bwd_local(const uint8_t* tdy, const uint8_t* tx, const uint8_t* tr, const uint8_t* ti,
                                          int off0, const float (&K)[CV], const uint32_t (&fl)[(TS + 3) / 4],
                                          BwdRegs<IO, TS>& R, float (&aggF)[2][CV], float (&aggR)[2][CV]) {
  constexpr int ROWB = CH * sizeof(IO);
  float p[CV], s[CV];
#pragma unroll
  for (int ch = 0; ch < CV; ++ch) { p[ch] = 1.0f; s[ch] = 0.0f; }
#pragma unroll
  for (int st = 0; st < TS; ++st) {
    const int off = off0 + st * ROWB;
    float xv[CV], rv[CV], iv[CV];
    Pack<IO>::unpack(Pack<IO>::load(tx + off), xv);
    Pack<IO>::unpack(Pack<IO>::load(tr + off), rv);
    Pack<IO>::unpack(Pack<IO>::load(ti + off), iv);
    R.dy[st] = Pack<IO>::load(tdy + off);
    const ElemFlags f = elem_flags<MASKED>(fl[st >> 2], st);
#pragma unroll
    for (int ch = 0; ch < CV; ++ch) {
      float r, i;
      sigmoid_pair(rv[ch], iv[ch], r, i);
      const float em = expm1_nonpos<POLY>(r * K[ch]);
      const float a = 1.0f + em;
      const float gsq = fmaxf(-em * (2.0f + em), 0.0f);
      const float rs = rsqrt_approx(gsq);                 // +inf at 0
      const float gam = gsq > 0.0f ? gsq * rs : 0.0f;     // sqrt(gsq)
      const float slope = fminf(0.5f * rs, SLOPE_CAP);    // 1/sqrt(max(4 gsq, 1e-6))
      const float ix = i * xv[ch];
      float am = a, ar = a;
      float c1 = gam * i;
      float b = gam * ix;
      float c3 = (a * a) * (2.0f * slope) * ix;
      if (MASKED) {
        if (f.reset) { am = 0.0f; ar = 0.0f; c3 = 0.0f; c1 = i; b = ix; }
        if (f.inactive) { am = 1.0f; ar = 0.0f; c3 = 0.0f; c1 = 0.0f; b = 0.0f; }
      }
      R.am[st][ch] = am;
      R.ar[st][ch] = ar;
      R.c1[st][ch] = c1;
      R.c2[st][ch] = b * (1.0f - i);
      R.c3[st][ch] = c3;
      R.rr[st][ch] = r;
      R.hb[st][ch] = b;
      p[ch] *= am;
      s[ch] = fmaf(am, s[ch], b);
    }
  }
#pragma unroll
  for (int ch = 0; ch < CV; ++ch) { aggF[0][ch] = p[ch]; aggF[1][ch] = s[ch]; }
  // Reverse aggregate: carry_out = q * carry_in + c, where the carry is a_t g_t.
  float q[CV], c[CV];
#pragma unroll
  for (int ch = 0; ch < CV; ++ch) { q[ch] = 1.0f; c[ch] = 0.0f; }
#pragma unroll
  for (int st = TS - 1; st >= 0; --st) {
    float dyv[CV];
    Pack<IO>::unpack(R.dy[st], dyv);
#pragma unroll
    for (int ch = 0; ch < CV; ++ch) {
      c[ch] = R.am[st][ch] * (dyv[ch] + c[ch]);
      q[ch] *= R.am[st][ch];
    }
  }
#pragma unroll
  for (int ch = 0; ch < CV; ++ch) { aggR[0][ch] = q[ch]; aggR[1][ch] = c[ch]; }
}

template <typename IO, int TS, int NSTAGE>
struct BwdSmem {
  static constexpr int TC = LANES * TS;
  static constexpr int TILE = TC * CH * sizeof(IO);
  static constexpr int STAGE = 4 * TILE;
  static constexpr int OFF_AGGF = NSTAGE * STAGE;
  static constexpr int OFF_AGGR = OFF_AGGF + LANES * CH * 8;
  static constexpr int OFF_EINF = OFF_AGGR + LANES * CH * 8;
  static constexpr int OFF_EINR = OFF_EINF + LANES * CH * 4;
  static constexpr int OFF_BAR = OFF_EINR + LANES * CH * 4;
  static constexpr int BYTES = OFF_BAR + NSTAGE * 8 + 16;
};

template <typename IO, int TS, int NSTAGE, bool USE_TMA>
__global__ void __launch_bounds__(NT) rglru_bwd_kernel(const __grid_constant__ BwdMaps maps, const ScanBwdArgs p) {
  using SM = BwdSmem<IO, TS, NSTAGE>;
  constexpr int TC = SM::TC;
  static_assert(TC == SAVE_EVERY, "backward chunk must match the saved-state spacing");
  constexpr int ROWB = CH * sizeof(IO);
  extern __shared__ __align__(128) uint8_t smem[];
  float2* aggF = reinterpret_cast<float2*>(smem + SM::OFF_AGGF);
  float2* aggR = reinterpret_cast<float2*>(smem + SM::OFF_AGGR);
  float* einF = reinterpret_cast<float*>(smem + SM::OFF_EINF);
  float* einR = reinterpret_cast<float*>(smem + SM::OFF_EINR);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);

  const int tid = threadIdx.x;
  const int lane_t = tid / NCV;
  const int vec = tid % NCV;
  const int b = blockIdx.y;
  const int d0 = blockIdx.x * CH;
  const int nchunks = (p.T + TC - 1) / TC;

  float K[CV];
  bool poly_ok = true;
#pragma unroll
  for (int ch = 0; ch < CV; ++ch) {
    K[ch] = decay_rate(p.lambda, d0 + vec * CV + ch, p.D, p.c);
    poly_ok = poly_ok && (K[ch] >= POLY_RANGE);
  }
  const bool poly = __syncthreads_and(poly_ok);

  auto issue = [&](int q) {  // q-th chunk in processing order == chunk nchunks-1-q in time
    const int k = nchunks - 1 - q;
    const int sidx = q % NSTAGE;
    uint8_t* st = smem + sidx * SM::STAGE;
    mbar_expect_tx(&bars[sidx], SM::STAGE);
    tma_load_3d(st, &maps.dy, d0, k * TC, b, &bars[sidx]);
    tma_load_3d(st + SM::TILE, &maps.x, d0, k * TC, b, &bars[sidx]);
    tma_load_3d(st + 2 * SM::TILE, &maps.ur, d0, k * TC, b, &bars[sidx]);
    tma_load_3d(st + 3 * SM::TILE, &maps.ui, d0, k * TC, b, &bars[sidx]);
  };

  if (USE_TMA) {
    if (tid == 0) {
      prefetch_map(&maps.dy); prefetch_map(&maps.x); prefetch_map(&maps.ur); prefetch_map(&maps.ui);
      prefetch_map(&maps.dx); prefetch_map(&maps.dur); prefetch_map(&maps.dui);
      for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[s], 1);
      mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0)
      for (int q = 0; q < NSTAGE && q < nchunks; ++q) issue(q);
  }

  // Threads 0..63 chain the forward lane aggregates, threads 64..127 the reverse ones.
  const int cch = tid & (CH - 1);
  const int dch = d0 + cch;
  const bool fwd_chain = tid < CH;
  const bool rev_chain = tid >= CH && tid < 2 * CH;
  float carry_rev = 0.0f;
  if (rev_chain && dch < p.D && p.dh_last) carry_rev = p.dh_last[static_cast<size_t>(b) * p.D + dch];

  float dlam[CV] = {0.0f, 0.0f, 0.0f, 0.0f};
  const int off0 = (lane_t * TS) * ROWB + vec * Pack<IO>::BYTES;
  bool alive = true;

  for (int q = 0; q < nchunks; ++q) {
    const int k = nchunks - 1 - q;
    const int stage = USE_TMA ? (q % NSTAGE) : 0;
    uint8_t* tiles = smem + stage * SM::STAGE;
    const int t0 = k * TC;
    uint32_t fl[(TS + 3) / 4];
    const bool masked = (p.tok != nullptr) || (t0 + TC > p.T);
    if (masked) load_flags<TS>(p.tok, b, p.T, t0 + lane_t * TS, fl);

    // State entering this chunk (saved by the forward kernel; chunk 0 starts from h0).
    float enter = 0.0f;
    if (fwd_chain && dch < p.D) {
      if (k == 0) enter = p.h0 ? p.h0[static_cast<size_t>(b) * p.D + dch] : 0.0f;
      else enter = p.states[(static_cast<size_t>(b) * nchunks + k) * p.D + dch];
    }

    if (USE_TMA) {
      alive = mbar_wait_bounded(&bars[stage], (q / NSTAGE) & 1);
    } else {
      tile_load_plain<IO>(tiles, p.dy, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<IO>(tiles + SM::TILE, p.x, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<IO>(tiles + 2 * SM::TILE, p.ur, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<IO>(tiles + 3 * SM::TILE, p.ui, b, t0, d0, TC, p.T, p.D);
      __syncthreads();
    }

    BwdRegs<IO, TS> R;
    float lf[2][CV], lr[2][CV];
    {
      const uint8_t* tdy = tiles;
      const uint8_t* tx = tiles + SM::TILE;
      const uint8_t* tr = tiles + 2 * SM::TILE;
      const uint8_t* ti = tiles + 3 * SM::TILE;
      if (masked) {
        if (poly) bwd_local<IO, TS, true, true>(tdy, tx, tr, ti, off0, K, fl, R, lf, lr);
        else bwd_local<IO, TS, true, false>(tdy, tx, tr, ti, off0, K, fl, R, lf, lr);
      } else {
        if (poly) bwd_local<IO, TS, false, true>(tdy, tx, tr, ti, off0, K, fl, R, lf, lr);
        else bwd_local<IO, TS, false, false>(tdy, tx, tr, ti, off0, K, fl, R, lf, lr);
      }
    }
    {
      float4* df = reinterpret_cast<float4*>(aggF + lane_t * CH + vec * CV);
      df[0] = make_float4(lf[0][0], lf[1][0], lf[0][1], lf[1][1]);
      df[1] = make_float4(lf[0][2], lf[1][2], lf[0][3], lf[1][3]);
      float4* dr = reinterpret_cast<float4*>(aggR + lane_t * CH + vec * CV);
      dr[0] = make_float4(lr[0][0], lr[1][0], lr[0][1], lr[1][1]);
      dr[1] = make_float4(lr[0][2], lr[1][2], lr[0][3], lr[1][3]);
    }
    alive = __syncthreads_and(alive);
    if (!alive) break;

    if (fwd_chain) {
      float2 ag[LANES];
#pragma unroll
      for (int j = 0; j < LANES; ++j) ag[j] = aggF[j * CH + cch];
      float e = enter;
#pragma unroll
      for (int j = 0; j < LANES; ++j) {
        einF[j * CH + cch] = e;
        e = fmaf(ag[j].x, e, ag[j].y);
      }
    } else if (rev_chain) {
      float2 ag[LANES];
#pragma unroll
      for (int j = 0; j < LANES; ++j) ag[j] = aggR[j * CH + cch];
      float e = carry_rev;
#pragma unroll
      for (int j = LANES - 1; j >= 0; --j) {
        einR[j * CH + cch] = e;
        e = fmaf(ag[j].x, e, ag[j].y);
      }
      carry_rev = e;
    }
    __syncthreads();

    {
      const float4 f4 = *reinterpret_cast<const float4*>(einF + lane_t * CH + vec * CV);
      const float4 r4 = *reinterpret_cast<const float4*>(einR + lane_t * CH + vec * CV);
      float h[CV] = {f4.x, f4.y, f4.z, f4.w};
      float c[CV] = {r4.x, r4.y, r4.z, r4.w};
      // States entering each step, rebuilt forward in time.
#pragma unroll
      for (int st = 0; st < TS; ++st) {
#pragma unroll
        for (int ch = 0; ch < CV; ++ch) {
          const float hin = h[ch];
          h[ch] = fmaf(R.am[st][ch], hin, R.hb[st][ch]);
          R.hb[st][ch] = hin;
        }
      }
      uint8_t* tdx = tiles + SM::TILE;       // over x
      uint8_t* tdr = tiles + 2 * SM::TILE;   // over u_r
      uint8_t* tdi = tiles + 3 * SM::TILE;   // over u_i
#pragma unroll
      for (int st = TS - 1; st >= 0; --st) {
        float dyv[CV], dxv[CV], drv[CV], div[CV];
        Pack<IO>::unpack(R.dy[st], dyv);
#pragma unroll
        for (int ch = 0; ch < CV; ++ch) {
          const float g = dyv[ch] + c[ch];
          c[ch] = R.am[st][ch] * g;
          dxv[ch] = g * R.c1[st][ch];
          div[ch] = g * R.c2[st][ch];
          const float dl = g * fmaf(R.hb[st][ch], R.ar[st][ch], -R.c3[st][ch]);
          const float w = dl * R.rr[st][ch];
          dlam[ch] += w;
          drv[ch] = w * fmaf(-K[ch], R.rr[st][ch], K[ch]);
        }
        const int off = off0 + st * ROWB;
        Pack<IO>::store(tdx + off, dxv);
        Pack<IO>::store(tdr + off, drv);
        Pack<IO>::store(tdi + off, div);
      }
    }
    if (USE_TMA) {
      fence_async_smem();
      __syncthreads();
      if (tid == 0) {
        tma_store_3d(&maps.dx, tiles + SM::TILE, d0, t0, b);
        tma_store_3d(&maps.dur, tiles + 2 * SM::TILE, d0, t0, b);
        tma_store_3d(&maps.dui, tiles + 3 * SM::TILE, d0, t0, b);
        tma_commit();
        const int qp = q - 1;
        if (qp >= 0 && qp + NSTAGE < nchunks) {
          tma_wait_read<1>();
          issue(qp + NSTAGE);
        }
      }
    } else {
      __syncthreads();
      tile_store_plain<IO>(tiles + SM::TILE, p.dx, b, t0, d0, TC, p.T, p.D);
      tile_store_plain<IO>(tiles + 2 * SM::TILE, p.dur, b, t0, d0, TC, p.T, p.D);
      tile_store_plain<IO>(tiles + 3 * SM::TILE, p.dui, b, t0, d0, TC, p.T, p.D);
      __syncthreads();
    }
  }

  if (USE_TMA && tid == 0) {
    tma_wait_all<0>();
    if (!alive) atomicExch(p.status, DEV_TIMEOUT_LOAD);
  }
  if (!alive) return;
  if (rev_chain && dch < p.D && p.dh0) p.dh0[static_cast<size_t>(b) * p.D + dch] = carry_rev;

  // Per-row partial of sum_t dl * r: fold the 16 time-lanes in a fixed order.
  __syncthreads();
  *reinterpret_cast<float4*>(einF + lane_t * CH + vec * CV) = make_float4(dlam[0], dlam[1], dlam[2], dlam[3]);
  __syncthreads();
  if (tid < CH && dch < p.D) {
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < LANES; ++j) acc += einF[j * CH + tid];
    p.dlam_part[static_cast<size_t>(b) * p.D + dch] = acc;
  }
}

// dLambda[d] = sigmoid(-Lambda_d) * c * sum_b partial[b, d], rows added in index order.
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

constexpr int RAW_TS = 4;
constexpr int RAW_TC = LANES * RAW_TS;
constexpr int RAW_TILE = RAW_TC * CH * 4;

template <int NSTAGE>
struct RawSmem {
  static constexpr int NTILE = 3;
  static constexpr int STAGE = NTILE * RAW_TILE;
  static constexpr int OFF_AGG = NSTAGE * STAGE;
  static constexpr int OFF_EIN = OFF_AGG + LANES * CH * 8;
  static constexpr int OFF_BAR = OFF_EIN + LANES * CH * 4;
  static constexpr int BYTES = OFF_BAR + NSTAGE * 8 + 16;
};

template <int NSTAGE, bool USE_TMA>
__global__ void __launch_bounds__(NT) rawscan_fwd_kernel(const __grid_constant__ RawFwdMaps maps, const RawScanArgs p) {
  using SM = RawSmem<NSTAGE>;
  constexpr int TS = RAW_TS, TC = RAW_TC, ROWB = CH * 4;
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
      tile_load_plain<float>(tiles, p.drive, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<float>(tiles + RAW_TILE, p.decay, b, t0, d0, TC, p.T, p.D);
      __syncthreads();
    }
    float P[TS][CV], S[TS][CV];
    {
      float pp[CV] = {1.0f, 1.0f, 1.0f, 1.0f}, ss[CV] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int st = 0; st < TS; ++st) {
        float bv[CV], av[CV];
        Pack<float>::unpack(Pack<float>::load(tiles + off0 + st * ROWB), bv);
        Pack<float>::unpack(Pack<float>::load(tiles + RAW_TILE + off0 + st * ROWB), av);
        const bool pad = t0 + lane_t * TS + st >= p.T;  // steps past T carry the state through
#pragma unroll
        for (int ch = 0; ch < CV; ++ch) {
          const float a = pad ? 1.0f : av[ch];
          const float bb = pad ? 0.0f : bv[ch];
          pp[ch] *= a;
          ss[ch] = fmaf(a, ss[ch], bb);
          P[st][ch] = pp[ch];
          S[st][ch] = ss[ch];
        }
      }
    }
    {
      float4* dst = reinterpret_cast<float4*>(agg + lane_t * CH + vec * CV);
      dst[0] = make_float4(P[TS - 1][0], S[TS - 1][0], P[TS - 1][1], S[TS - 1][1]);
      dst[1] = make_float4(P[TS - 1][2], S[TS - 1][2], P[TS - 1][3], S[TS - 1][3]);
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
      const float e[CV] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
      for (int st = 0; st < TS; ++st) {
        float yv[CV];
#pragma unroll
        for (int ch = 0; ch < CV; ++ch) yv[ch] = fmaf(P[st][ch], e[ch], S[st][ch]);
        Pack<float>::store(tiles + off0 + st * ROWB, yv);
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
      tile_store_plain<float>(tiles, p.out, b, t0, d0, TC, p.T, p.D);
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
__global__ void __launch_bounds__(NT) rawscan_bwd_kernel(const __grid_constant__ RawBwdMaps maps, const RawScanArgs p) {
  using SM = RawSmem<NSTAGE>;
  constexpr int TS = RAW_TS, TC = RAW_TC, ROWB = CH * 4;
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
      tile_load_plain<float>(tiles, p.dout, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<float>(tiles + RAW_TILE, p.decay, b, t0, d0, TC, p.T, p.D);
      tile_load_plain<float>(tiles + 2 * RAW_TILE, p.out_in, b, t0 - 1, d0, TC, p.T, p.D);
      __syncthreads();
    }
    float av[TS][CV], gv[TS][CV], hv[TS][CV];
    float qq[CV] = {1.0f, 1.0f, 1.0f, 1.0f}, cc[CV] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int st = 0; st < TS; ++st) {
      Pack<float>::unpack(Pack<float>::load(tiles + off0 + st * ROWB), gv[st]);
      Pack<float>::unpack(Pack<float>::load(tiles + RAW_TILE + off0 + st * ROWB), av[st]);
      Pack<float>::unpack(Pack<float>::load(tiles + 2 * RAW_TILE + off0 + st * ROWB), hv[st]);
    }
    if (k == 0 && lane_t == 0) {  // the state entering t = 0
#pragma unroll
      for (int ch = 0; ch < CV; ++ch) {
        const int d = d0 + vec * CV + ch;
        hv[0][ch] = (p.h0 && d < p.D) ? p.h0[static_cast<size_t>(b) * p.D + d] : 0.0f;
      }
    }
#pragma unroll
    for (int st = TS - 1; st >= 0; --st)
#pragma unroll
      for (int ch = 0; ch < CV; ++ch) {
        cc[ch] = av[st][ch] * (gv[st][ch] + cc[ch]);
        qq[ch] *= av[st][ch];
      }
    {
      float4* dst = reinterpret_cast<float4*>(agg + lane_t * CH + vec * CV);
      dst[0] = make_float4(qq[0], cc[0], qq[1], cc[1]);
      dst[1] = make_float4(qq[2], cc[2], qq[3], cc[3]);
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
      float c[CV] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
      for (int st = TS - 1; st >= 0; --st) {
        float da[CV], db[CV];
#pragma unroll
        for (int ch = 0; ch < CV; ++ch) {
          const float g = gv[st][ch] + c[ch];
          c[ch] = av[st][ch] * g;
          db[ch] = g;
          da[ch] = g * hv[st][ch];
        }
        Pack<float>::store(tiles + off0 + st * ROWB, db);
        Pack<float>::store(tiles + RAW_TILE + off0 + st * ROWB, da);
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
      tile_store_plain<float>(tiles, p.ddrive, b, t0, d0, TC, p.T, p.D);
      tile_store_plain<float>(tiles + RAW_TILE, p.ddecay, b, t0, d0, TC, p.T, p.D);
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
// Launchers
// ======================================================================

constexpr int FWD_TS = 4;
constexpr int BWD_TS = 4;
constexpr int FWD_STAGES_BF16 = 4, FWD_STAGES_F32 = 3;
constexpr int BWD_STAGES_BF16 = 3, BWD_STAGES_F32 = 2;

int scan_fwd_box_rows(bool) { return LANES * FWD_TS; }
int scan_bwd_box_rows(bool) { return LANES * BWD_TS; }

template <typename Kern>
static cudaError_t set_smem(Kern kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <typename IO, int NSTAGE, bool USE_TMA>
static cudaError_t launch_fwd_t(const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  constexpr int ST = USE_TMA ? NSTAGE : 1;
  auto kern = rglru_fwd_kernel<IO, FWD_TS, ST, USE_TMA>;
  constexpr int bytes = FwdSmem<IO, FWD_TS, ST>::BYTES;
  cudaError_t e = set_smem(kern, bytes);
  if (e != cudaSuccess) return e;
  dim3 grid((a.D + CH - 1) / CH, a.B);
  kern<<<grid, NT, bytes, s>>>(maps, a);
  return cudaGetLastError();
}

cudaError_t launch_scan_fwd(bool bf16, bool use_tma, const FwdMaps& maps, const ScanFwdArgs& a, cudaStream_t s) {
  if (bf16) {
    return use_tma ? launch_fwd_t<__nv_bfloat16, FWD_STAGES_BF16, true>(maps, a, s)
                   : launch_fwd_t<__nv_bfloat16, 1, false>(maps, a, s);
  }
  return use_tma ? launch_fwd_t<float, FWD_STAGES_F32, true>(maps, a, s) : launch_fwd_t<float, 1, false>(maps, a, s);
}

template <typename IO, int NSTAGE, bool USE_TMA>
static cudaError_t launch_bwd_t(const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  constexpr int ST = USE_TMA ? NSTAGE : 1;
  auto kern = rglru_bwd_kernel<IO, BWD_TS, ST, USE_TMA>;
  constexpr int bytes = BwdSmem<IO, BWD_TS, ST>::BYTES;
  cudaError_t e = set_smem(kern, bytes);
  if (e != cudaSuccess) return e;
  dim3 grid((a.D + CH - 1) / CH, a.B);
  kern<<<grid, NT, bytes, s>>>(maps, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  rglru_dlambda_kernel<<<(a.D + 255) / 256, 256, 0, s>>>(a.dlam_part, a.lambda, a.dlambda, a.B, a.D, a.c);
  return cudaGetLastError();
}

cudaError_t launch_scan_bwd(bool bf16, bool use_tma, const BwdMaps& maps, const ScanBwdArgs& a, cudaStream_t s) {
  if (bf16) {
    return use_tma ? launch_bwd_t<__nv_bfloat16, BWD_STAGES_BF16, true>(maps, a, s)
                   : launch_bwd_t<__nv_bfloat16, 1, false>(maps, a, s);
  }
  return use_tma ? launch_bwd_t<float, BWD_STAGES_F32, true>(maps, a, s) : launch_bwd_t<float, 1, false>(maps, a, s);
}

int raw_box_rows() { return RAW_TC; }

template <int NSTAGE, bool USE_TMA>
static cudaError_t launch_raw_fwd_t(const RawFwdMaps& maps, const RawScanArgs& a, cudaStream_t s) {
  auto kern = rawscan_fwd_kernel<NSTAGE, USE_TMA>;
  constexpr int bytes = RawSmem<NSTAGE>::BYTES;
  cudaError_t e = set_smem(kern, bytes);
  if (e != cudaSuccess) return e;
  dim3 grid((a.D + CH - 1) / CH, a.B);
  kern<<<grid, NT, bytes, s>>>(maps, a);
  return cudaGetLastError();
}
cudaError_t launch_raw_fwd(bool use_tma, const RawFwdMaps& maps, const RawScanArgs& a, cudaStream_t s) {
  return use_tma ? launch_raw_fwd_t<3, true>(maps, a, s) : launch_raw_fwd_t<1, false>(maps, a, s);
}
template <int NSTAGE, bool USE_TMA>
static cudaError_t launch_raw_bwd_t(const RawBwdMaps& maps, const RawScanArgs& a, cudaStream_t s) {
  auto kern = rawscan_bwd_kernel<NSTAGE, USE_TMA>;
  constexpr int bytes = RawSmem<NSTAGE>::BYTES;
  cudaError_t e = set_smem(kern, bytes);
  if (e != cudaSuccess) return e;
  dim3 grid((a.D + CH - 1) / CH, a.B);
  kern<<<grid, NT, bytes, s>>>(maps, a);
  return cudaGetLastError();
}
cudaError_t launch_raw_bwd(bool use_tma, const RawBwdMaps& maps, const RawScanArgs& a, cudaStream_t s) {
  return use_tma ? launch_raw_bwd_t<3, true>(maps, a, s) : launch_raw_bwd_t<1, false>(maps, a, s);
}

}  // namespace rglru
