// Causal depthwise convolution (kernel width 4) in front of the RG-LRU, its
// backward, and the two single-token decode kernels.  All are streaming
// kernels: every activation is read once and written once, each thread owning
// four channels and sliding a 4-row register window over a run of time-steps
// (the three-row halo is re-read once per run).  A thread issues the loads of
// several steps before it touches the first of them, and batches made only of
// ordinary tokens (no document boundary, no padding) take a mask-free path.
//
// Reference behaviour: griffin/griffin.py:474-487 (dense path), :488-510
// (right-padded path), :459-528 at T = 1 (decode).

#include "rglru_device.cuh"
#include "rglru_internal.h"

namespace rglru {

constexpr int CONV_TAPS = 4;
// Time-steps whose loads a thread issues together: 8 rows of 8 bytes for bf16, 4 rows of 16 bytes for fp32
// (measured on B200: deeper batches spill for fp32, shallower ones leave bf16 latency-bound).
template <typename IO>
struct ConvUnroll { static constexpr int value = sizeof(IO) == 2 ? 8 : 4; };

template <int BYTES> struct RawWord { using type = uint32_t; };
template <> struct RawWord<8> { using type = uint2; };
template <> struct RawWord<16> { using type = uint4; };

// VEC channels of IO as one aligned 8- or 16-byte access (VEC == 1: scalar fallback for odd widths).  The
// raw form is what a thread keeps in registers while several loads are in flight.
template <typename IO, int VEC>
struct Vec {
  static constexpr int BYTES = VEC * static_cast<int>(sizeof(IO));
  static_assert(VEC == 1 || BYTES == 8 || BYTES == 16, "one 8- or 16-byte access per thread and row");
  using Raw = typename RawWord<VEC == 1 ? 4 : BYTES>::type;

  static __device__ __forceinline__ Raw load_raw(const IO* p) {
    if constexpr (VEC == 1) {
      if constexpr (sizeof(IO) == 4) return __float_as_uint(p[0]);
      else return static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(p)) << 16;
    } else {
      return *reinterpret_cast<const Raw*>(p);
    }
  }
  static __device__ __forceinline__ void unpack(const Raw& r, float (&v)[VEC]) {
    if constexpr (VEC == 1) {
      v[0] = __uint_as_float(r);
    } else {
      constexpr int NW = BYTES / 4;
      uint32_t w[NW];
      if constexpr (NW == 2) { w[0] = r.x; w[1] = r.y; }
      else { w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w; }
      if constexpr (sizeof(IO) == 4) {
#pragma unroll
        for (int k = 0; k < NW; ++k) v[k] = __uint_as_float(w[k]);
      } else {
#pragma unroll
        for (int k = 0; k < NW; ++k) {
          v[2 * k] = __uint_as_float(w[k] << 16);
          v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        }
      }
    }
  }
  static __device__ __forceinline__ void load(const IO* p, float (&v)[VEC]) { unpack(load_raw(p), v); }
  static __device__ __forceinline__ void store(IO* p, const float (&v)[VEC]) {
    if constexpr (VEC == 1) {
      p[0] = Pack<IO>::from_float(v[0]);
    } else {
      constexpr int NW = BYTES / 4;
      uint32_t w[NW];
      if constexpr (sizeof(IO) == 4) {
#pragma unroll
        for (int k = 0; k < NW; ++k) w[k] = __float_as_uint(v[k]);
      } else {
#pragma unroll
        for (int k = 0; k < NW; ++k) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
          w[k] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      if constexpr (NW == 2) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
      else *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
};

// Channels per thread of the conv kernels: 4 for both element types (8-byte accesses for bf16), which keeps
// the per-thread weights, windows and raw batch small enough for several resident blocks per SM.  The decode
// kernels, with nothing to keep, use full 16-byte accesses.
template <typename IO>
constexpr int vec_width() { return 16 / sizeof(IO); }
constexpr int CONV_VEC = 4;

// The four taps of VEC channels starting at d: wt[k][v] = w[d + v, k] (one 16-byte load per channel).
template <int VEC>
__device__ __forceinline__ void load_conv_weights(const float* __restrict__ w, int d, float (&wt)[CONV_TAPS][VEC]) {
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    if constexpr (VEC == 1) {
#pragma unroll
      for (int k = 0; k < CONV_TAPS; ++k) wt[k][v] = w[(d + v) * CONV_TAPS + k];
    } else {
      const float4 q = *reinterpret_cast<const float4*>(w + static_cast<size_t>(d + v) * CONV_TAPS);
      wt[0][v] = q.x; wt[1][v] = q.y; wt[2][v] = q.z; wt[3][v] = q.w;
    }
  }
}

// ---------------------------------------------------------------- forward
// Thread = (batch row, run of RUN time-steps, VEC channels).
template <typename IO, int VEC, int RUN>
__global__ void __launch_bounds__(256, 3) conv_fwd_kernel(const IO* __restrict__ xin, const float* __restrict__ w,
                                                       const float* __restrict__ bias, const IO* __restrict__ state,
                                                       const uint8_t* __restrict__ tok, IO* __restrict__ out, int B,
                                                       int T, int D) {
  constexpr int UNROLL = ConvUnroll<IO>::value;
  const int nvec = D / VEC;
  const int nrun = (T + RUN - 1) / RUN;
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<long long>(B) * nrun * nvec) return;
  const int dv = static_cast<int>(gid % nvec);
  const int run = static_cast<int>((gid / nvec) % nrun);
  const int b = static_cast<int>(gid / nvec / nrun);
  const int d = dv * VEC;
  const int t_begin = run * RUN;
  const int t_end = min(T, t_begin + RUN);

  float wt[CONV_TAPS][VEC], bs[VEC];
  load_conv_weights<VEC>(w, d, wt);
#pragma unroll
  for (int v = 0; v < VEC; ++v) bs[v] = bias ? bias[d + v] : 0.0f;
  // hist[l-1] holds the input l steps before the current one.
  float hist[CONV_TAPS - 1][VEC];
#pragma unroll
  for (int l = 1; l < CONV_TAPS; ++l) {
    const int t = t_begin - l;
    if (t >= 0) {
      Vec<IO, VEC>::load(xin + (static_cast<size_t>(b) * T + t) * D + d, hist[l - 1]);
    } else if (state) {
      Vec<IO, VEC>::load(state + (static_cast<size_t>(b) * (CONV_TAPS - 1) + (CONV_TAPS - 1 + t)) * D + d, hist[l - 1]);
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) hist[l - 1][v] = 0.0f;
    }
  }
  // Steps are taken UNROLL at a time with all of a batch's loads issued before its arithmetic, so that
  // every thread keeps several 16-byte requests in flight.
  for (int t0 = t_begin; t0 < t_end; t0 += UNROLL) {
    typename Vec<IO, VEC>::Raw raw[UNROLL];
    uint32_t fl[UNROLL];
    uint32_t any_flag = 0u;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int t = t0 + u;
      fl[u] = 0u;
      if (t < t_end) {
        raw[u] = Vec<IO, VEC>::load_raw(xin + (static_cast<size_t>(b) * T + t) * D + d);
        if (tok) fl[u] = tok[static_cast<size_t>(b) * T + t];
      }
      any_flag |= fl[u];
    }
    if (any_flag == 0u && t0 + UNROLL <= t_end) {
      // Ordinary tokens only (uniform across the warp, whose threads share the time range): all four taps.
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        float acc[VEC], cur[VEC];
        Vec<IO, VEC>::unpack(raw[u], cur);
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          float a = fmaf(wt[3][v], cur[v], bs[v]);
          a = fmaf(wt[2][v], hist[0][v], a);
          a = fmaf(wt[1][v], hist[1][v], a);
          acc[v] = fmaf(wt[0][v], hist[2][v], a);
        }
        Vec<IO, VEC>::store(out + (static_cast<size_t>(b) * T + t0 + u) * D + d, acc);
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          hist[2][v] = hist[1][v];
          hist[1][v] = hist[0][v];
          hist[0][v] = cur[v];
        }
      }
      continue;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int t = t0 + u;
      if (t >= t_end) break;
      const uint32_t f = fl[u];
      const int reach = 3 - static_cast<int>(f & TOK_CUT_MASK);  // taps with lag <= reach stay inside the document
      float acc[VEC], cur[VEC];
      Vec<IO, VEC>::unpack(raw[u], cur);
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        float a = fmaf(wt[3][v], cur[v], bs[v]);
        if (reach >= 1) a = fmaf(wt[2][v], hist[0][v], a);
        if (reach >= 2) a = fmaf(wt[1][v], hist[1][v], a);
        if (reach >= 3) a = fmaf(wt[0][v], hist[2][v], a);
        acc[v] = (f & TOK_INACTIVE) ? 0.0f : a;
      }
      Vec<IO, VEC>::store(out + (static_cast<size_t>(b) * T + t) * D + d, acc);
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        hist[2][v] = hist[1][v];
        hist[1][v] = hist[0][v];
        hist[0][v] = cur[v];
      }
    }
  }
}

// Next conv state: the last three inputs of the active prefix of each row (older
// entries come from the previous state); entries older than the last token flagged
// ZERO_HISTORY are zero.  One block per (channel slab, row).
template <typename IO>
__global__ void conv_state_kernel(const IO* __restrict__ xin, const IO* __restrict__ state,
                                  const uint8_t* __restrict__ tok, IO* __restrict__ new_state, int T, int D) {
  __shared__ int s_len, s_zero;
  const int b = blockIdx.y;
  if (threadIdx.x == 0) { s_len = tok ? 0 : T; s_zero = -4; }
  __syncthreads();
  if (tok) {
    int len = 0, zero_at = -4;
    for (int t = threadIdx.x; t < T; t += blockDim.x) {
      const uint32_t f = tok[static_cast<size_t>(b) * T + t];
      if (!(f & TOK_INACTIVE)) {
        len = max(len, t + 1);
        if (f & TOK_ZERO_HISTORY) zero_at = max(zero_at, t);
      }
    }
    atomicMax(&s_len, len);
    atomicMax(&s_zero, zero_at);
    __syncthreads();
  }
  const int len = s_len, zero_at = s_zero;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
#pragma unroll
  for (int slot = 0; slot < CONV_TAPS - 1; ++slot) {
    const int t = len - (CONV_TAPS - 1) + slot;
    float v = 0.0f;
    if (t >= zero_at) {
      if (t >= 0) v = Pack<IO>::to_float(xin[(static_cast<size_t>(b) * T + t) * D + d]);
      else if (state) v = Pack<IO>::to_float(state[(static_cast<size_t>(b) * (CONV_TAPS - 1) + (CONV_TAPS - 1 + t)) * D + d]);
    }
    new_state[(static_cast<size_t>(b) * (CONV_TAPS - 1) + slot) * D + d] = Pack<IO>::from_float(v);
  }
}

// ---------------------------------------------------------------- backward
// dx_in[t] = sum_lag w[3-lag] * dconv[t+lag] * [tap (t+lag, lag) inside its document]
// d_w[3-lag] += dconv[t] * xin[t-lag] (same mask), d_b += dconv[t].
// Block = 8 runs x 32 channel vectors; the 8 runs are folded in shared memory so one
// partial row [5, D] is written per (row, 8*RUN time-steps).
template <typename IO, int VEC, int RUN>
__global__ void __launch_bounds__(256, 2) conv_bwd_kernel(const IO* __restrict__ dconv, const IO* __restrict__ xin,
                                                       const float* __restrict__ w, const IO* __restrict__ state,
                                                       const uint8_t* __restrict__ tok, IO* __restrict__ dxin,
                                                       IO* __restrict__ dstate, float* __restrict__ part, int B, int T,
                                                       int D) {
  constexpr int RUNS_PER_BLOCK = 8, VECS_PER_BLOCK = 32;
  constexpr int UNROLL = ConvUnroll<IO>::value;
  __shared__ float red[RUNS_PER_BLOCK][5][VECS_PER_BLOCK * VEC + 1];
  const int nvec = D / VEC;
  const int vslot = threadIdx.x % VECS_PER_BLOCK;
  const int rslot = threadIdx.x / VECS_PER_BLOCK;
  const int dv = blockIdx.x * VECS_PER_BLOCK + vslot;
  const int run = blockIdx.y * RUNS_PER_BLOCK + rslot;
  const int b = blockIdx.z;
  const bool live = dv < nvec;
  const int d = dv * VEC;
  const int t_begin = run * RUN;
  const int t_end = min(T, t_begin + RUN);

  float gw[5][VEC];
#pragma unroll
  for (int k = 0; k < 5; ++k)
#pragma unroll
    for (int v = 0; v < VEC; ++v) gw[k][v] = 0.0f;

  if (live && t_begin < T) {
    float wt[CONV_TAPS][VEC];
    load_conv_weights<VEC>(w, d, wt);

    auto load_in = [&](int t, float (&v)[VEC]) {
      if (t >= 0) Vec<IO, VEC>::load(xin + (static_cast<size_t>(b) * T + t) * D + d, v);
      else if (state) Vec<IO, VEC>::load(state + (static_cast<size_t>(b) * (CONV_TAPS - 1) + (CONV_TAPS - 1 + t)) * D + d, v);
      else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] = 0.0f;
      }
    };
    // Masked upstream gradient of the token at time t (zero outside [0, T) and on padding)
    // together with how far back its taps reach.
    auto load_grad = [&](int t, float (&g)[VEC], int& reach) {
      reach = -1;
#pragma unroll
      for (int k = 0; k < VEC; ++k) g[k] = 0.0f;
      if (t < 0 || t >= T) return;
      const uint32_t f = tok ? tok[static_cast<size_t>(b) * T + t] : 0u;
      if (f & TOK_INACTIVE) return;
      reach = 3 - static_cast<int>(f & TOK_CUT_MASK);
      Vec<IO, VEC>::load(dconv + (static_cast<size_t>(b) * T + t) * D + d, g);
    };
    // The same in raw form: reach < 0 means "contributes nothing" and the raw value is then unspecified.
    using Raw = typename Vec<IO, VEC>::Raw;
    auto load_grad_raw = [&](int t, Raw& g, int& reach) {
      reach = -1;
      if (t < 0 || t >= T) return;
      const uint32_t f = tok ? tok[static_cast<size_t>(b) * T + t] : 0u;
      if (f & TOK_INACTIVE) return;
      reach = 3 - static_cast<int>(f & TOK_CUT_MASK);
      g = Vec<IO, VEC>::load_raw(dconv + (static_cast<size_t>(b) * T + t) * D + d);
    };

    // Sliding windows: xin at t-1..t-3 (for d_w) and dconv at t+1..t+3 (for dx_in).
    float hist[3][VEC];
#pragma unroll
    for (int l = 1; l <= 3; ++l) load_in(t_begin - l, hist[l - 1]);
    float g0[VEC], g1[VEC], g2[VEC], g3[VEC];
    int r0, r1, r2, r3;
    load_grad(t_begin, g0, r0);
    load_grad(t_begin + 1, g1, r1);
    load_grad(t_begin + 2, g2, r2);

    // History rows before t = 0 receive gradient only from the first run of a row.
    if (dstate && t_begin == 0) {
      float e1[VEC], e2[VEC];
      int q1, q2;
      load_grad(1, e1, q1);
      load_grad(2, e2, q2);
#pragma unroll
      for (int slot = 0; slot < 3; ++slot) {  // slot holds time slot-3
        float acc[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          float a = 0.0f;
          // token at time u reads this row with lag u - (slot-3)
          if (3 - slot <= r0) a = fmaf(wt[slot][v], g0[v], a);
          if (slot >= 1 && 4 - slot <= q1) a = fmaf(wt[slot >= 1 ? slot - 1 : 0][v], e1[v], a);
          if (slot >= 2 && 5 - slot <= q2) a = fmaf(wt[slot >= 2 ? slot - 2 : 0][v], e2[v], a);
          acc[v] = a;
        }
        Vec<IO, VEC>::store(dstate + (static_cast<size_t>(b) * 3 + slot) * D + d, acc);
      }
    }

    // UNROLL steps at a time, loads first (see the forward kernel).
    for (int t0 = t_begin; t0 < t_end; t0 += UNROLL) {
      Raw curs[UNROLL], gin[UNROLL];
      int rin[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        rin[u] = -1;
        if (t0 + u < t_end) {   // t0 + u >= 0 here, so the input row comes from xin itself
          curs[u] = Vec<IO, VEC>::load_raw(xin + (static_cast<size_t>(b) * T + t0 + u) * D + d);
          load_grad_raw(t0 + u + 3, gin[u], rin[u]);
        }
      }
      bool ordinary = (t0 + UNROLL <= t_end) && r0 == 3 && r1 == 3 && r2 == 3;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) ordinary = ordinary && rin[u] == 3;
      if (ordinary) {
        // Every token that touches this batch is an ordinary one (uniform across the warp): no tap masks.
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          float dx[VEC], cur[VEC];
          Vec<IO, VEC>::unpack(curs[u], cur);
          Vec<IO, VEC>::unpack(gin[u], g3);
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            float a = wt[3][v] * g0[v];
            a = fmaf(wt[2][v], g1[v], a);
            a = fmaf(wt[1][v], g2[v], a);
            dx[v] = fmaf(wt[0][v], g3[v], a);
            gw[4][v] += g0[v];
            gw[3][v] = fmaf(g0[v], cur[v], gw[3][v]);
            gw[2][v] = fmaf(g0[v], hist[0][v], gw[2][v]);
            gw[1][v] = fmaf(g0[v], hist[1][v], gw[1][v]);
            gw[0][v] = fmaf(g0[v], hist[2][v], gw[0][v]);
          }
          Vec<IO, VEC>::store(dxin + (static_cast<size_t>(b) * T + t0 + u) * D + d, dx);
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            hist[2][v] = hist[1][v]; hist[1][v] = hist[0][v]; hist[0][v] = cur[v];
            g0[v] = g1[v]; g1[v] = g2[v]; g2[v] = g3[v];
          }
        }
        continue;
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int t = t0 + u;
        if (t >= t_end) break;
        float dx[VEC], cur[VEC];
        r3 = rin[u];
        Vec<IO, VEC>::unpack(curs[u], cur);
        if (r3 >= 0) Vec<IO, VEC>::unpack(gin[u], g3);
        else {
#pragma unroll
          for (int v = 0; v < VEC; ++v) g3[v] = 0.0f;
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          float a = 0.0f;
          if (r0 >= 0) a = wt[3][v] * g0[v];
          if (r1 >= 1) a = fmaf(wt[2][v], g1[v], a);
          if (r2 >= 2) a = fmaf(wt[1][v], g2[v], a);
          if (r3 >= 3) a = fmaf(wt[0][v], g3[v], a);
          dx[v] = a;
          gw[4][v] += g0[v];
          gw[3][v] = fmaf(g0[v], cur[v], gw[3][v]);
          if (r0 >= 1) gw[2][v] = fmaf(g0[v], hist[0][v], gw[2][v]);
          if (r0 >= 2) gw[1][v] = fmaf(g0[v], hist[1][v], gw[1][v]);
          if (r0 >= 3) gw[0][v] = fmaf(g0[v], hist[2][v], gw[0][v]);
        }
        Vec<IO, VEC>::store(dxin + (static_cast<size_t>(b) * T + t) * D + d, dx);
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          hist[2][v] = hist[1][v]; hist[1][v] = hist[0][v]; hist[0][v] = cur[v];
          g0[v] = g1[v]; g1[v] = g2[v]; g2[v] = g3[v];
        }
        r0 = r1; r1 = r2; r2 = r3;
      }
    }
  }

#pragma unroll
  for (int k = 0; k < 5; ++k)
#pragma unroll
    for (int v = 0; v < VEC; ++v) red[rslot][k][vslot * VEC + v] = gw[k][v];
  __syncthreads();
  // Fold the 8 runs in index order; thread -> (k, channel) pairs of this block.
  const int nblk_t = gridDim.y;
  float* row = part + (static_cast<size_t>(b) * nblk_t + blockIdx.y) * 5 * D;
  for (int idx = threadIdx.x; idx < 5 * VECS_PER_BLOCK * VEC; idx += blockDim.x) {
    const int k = idx / (VECS_PER_BLOCK * VEC);
    const int cc = idx % (VECS_PER_BLOCK * VEC);
    const int dd = blockIdx.x * VECS_PER_BLOCK * VEC + cc;
    if (dd >= D) continue;
    float acc = 0.0f;
#pragma unroll
    for (int r = 0; r < RUNS_PER_BLOCK; ++r) acc += red[r][k][cc];
    row[static_cast<size_t>(k) * D + dd] = acc;
  }
}

// d_w[d, k] = sum over partial rows; d_b[d] likewise.  Rows are added in index order.
__global__ void conv_bwd_reduce_kernel(const float* __restrict__ part, float* __restrict__ dw, float* __restrict__ db,
                                       int rows, int D) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= 5 * D) return;
  const int k = idx / D, d = idx % D;
  float acc = 0.0f;
  for (int r = 0; r < rows; ++r) acc += part[(static_cast<size_t>(r) * 5 + k) * D + d];
  if (k < 4) dw[d * CONV_TAPS + k] = acc;
  else if (db) db[d] = acc;
}

// ---------------------------------------------------------------- column sums
// out[c] = sum over rows of src[r, c] for a dense row-major [rows, cols] matrix (the bias gradient of a linear
// layer from the gradient of its output).  Two launches, fixed summation order, no atomics: a grid of
// (column tile, row block) CTAs of 32 column vectors x 8 row lanes keeps UNROLL 16-byte loads per thread in
// flight and leaves one fp32 partial row per row block; the second kernel folds the partial rows, eight
// interleaved lanes per column combined in lane order.
constexpr int COLSUM_LANES = 8;
constexpr int COLSUM_UNROLL = 4;

template <typename IO, int VEC>
__global__ void __launch_bounds__(32 * COLSUM_LANES) colsum_partial_kernel(const IO* __restrict__ src,
                                                                          float* __restrict__ part, long long rows,
                                                                          int cols, long long rows_per_block) {
  __shared__ float red[COLSUM_LANES][32][VEC + 1];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + tx) * VEC;
  const long long r0 = blockIdx.y * rows_per_block;
  const long long r1 = (r0 + rows_per_block < rows) ? r0 + rows_per_block : rows;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.0f;
  if (col < cols) {
    const IO* base = src + col;
    long long r = r0 + ty;
    for (; r + (COLSUM_UNROLL - 1) * COLSUM_LANES < r1; r += COLSUM_UNROLL * COLSUM_LANES) {
      typename Vec<IO, VEC>::Raw raw[COLSUM_UNROLL];
#pragma unroll
      for (int u = 0; u < COLSUM_UNROLL; ++u) raw[u] = Vec<IO, VEC>::load_raw(base + (r + u * COLSUM_LANES) * cols);
#pragma unroll
      for (int u = 0; u < COLSUM_UNROLL; ++u) {
        float v[VEC];
        Vec<IO, VEC>::unpack(raw[u], v);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] += v[k];
      }
    }
    for (; r < r1; r += COLSUM_LANES) {
      float v[VEC];
      Vec<IO, VEC>::load(base + r * cols, v);
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[k] += v[k];
    }
  }
#pragma unroll
  for (int k = 0; k < VEC; ++k) red[ty][tx][k] = acc[k];
  __syncthreads();
  if (ty == 0 && col < cols) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float t = red[0][tx][k];
#pragma unroll
      for (int l = 1; l < COLSUM_LANES; ++l) t += red[l][tx][k];
      part[static_cast<size_t>(blockIdx.y) * cols + col + k] = t;
    }
  }
}

__global__ void __launch_bounds__(32 * COLSUM_LANES) colsum_fold_kernel(const float* __restrict__ part,
                                                                       float* __restrict__ out, int nrow, int cols) {
  __shared__ float red[COLSUM_LANES][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + tx;
  float acc = 0.0f;
  if (col < cols)
    for (int r = ty; r < nrow; r += COLSUM_LANES) acc += part[static_cast<size_t>(r) * cols + col];
  red[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && col < cols) {
    float t = red[0][tx];
#pragma unroll
    for (int l = 1; l < COLSUM_LANES; ++l) t += red[l][tx];
    out[col] = t;
  }
}

// Row blocks of a column-sum call: enough CTAs for four per SM, at least 64 rows each.
int colsum_row_blocks(long long rows, int cols) {
  const long long tiles = (cols + 255) / 256 > 0 ? (cols + 255) / 256 : 1;
  long long want = (4 * 148 + tiles - 1) / tiles;
  const long long most = (rows + 63) / 64;
  if (want > most) want = most;
  if (want < 1) want = 1;
  if (want > 65535) want = 65535;
  return static_cast<int>(want);
}

template <typename IO>
static cudaError_t column_sums_t(const void* src, float* out, float* part, long long rows, int cols, bool vector_ok,
                                 cudaStream_t s) {
  constexpr int V = vec_width<IO>();
  const int nblk = colsum_row_blocks(rows, cols);
  const long long per = (rows + nblk - 1) / nblk;
  const IO* p = static_cast<const IO*>(src);
  if (vector_ok) {
    const dim3 grid(static_cast<unsigned>((cols / V + 31) / 32), static_cast<unsigned>(nblk));
    colsum_partial_kernel<IO, V><<<grid, 32 * COLSUM_LANES, 0, s>>>(p, part, rows, cols, per);
  } else {
    const dim3 grid(static_cast<unsigned>((cols + 31) / 32), static_cast<unsigned>(nblk));
    colsum_partial_kernel<IO, 1><<<grid, 32 * COLSUM_LANES, 0, s>>>(p, part, rows, cols, per);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  colsum_fold_kernel<<<(cols + 31) / 32, 32 * COLSUM_LANES, 0, s>>>(part, out, nblk, cols);
  return cudaGetLastError();
}

cudaError_t launch_column_sums(bool bf16, const void* src, float* out, float* part, long long rows, int cols,
                               bool vector_ok, cudaStream_t s) {
  return bf16 ? column_sums_t<__nv_bfloat16>(src, out, part, rows, cols, vector_ok, s)
              : column_sums_t<float>(src, out, part, rows, cols, vector_ok, s);
}

// ---------------------------------------------------------------- decode
template <typename IO, int VEC>
__global__ void __launch_bounds__(256) decode_conv_kernel(const IO* __restrict__ xin, const float* __restrict__ w,
                                                          const float* __restrict__ bias, IO* __restrict__ state,
                                                          const uint8_t* __restrict__ tok, IO* __restrict__ out, int B,
                                                          int D) {
  const int nvec = D / VEC;
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<long long>(B) * nvec) return;
  const int b = static_cast<int>(gid / nvec);
  const int d = static_cast<int>(gid % nvec) * VEC;
  const uint32_t f = tok ? tok[b] : 0u;
  float cur[VEC], s0[VEC], s1[VEC], s2[VEC], acc[VEC];
  IO* st = state + static_cast<size_t>(b) * 3 * D + d;
  Vec<IO, VEC>::load(xin + static_cast<size_t>(b) * D + d, cur);
  Vec<IO, VEC>::load(st, s0);
  Vec<IO, VEC>::load(st + D, s1);
  Vec<IO, VEC>::load(st + 2 * static_cast<size_t>(D), s2);
  const int reach = 3 - static_cast<int>(f & TOK_CUT_MASK);
  const bool inactive = (f & TOK_INACTIVE) != 0;
  const bool wipe = (f & TOK_ZERO_HISTORY) != 0;
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    float a = fmaf(w[(d + v) * CONV_TAPS + 3], cur[v], bias ? bias[d + v] : 0.0f);
    if (reach >= 1) a = fmaf(w[(d + v) * CONV_TAPS + 2], s2[v], a);
    if (reach >= 2) a = fmaf(w[(d + v) * CONV_TAPS + 1], s1[v], a);
    if (reach >= 3) a = fmaf(w[(d + v) * CONV_TAPS + 0], s0[v], a);
    acc[v] = inactive ? 0.0f : a;
    if (wipe) { s1[v] = 0.0f; s2[v] = 0.0f; }
  }
  Vec<IO, VEC>::store(out + static_cast<size_t>(b) * D + d, acc);
  if (!inactive) {
    Vec<IO, VEC>::store(st, s1);
    Vec<IO, VEC>::store(st + D, s2);
    Vec<IO, VEC>::store(st + 2 * static_cast<size_t>(D), cur);
  }
}

// One token of the RG-LRU for every batch row.  A thread owns VEC channels of DECODE_ROWS consecutive batch
// rows: the per-channel rate c * logsigmoid(Lambda) is formed once per thread instead of once per element,
// and the loads of all its rows are in flight before the first is used.
constexpr int DECODE_ROWS = 2;

template <typename IO, int VEC>
__global__ void __launch_bounds__(256) decode_step_kernel(const IO* __restrict__ x, const IO* __restrict__ ur,
                                                          const IO* __restrict__ ui, const float* __restrict__ lambda,
                                                          float* __restrict__ h, const uint8_t* __restrict__ tok,
                                                          IO* __restrict__ y, int B, int D, float c) {
  using V = Vec<IO, VEC>;
  const int nvec = D / VEC;
  const int ngroup = (B + DECODE_ROWS - 1) / DECODE_ROWS;
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<long long>(ngroup) * nvec) return;
  const int b0 = static_cast<int>(gid / nvec) * DECODE_ROWS;
  const int d = static_cast<int>(gid % nvec) * VEC;

  typename V::Raw xr[DECODE_ROWS], rr[DECODE_ROWS], ir[DECODE_ROWS];
  float hv[DECODE_ROWS][VEC];
  uint32_t fl[DECODE_ROWS];
#pragma unroll
  for (int q = 0; q < DECODE_ROWS; ++q) {
    const int b = b0 + q;
    fl[q] = 0u;
    if (b < B) {
      const size_t at = static_cast<size_t>(b) * D + d;
      xr[q] = V::load_raw(x + at);
      rr[q] = V::load_raw(ur + at);
      ir[q] = V::load_raw(ui + at);
      if (tok) fl[q] = tok[b];
      if constexpr (VEC == 1) {
        hv[q][0] = h[at];
      } else {
#pragma unroll
        for (int v = 0; v < VEC; v += 4) {
          const float4 t4 = *reinterpret_cast<const float4*>(h + at + v);
          hv[q][v] = t4.x; hv[q][v + 1] = t4.y; hv[q][v + 2] = t4.z; hv[q][v + 3] = t4.w;
        }
      }
    }
  }
  float rate[VEC];   // K = -c * logsigmoid(Lambda) >= 0
  float kmax = 0.0f;
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    const float lam = lambda[d + v];
    rate[v] = c * (lam >= 0.0f ? log1pf(__expf(-lam)) : log1pf(__expf(lam)) - lam);
    kmax = fmaxf(kmax, rate[v]);
  }
  const bool poly = kmax <= -POLY_RANGE;   // every r * K of this thread lies in the polynomial's range
#pragma unroll
  for (int q = 0; q < DECODE_ROWS; ++q) {
    const int b = b0 + q;
    if (b >= B) break;
    const size_t at = static_cast<size_t>(b) * D + d;
    const uint32_t f = fl[q];
    const float keep = (f & TOK_RESET) ? 0.0f : 1.0f;
    const float live = (f & TOK_INACTIVE) ? 0.0f : 1.0f;
    float xv[VEC], rv[VEC], iv[VEC], yv[VEC];
    V::unpack(xr[q], xv);
    V::unpack(rr[q], rv);
    V::unpack(ir[q], iv);
    if constexpr (VEC == 1) {
      float r, i;
      sigmoid_pair(rv[0], iv[0], r, i);
      const float em = expm1_nonpos<false>(-r * rate[0]);
      float a = 1.0f + em;
      float gam = sqrt_approx(fmaxf(-em * (2.0f + em), 0.0f));
      a = a * keep * live + (1.0f - live);
      gam = (gam * keep + (1.0f - keep)) * live;
      hv[q][0] = fmaf(a, hv[q][0], gam * i * xv[0]);
      yv[0] = hv[q][0];
    } else {
      // the arithmetic of the scan kernels' forward (same helpers, so prefill and decode agree to rounding)
#pragma unroll
      for (int v = 0; v < VEC; v += 2) {
        const float2 x2 = make_float2(xv[v], xv[v + 1]);
        const float2 K2 = make_float2(rate[v], rate[v + 1]);
        float2 r, i;
        sigmoid_pair2<sizeof(IO) == 2>(make_float2(rv[v], rv[v + 1]), make_float2(iv[v], iv[v + 1]), r, i);
        const float2 y2 = mul2(r, K2);
        const float2 e = poly ? one_minus_exp_neg2<true, sizeof(IO) == 2>(y2) : one_minus_exp_neg2<false, sizeof(IO) == 2>(y2);
        float2 a = fma2(e, f2(-1.0f), f2(1.0f));
        const float2 gq = add2(mul2(e, fma2(e, f2(-1.0f), f2(2.0f))), f2(1e-30f));
        float2 gam = mul2(gq, make_float2(rsqrt_approx(gq.x), rsqrt_approx(gq.y)));
        if (f) {
          a = fma2(mul2(a, f2(keep)), f2(live), f2(1.0f - live));
          gam = mul2(fma2(gam, f2(keep), f2(1.0f - keep)), f2(live));
        }
        const float2 h2 = fma2(a, make_float2(hv[q][v], hv[q][v + 1]), mul2(mul2(gam, i), x2));
        hv[q][v] = h2.x; hv[q][v + 1] = h2.y;
        yv[v] = h2.x; yv[v + 1] = h2.y;
      }
    }
    V::store(y + at, yv);
    if constexpr (VEC == 1) {
      h[at] = hv[q][0];
    } else {
#pragma unroll
      for (int v = 0; v < VEC; v += 4)
        *reinterpret_cast<float4*>(h + at + v) = make_float4(hv[q][v], hv[q][v + 1], hv[q][v + 2], hv[q][v + 3]);
    }
  }
}

// ---------------------------------------------------------------- launchers
constexpr int CONV_RUN = 32;

template <typename IO>
static cudaError_t conv_fwd_t(const ConvArgs& a, cudaStream_t s) {
  constexpr int V = CONV_VEC;
  const bool vec_ok = a.vector_ok;
  const int nvec = vec_ok ? a.D / V : a.D;
  const int nrun = (a.T + CONV_RUN - 1) / CONV_RUN;
  const long long total = static_cast<long long>(a.B) * nrun * nvec;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  const IO* xin = static_cast<const IO*>(a.x_in);
  const IO* st = static_cast<const IO*>(a.state);
  IO* out = static_cast<IO*>(a.out);
  cudaError_t e;
  if (a.maps) {   // enough (row, channel-tile) pairs to fill the machine: the TMA-staged kernel
    ConvTmaArgs t = {};
    t.w = a.w; t.bias = a.bias; t.state = a.state; t.tok = a.tok; t.B = a.B; t.T = a.T; t.D = a.D; t.status = a.status;
    e = launch_conv_tma_fwd(sizeof(IO) == 2, *a.maps, t, s);
  } else {
    if (vec_ok) conv_fwd_kernel<IO, V, CONV_RUN><<<blocks, 256, 0, s>>>(xin, a.w, a.bias, st, a.tok, out, a.B, a.T, a.D);
    else conv_fwd_kernel<IO, 1, CONV_RUN><<<blocks, 256, 0, s>>>(xin, a.w, a.bias, st, a.tok, out, a.B, a.T, a.D);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess || !a.new_state) return e;
  dim3 grid((a.D + 255) / 256, a.B);
  conv_state_kernel<IO><<<grid, 256, 0, s>>>(xin, st, a.tok, static_cast<IO*>(a.new_state), a.T, a.D);
  return cudaGetLastError();
}

cudaError_t launch_conv_fwd(bool bf16, const ConvArgs& a, cudaStream_t s) {
  return bf16 ? conv_fwd_t<__nv_bfloat16>(a, s) : conv_fwd_t<float>(a, s);
}

int conv_bwd_partial_rows(int B, int T) { return B * ((T + 8 * CONV_RUN - 1) / (8 * CONV_RUN)); }

template <typename IO>
static cudaError_t conv_bwd_t(const ConvBwdArgs& a, cudaStream_t s) {
  constexpr int V = CONV_VEC;
  const bool vec_ok = a.vector_ok;
  const int nvec = vec_ok ? a.D / V : a.D;
  const int tblocks = (a.T + 8 * CONV_RUN - 1) / (8 * CONV_RUN);
  dim3 grid((nvec + 31) / 32, tblocks, a.B);
  const IO* dc = static_cast<const IO*>(a.d_conv);
  const IO* xin = static_cast<const IO*>(a.x_in);
  const IO* st = static_cast<const IO*>(a.state);
  IO* dx = static_cast<IO*>(a.dx_in);
  IO* ds = static_cast<IO*>(a.d_state);
  cudaError_t e;
  int part_rows = a.B * tblocks;
  if (a.maps) {   // the TMA-staged kernel leaves one partial row per batch row
    ConvTmaArgs t = {};
    t.w = a.w; t.state = a.state; t.tok = a.tok; t.d_state = a.d_state; t.part = a.part;
    t.B = a.B; t.T = a.T; t.D = a.D; t.status = a.status;
    e = launch_conv_tma_bwd(sizeof(IO) == 2, *a.maps, t, s);
    part_rows = a.B;
  } else {
    if (vec_ok) conv_bwd_kernel<IO, V, CONV_RUN><<<grid, 256, 0, s>>>(dc, xin, a.w, st, a.tok, dx, ds, a.part, a.B, a.T, a.D);
    else conv_bwd_kernel<IO, 1, CONV_RUN><<<grid, 256, 0, s>>>(dc, xin, a.w, st, a.tok, dx, ds, a.part, a.B, a.T, a.D);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return e;
  conv_bwd_reduce_kernel<<<(5 * a.D + 255) / 256, 256, 0, s>>>(a.part, a.d_w, a.d_b, part_rows, a.D);
  return cudaGetLastError();
}

cudaError_t launch_conv_bwd(bool bf16, const ConvBwdArgs& a, cudaStream_t s) {
  return bf16 ? conv_bwd_t<__nv_bfloat16>(a, s) : conv_bwd_t<float>(a, s);
}

template <typename IO>
static cudaError_t decode_conv_t(const ConvArgs& a, cudaStream_t s) {
  constexpr int V = vec_width<IO>();
  const int nvec = a.vector_ok ? a.D / V : a.D;
  const long long total = static_cast<long long>(a.B) * nvec;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  const IO* xin = static_cast<const IO*>(a.x_in);
  IO* st = static_cast<IO*>(a.new_state);
  IO* out = static_cast<IO*>(a.out);
  if (a.vector_ok) decode_conv_kernel<IO, V><<<blocks, 256, 0, s>>>(xin, a.w, a.bias, st, a.tok, out, a.B, a.D);
  else decode_conv_kernel<IO, 1><<<blocks, 256, 0, s>>>(xin, a.w, a.bias, st, a.tok, out, a.B, a.D);
  return cudaGetLastError();
}

cudaError_t launch_decode_conv(bool bf16, const ConvArgs& a, cudaStream_t s) {
  return bf16 ? decode_conv_t<__nv_bfloat16>(a, s) : decode_conv_t<float>(a, s);
}

template <typename IO>
static cudaError_t decode_step_t(const DecodeArgs& a, cudaStream_t s) {
  constexpr int V = vec_width<IO>();
  const int nvec = a.vector_ok ? a.D / V : a.D;
  const long long total = static_cast<long long>((a.B + DECODE_ROWS - 1) / DECODE_ROWS) * nvec;
  const unsigned blocks = static_cast<unsigned>((total + 127) / 128);   // small blocks: an even spread over the SMs
  const IO* x = static_cast<const IO*>(a.x);
  const IO* ur = static_cast<const IO*>(a.ur);
  const IO* ui = static_cast<const IO*>(a.ui);
  IO* y = static_cast<IO*>(a.y);
  if (a.vector_ok) decode_step_kernel<IO, V><<<blocks, 128, 0, s>>>(x, ur, ui, a.lambda, a.h, a.tok, y, a.B, a.D, a.c);
  else decode_step_kernel<IO, 1><<<blocks, 128, 0, s>>>(x, ur, ui, a.lambda, a.h, a.tok, y, a.B, a.D, a.c);
  return cudaGetLastError();
}

cudaError_t launch_decode_step(bool bf16, const DecodeArgs& a, cudaStream_t s) {
  return bf16 ? decode_step_t<__nv_bfloat16>(a, s) : decode_step_t<float>(a, s);
}

}  // namespace rglru
