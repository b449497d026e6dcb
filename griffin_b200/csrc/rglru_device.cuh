// Device-side building blocks shared by the RG-LRU kernels: PTX wrappers for
// mbarrier / TMA (cp.async.bulk.tensor), fast-math primitives, the gate
// arithmetic, and packed I/O conversion.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rglru {

// ---------------------------------------------------------------- geometry
// One CTA owns CH adjacent channels of one batch row for the whole sequence.
// Its threads form a grid of LANES time-lanes x NCV channel-vectors; a
// thread handles CV adjacent channels over TS consecutive time-steps of each
// chunk, so one chunk covers LANES*TS time-steps.
// CH (32 or 64) and LANES are template parameters of the scan kernels.
constexpr int CV = 4;
// LANES (16 or 32 time-lanes per chunk) is a template parameter of the scan kernels;
// the CTA has LANES * NCV threads.

constexpr float LOG2E = 1.4426950408889634f;
constexpr float SLOPE_CAP = 1000.0f;  // bound on d sqrt / d gamma^2
// Channels whose c*logsigmoid(Lambda) is above this use a polynomial expm1.
constexpr float POLY_RANGE = -0.25f;

// Codes written to the device status word.
constexpr int DEV_TIMEOUT_LOAD = 1;   // a tile load never completed
constexpr int DEV_TIMEOUT_STORE = 2;  // the producer never saw a chunk's results
constexpr int DEV_TIMEOUT_SELFTEST = 3;  // the wait self-test (a barrier nothing completes) gave up, as it must
constexpr long long DEV_WAIT_CYCLES = 4000000000LL;   // about two seconds of SM clock

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about two seconds of SM clock and reports false.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < 256; ++spin)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - start > 4000000000LL) return false;
  }
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Wait used inside the pipelined kernels.  Once any thread of the CTA has seen a wait
// expire, `dead` is set and every later wait returns at once, so all threads keep
// executing the same barriers and the kernel runs to its end (producing garbage) with
// the device status word set, instead of hanging or leaving barriers unmatched.
__device__ __forceinline__ void mbar_wait_or_flag(uint64_t* bar, uint32_t parity, volatile int* dead, int* status,
                                                  int code, long long limit = DEV_WAIT_CYCLES) {
  if (mbar_try_wait(bar, parity)) return;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < 128; ++spin)
      if (mbar_try_wait(bar, parity)) return;
    if (*dead) return;
    if (clock64() - start > limit) {
      *dead = 1;
      atomicExch(status, code);
      return;
    }
  }
}
// Named barrier 1: the compute warps of a CTA (the TMA producer warp does not take part).
__device__ __forceinline__ void bar_compute(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}
// Named barrier 3: the threads that share the level-two chain of a chunk.
__device__ __forceinline__ void bar_chain(int nthreads) {
  asm volatile("bar.sync 3, %0;" ::"r"(nthreads) : "memory");
}
// Barrier 1 with an AND vote over its `nthreads` participants.
__device__ __forceinline__ bool bar_compute_and(int nthreads, bool pred) {
  uint32_t all;
  asm volatile(
      "{\n"
      " .reg .pred pin, pout;\n"
      " setp.ne.u32 pin, %2, 0;\n"
      " bar.red.and.pred pout, 1, %1, pin;\n"
      " selp.u32 %0, 1, 0, pout;\n"
      "}\n"
      : "=r"(all)
      : "r"(nthreads), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return all != 0;
}
// Named barrier 2: compute warps and the producer warp together (nthreads counts all of them).
__device__ __forceinline__ void bar_all(int nthreads) {
  __syncwarp();
  asm volatile("bar.sync 2, %0;" ::"r"(nthreads) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const void* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* map, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// Ask the copy engine to bring a tile into L2 without waiting for it and without touching shared memory.  A
// prefetch changes no data, so it may be issued before pdl_wait: if the preceding kernel is still writing the
// tensor, its writes land in the same L2 and nothing stale is ever read.
__device__ __forceinline__ void tma_prefetch_3d(const void* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// 5-D forms, for tensor maps that view the time axis as (eighth, half, step) so that a tile lands in shared
// memory with rows t and t + 4 side by side in one 128-byte line (see the paired forward tiles).
__device__ __forceinline__ void tma_load_5d(void* dst, const void* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4),
        "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_5d(const void* map, const void* src, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_5d(const void* map, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.prefetch.tensor.5d.L2.global.tile [%0, {%1, %2, %3, %4, %5}];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void prefetch_map(const void* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Programmatic dependent launch: `pdl_launch_dependents` lets the next kernel on the stream begin its
// launch and prologue while this grid is still running; `pdl_wait` (in that next kernel) returns once
// the preceding grid has completed and its writes are visible.  Every global access of a kernel
// launched with the attribute must come after pdl_wait.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------- fast math
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------- packed fp32 (two lanes per instruction)
// sm_100 executes add/mul/fma on a pair of fp32 values in one issue slot (the FMA pipe is busy two cycles
// for it, so lane throughput is unchanged; what is saved is instruction issue and dependency tracking), so
// all channel arithmetic is written on float2 pairs.
__device__ __forceinline__ float2 f2(float a) { return make_float2(a, a); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// r = sigmoid(ur), i = sigmoid(ui) for two channels.
//   HALF_IO = false: exp2 + one shared reciprocal, about 1e-7 relative (three MUFU operations per element).
//   HALF_IO = true : 0.5 + 0.5 tanh(u / 2) on the hardware tanh (two MUFU operations per element); its
//                    absolute error of 2.5e-4 is a sixteenth of the bf16 quantum of the tensors it feeds.
template <bool HALF_IO>
__device__ __forceinline__ void sigmoid_pair2(float2 ur, float2 ui, float2& r, float2& i) {
  if (HALF_IO) {
    const float2 hr = mul2(ur, f2(0.5f));
    const float2 hi = mul2(ui, f2(0.5f));
    r = fma2(make_float2(tanh_approx(hr.x), tanh_approx(hr.y)), f2(0.5f), f2(0.5f));
    i = fma2(make_float2(tanh_approx(hi.x), tanh_approx(hi.y)), f2(0.5f), f2(0.5f));
    return;
  }
  float2 tr = mul2(ur, f2(-LOG2E));
  float2 ti = mul2(ui, f2(-LOG2E));
  const float2 er = make_float2(ex2_approx(fminf(tr.x, 60.0f)), ex2_approx(fminf(tr.y, 60.0f)));
  const float2 ei = make_float2(ex2_approx(fminf(ti.x, 60.0f)), ex2_approx(fminf(ti.y, 60.0f)));
  const float2 dr = add2(er, f2(1.0f));
  const float2 di = add2(ei, f2(1.0f));
  const float2 d = mul2(dr, di);
  const float2 inv = make_float2(rcp_approx(d.x), rcp_approx(d.y));
  r = mul2(inv, di);
  i = mul2(inv, dr);
}

// The same with a per-channel bias added to each pre-activation.  The biases arrive pre-scaled by the
// factor the sigmoid applies to its argument (0.5 for HALF_IO, -log2 e otherwise; see gate_bias_scale), so
// the addition rides on the multiply that is there anyway.
template <bool HALF_IO>
__device__ __forceinline__ float gate_bias_scale() { return HALF_IO ? 0.5f : -LOG2E; }
template <bool HALF_IO>
__device__ __forceinline__ void sigmoid_pair2_biased(float2 ur, float2 ui, float2 br, float2 bi, float2& r, float2& i) {
  if (HALF_IO) {
    const float2 hr = fma2(ur, f2(0.5f), br);
    const float2 hi = fma2(ui, f2(0.5f), bi);
    r = fma2(make_float2(tanh_approx(hr.x), tanh_approx(hr.y)), f2(0.5f), f2(0.5f));
    i = fma2(make_float2(tanh_approx(hi.x), tanh_approx(hi.y)), f2(0.5f), f2(0.5f));
    return;
  }
  float2 tr = fma2(ur, f2(-LOG2E), br);
  float2 ti = fma2(ui, f2(-LOG2E), bi);
  const float2 er = make_float2(ex2_approx(fminf(tr.x, 60.0f)), ex2_approx(fminf(tr.y, 60.0f)));
  const float2 ei = make_float2(ex2_approx(fminf(ti.x, 60.0f)), ex2_approx(fminf(ti.y, 60.0f)));
  const float2 dr = add2(er, f2(1.0f));
  const float2 di = add2(ei, f2(1.0f));
  const float2 d = mul2(dr, di);
  const float2 inv = make_float2(rcp_approx(d.x), rcp_approx(d.y));
  r = mul2(inv, di);
  i = mul2(inv, dr);
}

// GeLU in its tanh form (griffin/griffin.py:464 of the reference): gelu(v) = v * s with
// s = sigmoid(2 z) = (1 + tanh z) / 2 and z = k0 v (1 + k1 v^2).  Returns s; precision as sigmoid_pair2.
constexpr float GELU_K0 = 0.7978845608028654f;   // sqrt(2 / pi)
constexpr float GELU_K1 = 0.044715f;
template <bool HALF_IO>
__device__ __forceinline__ float2 gelu_sigmoid2(float2 v) {
  const float2 z = mul2(mul2(v, f2(GELU_K0)), fma2(mul2(v, v), f2(GELU_K1), f2(1.0f)));
  if (HALF_IO) return fma2(make_float2(tanh_approx(z.x), tanh_approx(z.y)), f2(0.5f), f2(0.5f));
  const float2 t = mul2(z, f2(-2.0f * LOG2E));
  const float2 d = add2(make_float2(ex2_approx(fminf(t.x, 60.0f)), ex2_approx(fminf(t.y, 60.0f))), f2(1.0f));
  return make_float2(rcp_approx(d.x), rcp_approx(d.y));
}
// d gelu / d v = s + v s (1 - s) * 2 z',  2 z' = 2 k0 (1 + 3 k1 v^2)
__device__ __forceinline__ float2 gelu_slope2(float2 v, float2 s) {
  const float2 zp = fma2(mul2(v, v), f2(6.0f * GELU_K0 * GELU_K1), f2(2.0f * GELU_K0));
  return fma2(mul2(mul2(v, s), fma2(s, f2(-1.0f), f2(1.0f))), zp, s);
}

// E(y) = 1 - exp(-y) for y >= 0 (y = -c r logsigmoid(Lambda)), so that the decay is
// a = 1 - E and gamma^2 = 1 - a^2 = E (2 - E) without cancellation.
//   POLY: y is known to lie in [0, -POLY_RANGE]; alternating Taylor series, degree 6 (truncation < 5e-8
//         relative) for fp32 tensors, degree 4 (< 4e-5, a hundredth of the bf16 quantum) for bf16 tensors.
//   otherwise: the polynomial where valid, 1 - 2^(-y log2 e) elsewhere (chosen per element).
template <bool POLY, bool HALF_IO = false>
__device__ __forceinline__ float2 one_minus_exp_neg2(float2 y) {
  float2 t;
  if (HALF_IO) {
    t = fma2(y, f2(-1.0f / 24.0f), f2(1.0f / 6.0f));
  } else {
    t = fma2(y, f2(-1.0f / 720.0f), f2(1.0f / 120.0f));
    t = fma2(t, y, f2(-1.0f / 24.0f));
    t = fma2(t, y, f2(1.0f / 6.0f));
  }
  t = fma2(t, y, f2(-0.5f));
  float2 e = fma2(mul2(y, y), t, y);
  if (!POLY) {
    const float wx = 1.0f - ex2_approx(-LOG2E * y.x);
    const float wy = 1.0f - ex2_approx(-LOG2E * y.y);
    e.x = y.x < -POLY_RANGE ? e.x : wx;
    e.y = y.y < -POLY_RANGE ? e.y : wy;
  }
  return e;
}

// Both gate sigmoids with one reciprocal: 1/((1+er)(1+ei)) scaled by the other
// factor.  The exponent clamp keeps the product finite (sigmoid saturates at
// 2^-60, far below fp32 resolution of anything it multiplies).
__device__ __forceinline__ void sigmoid_pair(float ur, float ui, float& r, float& i) {
  const float er = ex2_approx(fminf(-LOG2E * ur, 60.0f));
  const float ei = ex2_approx(fminf(-LOG2E * ui, 60.0f));
  const float dr = 1.0f + er;
  const float di = 1.0f + ei;
  const float inv = rcp_approx(dr * di);
  r = inv * di;
  i = inv * dr;
}

// expm1(z) for z <= 0 with full relative accuracy.
//   POLY: z is known to lie in [POLY_RANGE, 0]; degree-6 Taylor, truncation < 5e-8 relative.
//   otherwise: the polynomial where it is valid, 2^(z log2 e) - 1 elsewhere.
template <bool POLY>
__device__ __forceinline__ float expm1_nonpos(float z) {
  float t = fmaf(z, 1.0f / 720.0f, 1.0f / 120.0f);
  t = fmaf(t, z, 1.0f / 24.0f);
  t = fmaf(t, z, 1.0f / 6.0f);
  t = fmaf(t, z, 0.5f);
  const float poly = fmaf(z * z, t, z);
  if (POLY) return poly;
  const float wide = ex2_approx(z * LOG2E) - 1.0f;
  return z > POLY_RANGE ? poly : wide;
}

// ---------------------------------------------------------------- packed I/O
template <typename IO>
struct Pack;

template <>
struct Pack<float> {
  static constexpr int BYTES = 16;
  using Raw = float4;
  static __device__ __forceinline__ Raw load(const void* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void unpack(const Raw& r, float (&v)[4]) {
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  static __device__ __forceinline__ void store(void* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  static __device__ __forceinline__ void unpack2(const Raw& r, float2 (&v)[2]) {
    v[0] = make_float2(r.x, r.y);
    v[1] = make_float2(r.z, r.w);
  }
  static __device__ __forceinline__ Raw pack2(const float2 (&v)[2]) { return make_float4(v[0].x, v[0].y, v[1].x, v[1].y); }
  static __device__ __forceinline__ void store_raw(void* p, const Raw& r) { *reinterpret_cast<float4*>(p) = r; }
  static __device__ __forceinline__ void store2(void* p, const float2 (&v)[2]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
  }
  static __device__ __forceinline__ float to_float(float x) { return x; }
  static __device__ __forceinline__ float from_float(float x) { return x; }
};

template <>
struct Pack<__nv_bfloat16> {
  static constexpr int BYTES = 8;
  using Raw = uint2;
  static __device__ __forceinline__ Raw load(const void* p) { return *reinterpret_cast<const uint2*>(p); }
  static __device__ __forceinline__ void unpack(const Raw& r, float (&v)[4]) {
    v[0] = __uint_as_float(r.x << 16);
    v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16);
    v[3] = __uint_as_float(r.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(void* p, const float (&v)[4]) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
  }
  static __device__ __forceinline__ void unpack2(const Raw& r, float2 (&v)[2]) {
    v[0] = make_float2(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u));
    v[1] = make_float2(__uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
  }
  static __device__ __forceinline__ Raw pack2(const float2 (&v)[2]) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0].x, v[0].y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v[1].x, v[1].y);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    return raw;
  }
  static __device__ __forceinline__ void store_raw(void* p, const Raw& r) { *reinterpret_cast<uint2*>(p) = r; }
  static __device__ __forceinline__ void store2(void* p, const float2 (&v)[2]) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0].x, v[0].y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v[1].x, v[1].y);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

// Token flag bits (mirrors include/rglru_b200.h).
constexpr uint32_t TOK_CUT_MASK = 0x03u;
constexpr uint32_t TOK_RESET = 0x04u;
constexpr uint32_t TOK_INACTIVE = 0x08u;
constexpr uint32_t TOK_ZERO_HISTORY = 0x10u;

}  // namespace rglru
