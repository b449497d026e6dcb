// rglru_conv_bwd_noalloc: the conv backward for callers that must not allocate device memory.
//
// rglru_conv_bwd needs scratch for its per-block partial sums of d_w / d_b and asks the caller for
// it.  Some callers cannot provide any: code running inside a region where the allocator must not be
// entered (a serving loop with a frozen memory plan, a plugin hosted by a runtime that owns all
// device memory and hands out none, a callback where cudaMalloc would synchronise the device).  For
// them this entry point keeps the scratch in a fixed array that is part of the library image.
//
// Cost and limits: the array occupies kScratchFloats * 4 bytes on every GPU on which the library's
// device code gets loaded, until process exit.  With CUDA's lazy module loading (the default) that
// happens at the first use on a device -- the first call of this entry point resolves the array's
// address and loads the kernels, which may itself allocate and synchronise -- so a host with a
// no-allocation region makes ONE warm-up call per device before entering it (and before any stream
// capture).  Larger problems are refused with RGLRU_ERR_TOO_LARGE.  All calls share the one array, so
// two calls whose kernels can overlap on the GPU (different streams) race on it; calls on one stream
// are safe.  The scratch address belongs to the device that is current at the call, so `stream` must
// be a stream of that device.  This entry point always runs the kernels that split the time axis
// (one thread per run of 32 steps); it never takes the TMA-staged kernels that rglru_conv_bwd may
// choose for large batches, so the two can differ in speed, not in results beyond rounding.

#include <mutex>

#include "../../include/rglru_b200.h"
#include "rglru_internal.h"

namespace rglru {

// 4 MiB of fp32 partial sums: enough for B * ceil(T / 256) * 5 * D <= 1,048,576,
// e.g. B = 16, T = 2048, D = 1024 (655,360) or B = 8, T = 4096, D = 1536 (983,040).
constexpr size_t kScratchFloats = size_t(1) << 20;
static __device__ __align__(256) float g_conv_bwd_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
static std::mutex g_noalloc_mutex;
static float* g_scratch_ptr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; kernels need its device address, which differs per
// device.  Resolve it once per device, with that device current.
static int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (dev < 0 || dev >= kMaxDevices) return RGLRU_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_scratch_ptr[dev]) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (major != 10) return RGLRU_ERR_UNSUPPORTED;
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_conv_bwd_scratch);
    if (e != cudaSuccess || !ptr) return record_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return RGLRU_OK;
}

}  // namespace rglru

using namespace rglru;

extern "C" {

size_t rglru_conv_bwd_noalloc_max_bytes(void) { return kScratchFloats * sizeof(float); }

int rglru_conv_bwd_noalloc(const void* d_conv, const void* x_in, const float* conv_w, const void* conv_state,
                           const uint8_t* tok, void* dx_in, float* d_w, float* d_b, void* d_state, int B, int T,
                           int D, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!d_conv || !x_in || !conv_w || !dx_in || !d_w) return RGLRU_ERR_NULL_POINTER;
  if (B <= 0 || T <= 0 || D <= 0 || B > 65535) return RGLRU_ERR_BAD_SHAPE;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  auto aligned = [](const void* p, size_t n) { return reinterpret_cast<uintptr_t>(p) % n == 0; };
  if (!aligned(d_conv, es) || !aligned(x_in, es) || !aligned(dx_in, es) || !aligned(conv_state, es) ||
      !aligned(d_state, es) || !aligned(conv_w, 4) || !aligned(d_w, 4) || !aligned(d_b, 4))
    return RGLRU_ERR_MISALIGNED;
  // The same size rglru_conv_bwd_workspace_bytes reports, held against the fixed array.
  const size_t need = static_cast<size_t>(conv_bwd_partial_rows(B, T)) * 5 * static_cast<size_t>(D);
  if (need > kScratchFloats) return RGLRU_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != RGLRU_OK) return rc;

  // Nothing in the scratch has to start at zero: the backward kernel writes every partial-sum entry
  // that the reduction kernel of the same call then reads, so stale contents of an earlier call are
  // never observed.
  ConvBwdArgs a = {};
  a.d_conv = d_conv; a.x_in = x_in; a.w = conv_w; a.state = conv_state; a.tok = tok; a.dx_in = dx_in;
  a.d_w = d_w; a.d_b = d_b; a.d_state = d_state; a.part = scratch;
  a.B = B; a.T = T; a.D = D;
  a.vector_ok = (static_cast<size_t>(D) * es) % 16 == 0 && aligned(d_conv, 16) && aligned(x_in, 16) &&
                aligned(dx_in, 16) && aligned(conv_state, 16) && aligned(d_state, 16) && aligned(conv_w, 16);
  const cudaError_t e = launch_conv_bwd(bf16, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : record_cuda_error(e);
}

}  // extern "C"
