// extern "C" surface of librglru_b200.so: argument validation, tensor-map
// construction, and dispatch to the kernel launchers.  Declarations and the
// reference lines each entry point replaces are in include/rglru_b200.h.

#include <mutex>

#include "../../include/rglru_b200.h"
#include "rglru_device.cuh"
#include "rglru_internal.h"

namespace rglru {

__device__ int g_device_status = 0;

static thread_local cudaError_t t_last_cuda = cudaSuccess;

static int fail_cuda(cudaError_t e) {
  t_last_cuda = e;
  return RGLRU_ERR_LAUNCH;
}
int record_cuda_error(cudaError_t e) { return fail_cuda(e); }

constexpr int MAX_DEVICES = 64;
static std::mutex g_mutex;
static int* g_status_ptr[MAX_DEVICES] = {nullptr};
static int g_arch_ok[MAX_DEVICES] = {0};  // 0 unknown, 1 sm_100, -1 other

// Device address of the status word and architecture check, once per device.
static int device_setup(int** status) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e);
  if (dev < 0 || dev >= MAX_DEVICES) return RGLRU_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_arch_ok[dev] == 0) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return fail_cuda(e);
    g_arch_ok[dev] = (major == 10) ? 1 : -1;
    if (g_arch_ok[dev] == 1) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_device_status);
      if (e != cudaSuccess) { g_arch_ok[dev] = 0; return fail_cuda(e); }
      g_status_ptr[dev] = static_cast<int*>(p);
    }
  }
  if (g_arch_ok[dev] != 1) return RGLRU_ERR_UNSUPPORTED;
  *status = g_status_ptr[dev];
  return RGLRU_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 3-D map over a dense [B, T, D] tensor with a [1, rows, cols] box; out-of-range parts
// of a box read as zero and are dropped on store.
static bool encode_map(CUtensorMap* map, const void* base, bool bf16, int B, int T, int D, int rows, int cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const size_t es = bf16 ? 2 : 4;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * es, static_cast<cuuint64_t>(D) * es * T};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(cols), static_cast<cuuint32_t>(rows), 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 5-D map over the same tensor for the paired-row tiles of the 32-channel forward: time is viewed as
// t = 8 q + 4 h + j and the dimensions are ordered (channel, h, j, q, batch), so that a box of
// [32 channels, 2, 4, rows / 8, 1] arrives in shared memory as [q][j][h][channel]: rows t and t + 4 side by side
// in one 128-byte line.  T must be a multiple of 8 (the caller asks for it only on whole 128-step chunks).
static bool encode_map_paired(CUtensorMap* map, const void* base, bool bf16, int B, int T, int D, int rows, int cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || T % 8 != 0 || rows % 8 != 0) return false;
  const size_t es = bf16 ? 2 : 4;
  const cuuint64_t pitch = static_cast<cuuint64_t>(D) * es;
  const cuuint64_t dims[5] = {static_cast<cuuint64_t>(D), 2u, 4u, static_cast<cuuint64_t>(T / 8), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[4] = {4 * pitch, pitch, 8 * pitch, pitch * T};
  const cuuint32_t box[5] = {static_cast<cuuint32_t>(cols), 2u, 4u, static_cast<cuuint32_t>(rows / 8), 1u};
  const cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
  const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// A tensor map is a pure function of (base address, element type, shape, box), and a training loop calls with
// the same handful of buffers step after step (the caching allocator hands the same blocks back), so encoded
// maps are kept in a small per-thread table: a hit costs a compare and a 128-byte copy instead of a driver call
// per map (seven to nine of them per backward call).
struct MapKey {
  const void* base;
  int B, T, D, rows, cols, bf16;
  bool operator==(const MapKey& o) const {
    return base == o.base && B == o.B && T == o.T && D == o.D && rows == o.rows && cols == o.cols && bf16 == o.bf16;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int MAP_CACHE_SLOTS = 256;   // direct-mapped

static bool make_map(CUtensorMap* map, const void* base, bool bf16, int B, int T, int D, int rows, int cols,
                     bool paired = false) {
  static thread_local MapSlot table[MAP_CACHE_SLOTS] = {};
  const MapKey key{base, B, T, D, paired ? -rows : rows, cols, bf16 ? 1 : 0};   // negative rows: the paired 5-D form
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 8;
  h ^= (static_cast<uint64_t>(rows) << 3) ^ (static_cast<uint64_t>(cols) << 11) ^ (static_cast<uint64_t>(D) << 17) ^
       (static_cast<uint64_t>(T) << 29) ^ (static_cast<uint64_t>(B) << 41);
  h ^= h >> 29;
  MapSlot& slot = table[(h * 0x9E3779B97F4A7C15ull) >> 56];
  if (slot.used && slot.key == key) {
    *map = slot.map;
    return true;
  }
  if (!(paired ? encode_map_paired(map, base, bf16, B, T, D, rows, cols) : encode_map(map, base, bf16, B, T, D, rows, cols)))
    return false;
  slot.key = key;
  slot.map = *map;
  slot.used = true;
  return true;
}

static bool aligned(const void* p, size_t n) { return (reinterpret_cast<uintptr_t>(p) % n) == 0; }

// TMA needs 16-byte aligned bases and row pitches, and strides below 2^40 bytes.
static bool tma_shape_ok(int T, int D, size_t es) {
  const unsigned long long pitch = static_cast<unsigned long long>(D) * es;
  return (pitch % 16 == 0) && (pitch * static_cast<unsigned long long>(T) < (1ull << 40));
}

// The TMA-staged conv kernels run one CTA per (batch row, 64-channel tile) over the whole sequence; they pay
// once those pairs fill the 148 SMs, below that the kernels that also split the time axis are used.
static bool conv_tma_pays(int B, int D) { return static_cast<long long>(B) * ((D + 63) / 64) >= 148; }

static int check_dims(int B, int T, int D) {
  if (B <= 0 || T <= 0 || D <= 0) return RGLRU_ERR_BAD_SHAPE;
  if (B > 65535) return RGLRU_ERR_BAD_SHAPE;  // batch rows map to gridDim.y
  return RGLRU_OK;
}

}  // namespace rglru

using namespace rglru;

extern "C" {

const char* rglru_status_string(int status) {
  switch (status) {
    case RGLRU_OK: return "ok";
    case RGLRU_ERR_NULL_POINTER: return "a required pointer is NULL";
    case RGLRU_ERR_BAD_DTYPE: return "unknown io_dtype";
    case RGLRU_ERR_BAD_SHAPE: return "bad shape: every dimension must be positive and B <= 65535";
    case RGLRU_ERR_MISALIGNED: return "pointer not aligned to its element size";
    case RGLRU_ERR_WORKSPACE: return "workspace missing or too small";
    case RGLRU_ERR_LAUNCH: return "CUDA launch failed";
    case RGLRU_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired";
    case RGLRU_ERR_UNSUPPORTED: return "unsupported device: CUDA kernels are built for sm_100a only";
    case RGLRU_ERR_TOO_LARGE: return "problem larger than the fixed capacity of this entry point";
    default: return "unknown status";
  }
}

const char* rglru_last_cuda_error(void) { return cudaGetErrorString(t_last_cuda); }

int rglru_abi_version(void) { return 2; }

int rglru_device_status(int* detail) {
  int* status = nullptr;
  int rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e);
  int host = 0;
  e = cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail_cuda(e);
  if (detail) *detail = host;
  if (host != 0) {
    const int zero = 0;
    cudaMemcpy(status, &zero, sizeof(int), cudaMemcpyHostToDevice);
    return RGLRU_ERR_DEVICE_TIMEOUT;
  }
  return RGLRU_OK;
}

int rglru_selftest_wait_timeout(unsigned limit_us, int* finished, void* stream) {
  if (limit_us == 0 || limit_us > 100000u) return RGLRU_ERR_BAD_SHAPE;   // at most a tenth of a second
  if (!aligned(finished, 4)) return RGLRU_ERR_MISALIGNED;
  int* status = nullptr;
  const int rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  const long long cycles = static_cast<long long>(limit_us) * 2000;         // SM clock is about 2 GHz
  const cudaError_t e = launch_wait_selftest(status, finished, cycles, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_chunk_steps(int io_dtype) {
  (void)io_dtype;
  return SAVE_EVERY;
}

size_t rglru_workspace_bytes(int B, int T, int D, int io_dtype) {
  (void)io_dtype;
  if (B <= 0 || T <= 0 || D <= 0) return 0;
  const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
  // chunk-entry states [B, nsave, D] | dLambda partial rows [B, D] | tail (completion ticket) | gate-sum partial rows [B, 2 D]
  return (static_cast<size_t>(B) * nsave * D + static_cast<size_t>(B) * D) * sizeof(float) + WS_TAIL_BYTES +
         static_cast<size_t>(B) * 2 * D * sizeof(float);
}

static int fwd_common(const void* x, const void* u_r, const void* u_i, const float* lambda, const float* h0,
                      const uint8_t* tok, void* y, float* h_last, float* decay_prod, void* ws, size_t ws_bytes, int B, int T,
                      int D, float c, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!x || !u_r || !u_i || !lambda || (!y && !decay_prod)) return RGLRU_ERR_NULL_POINTER;   // no y: carry-only call
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(x, es) || !aligned(u_r, es) || !aligned(u_i, es) || !aligned(y, es) || !aligned(lambda, 4) ||
      !aligned(h0, 4) || !aligned(h_last, 4) || !aligned(decay_prod, 4) || !aligned(ws, 4))
    return RGLRU_ERR_MISALIGNED;
  if (ws && ws_bytes < rglru_workspace_bytes(B, T, D, io_dtype)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;

  ScanFwdArgs a = {};
  a.x = x; a.ur = u_r; a.ui = u_i; a.y = y;
  a.lambda = lambda; a.h0 = h0; a.tok = tok; a.h_last = h_last; a.decay_prod = decay_prod;
  a.states = static_cast<float*>(ws);
  {
    const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
    a.ticket = ws ? reinterpret_cast<unsigned*>(static_cast<float*>(ws) + static_cast<size_t>(B) * nsave * D +
                                               static_cast<size_t>(B) * D)
                  : nullptr;
  }
  a.B = B; a.T = T; a.D = D; a.c = c; a.status = status;

  FwdMaps maps;
  bool tma = tma_shape_ok(T, D, es) && aligned(x, 16) && aligned(u_r, 16) && aligned(u_i, 16) && aligned(y, 16);
  const int variant = y ? scan_fwd_variant(B, T, D, bf16) : 0;   // the carry-only pass exists in the 64-channel shape only
  if (tma) {
    const int rows = scan_fwd_box_rows(variant), cols = scan_fwd_box_cols(variant);
    const void* yy = y ? y : x;   // without y the map is never used
    a.paired = scan_fwd_paired(variant, bf16, tok, T) && make_map(&maps.x, x, bf16, B, T, D, rows, cols, true) &&
               make_map(&maps.ur, u_r, bf16, B, T, D, rows, cols, true) &&
               make_map(&maps.ui, u_i, bf16, B, T, D, rows, cols, true) && make_map(&maps.y, yy, bf16, B, T, D, rows, cols, true);
    if (!a.paired)
      tma = make_map(&maps.x, x, bf16, B, T, D, rows, cols) && make_map(&maps.ur, u_r, bf16, B, T, D, rows, cols) &&
            make_map(&maps.ui, u_i, bf16, B, T, D, rows, cols) && make_map(&maps.y, yy, bf16, B, T, D, rows, cols);
  }
  const cudaError_t e = launch_scan_fwd(bf16, tma, variant, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_fwd(const void* x, const void* u_r, const void* u_i, const float* lambda, const float* h0,
              const uint8_t* tok, void* y, float* h_last, void* ws, size_t ws_bytes, int B, int T, int D, float c,
              int io_dtype, void* stream) {
  return fwd_common(x, u_r, u_i, lambda, h0, tok, y, h_last, nullptr, ws, ws_bytes, B, T, D, c, io_dtype, stream);
}

int rglru_fwd_carry(const void* x, const void* u_r, const void* u_i, const float* lambda, const float* h0,
                    const uint8_t* tok, void* y, float* h_last, float* decay_prod, void* ws, size_t ws_bytes, int B,
                    int T, int D, float c, int io_dtype, void* stream) {
  if (!h_last || !decay_prod) return RGLRU_ERR_NULL_POINTER;
  return fwd_common(x, u_r, u_i, lambda, h0, tok, y, h_last, decay_prod, ws, ws_bytes, B, T, D, c, io_dtype, stream);
}

int rglru_bwd(const void* dy, const float* dh_last, const void* x, const void* u_r, const void* u_i,
              const float* lambda, const float* h0, const uint8_t* tok, void* ws, size_t ws_bytes, void* dx,
              void* du_r, void* du_i, float* dlambda, float* dh0, int B, int T, int D, float c, int io_dtype,
              void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!dy || !x || !u_r || !u_i || !lambda) return RGLRU_ERR_NULL_POINTER;
  // Carry-only call: dx, du_r, du_i and dlambda all absent and dh0 present; otherwise all four are required.
  const bool carry_only = !dx && !du_r && !du_i && !dlambda && dh0;
  if (!carry_only && (!dx || !du_r || !du_i || !dlambda)) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(dy, es) || !aligned(x, es) || !aligned(u_r, es) || !aligned(u_i, es) || !aligned(dx, es) ||
      !aligned(du_r, es) || !aligned(du_i, es) || !aligned(lambda, 4) || !aligned(h0, 4) || !aligned(dh_last, 4) ||
      !aligned(dlambda, 4) || !aligned(dh0, 4) || !aligned(ws, 4))
    return RGLRU_ERR_MISALIGNED;
  if (!ws || ws_bytes < rglru_workspace_bytes(B, T, D, io_dtype)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;

  const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
  ScanBwdArgs a = {};
  a.dy = dy; a.x = x; a.ur = u_r; a.ui = u_i; a.dx = dx; a.dur = du_r; a.dui = du_i;
  a.lambda = lambda; a.h0 = h0; a.dh_last = dh_last; a.tok = tok;
  a.states = static_cast<const float*>(ws);
  a.dlam_part = static_cast<float*>(ws) + static_cast<size_t>(B) * nsave * D;
  a.dlambda = dlambda; a.dh0 = dh0;
  a.ticket = (B <= FUSED_DLAMBDA_MAX_B && !carry_only) ? reinterpret_cast<unsigned*>(a.dlam_part + static_cast<size_t>(B) * D) : nullptr;
  a.B = B; a.T = T; a.D = D; a.c = c; a.status = status;

  BwdMaps maps;
  bool tma = tma_shape_ok(T, D, es) && aligned(dy, 16) && aligned(x, 16) && aligned(u_r, 16) && aligned(u_i, 16) &&
             aligned(dx, 16) && aligned(du_r, 16) && aligned(du_i, 16);
  const int variant = scan_bwd_variant(B, T, D, bf16);
  if (tma) {
    const int rows = scan_bwd_box_rows(variant), cols = scan_bwd_box_cols(variant);
    tma = make_map(&maps.dy, dy, bf16, B, T, D, rows, cols) && make_map(&maps.x, x, bf16, B, T, D, rows, cols) &&
          make_map(&maps.ur, u_r, bf16, B, T, D, rows, cols) && make_map(&maps.ui, u_i, bf16, B, T, D, rows, cols) &&
          // (a carry-only call stores nothing: its three output maps are placeholders over the inputs)
          make_map(&maps.dx, dx ? dx : x, bf16, B, T, D, rows, cols) &&
          make_map(&maps.dur, du_r ? du_r : u_r, bf16, B, T, D, rows, cols) &&
          make_map(&maps.dui, du_i ? du_i : u_i, bf16, B, T, D, rows, cols);
  }
  const cudaError_t e = launch_scan_bwd(bf16, tma, variant, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_conv_scan_fwd(const void* x_in, const float* conv_w, const float* conv_b, const void* conv_state,
                        const void* u_r, const void* u_i, const float* lambda, const float* h0, const uint8_t* tok,
                        void* y, float* h_last, void* ws, size_t ws_bytes, int B, int T, int D, float c, int io_dtype,
                        void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!x_in || !conv_w || !u_r || !u_i || !lambda || !y) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(x_in, es) || !aligned(u_r, es) || !aligned(u_i, es) || !aligned(y, es) || !aligned(conv_state, es) ||
      !aligned(lambda, 4) || !aligned(conv_w, 4) || !aligned(conv_b, 4) || !aligned(h0, 4) || !aligned(h_last, 4) ||
      !aligned(ws, 4))
    return RGLRU_ERR_MISALIGNED;
  if (ws && ws_bytes < rglru_workspace_bytes(B, T, D, io_dtype)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;

  ScanFwdArgs a = {};
  a.x = x_in; a.ur = u_r; a.ui = u_i; a.y = y;
  a.lambda = lambda; a.h0 = h0; a.tok = tok; a.h_last = h_last;
  a.states = static_cast<float*>(ws);
  a.conv_w = conv_w; a.conv_b = conv_b; a.conv_state = conv_state;
  {
    const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
    a.ticket = ws ? reinterpret_cast<unsigned*>(static_cast<float*>(ws) + static_cast<size_t>(B) * nsave * D +
                                               static_cast<size_t>(B) * D)
                  : nullptr;
  }
  a.B = B; a.T = T; a.D = D; a.c = c; a.status = status;

  FwdMaps maps;
  bool tma = tma_shape_ok(T, D, es) && aligned(x_in, 16) && aligned(u_r, 16) && aligned(u_i, 16) && aligned(y, 16);
  if (tma) {
    const int rows = scan_fwd_box_rows(0), cols = scan_fwd_box_cols(0);
    tma = make_map(&maps.x, x_in, bf16, B, T, D, rows + 3, cols) && make_map(&maps.ur, u_r, bf16, B, T, D, rows, cols) &&
          make_map(&maps.ui, u_i, bf16, B, T, D, rows, cols) && make_map(&maps.y, y, bf16, B, T, D, rows, cols);
  }
  const cudaError_t e = launch_conv_scan_fwd(bf16, tma, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_conv_scan_bwd(const void* dy, const float* dh_last, const void* x_in, const float* conv_w, const float* conv_b,
                        const void* conv_state, const void* u_r, const void* u_i, const float* lambda, const float* h0,
                        const uint8_t* tok, void* ws, size_t ws_bytes, void* dx_conv, void* du_r, void* du_i,
                        float* dlambda, float* dh0, int B, int T, int D, float c, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!dy || !x_in || !conv_w || !u_r || !u_i || !lambda || !dx_conv || !du_r || !du_i || !dlambda)
    return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(dy, es) || !aligned(x_in, es) || !aligned(u_r, es) || !aligned(u_i, es) || !aligned(dx_conv, es) ||
      !aligned(du_r, es) || !aligned(du_i, es) || !aligned(conv_state, es) || !aligned(lambda, 4) ||
      !aligned(conv_w, 4) || !aligned(conv_b, 4) || !aligned(h0, 4) || !aligned(dh_last, 4) || !aligned(dlambda, 4) ||
      !aligned(dh0, 4) || !aligned(ws, 4))
    return RGLRU_ERR_MISALIGNED;
  if (!ws || ws_bytes < rglru_workspace_bytes(B, T, D, io_dtype)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;

  const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
  ScanBwdArgs a = {};
  a.dy = dy; a.x = x_in; a.ur = u_r; a.ui = u_i; a.dx = dx_conv; a.dur = du_r; a.dui = du_i;
  a.lambda = lambda; a.h0 = h0; a.dh_last = dh_last; a.tok = tok;
  a.states = static_cast<const float*>(ws);
  a.dlam_part = static_cast<float*>(ws) + static_cast<size_t>(B) * nsave * D;
  a.dlambda = dlambda; a.dh0 = dh0;
  a.ticket = (B <= FUSED_DLAMBDA_MAX_B) ? reinterpret_cast<unsigned*>(a.dlam_part + static_cast<size_t>(B) * D) : nullptr;
  a.conv_w = conv_w; a.conv_b = conv_b; a.conv_state = conv_state;
  a.B = B; a.T = T; a.D = D; a.c = c; a.status = status;

  BwdMaps maps;
  bool tma = tma_shape_ok(T, D, es) && aligned(dy, 16) && aligned(x_in, 16) && aligned(u_r, 16) && aligned(u_i, 16) &&
             aligned(dx_conv, 16) && aligned(du_r, 16) && aligned(du_i, 16);
  if (tma) {
    const int rows = scan_bwd_box_rows(0), cols = scan_bwd_box_cols(0);
    tma = make_map(&maps.dy, dy, bf16, B, T, D, rows, cols) && make_map(&maps.x, x_in, bf16, B, T, D, rows + 3, cols) &&
          make_map(&maps.ur, u_r, bf16, B, T, D, rows, cols) && make_map(&maps.ui, u_i, bf16, B, T, D, rows, cols) &&
          make_map(&maps.dx, dx_conv, bf16, B, T, D, rows, cols) && make_map(&maps.dur, du_r, bf16, B, T, D, rows, cols) &&
          make_map(&maps.dui, du_i, bf16, B, T, D, rows, cols);
  }
  const cudaError_t e = launch_conv_scan_bwd(bf16, tma, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_merge_fwd(const void* x, const float* conv_w, const float* conv_b, const void* conv_state, const void* u_r,
                    const void* u_i, const void* branch, const float* lambda, const float* h0, const uint8_t* tok,
                    void* out, float* h_last, void* ws, size_t ws_bytes, int B, int T, int D, float c, int io_dtype,
                    void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!x || !u_r || !u_i || !branch || !lambda || !out) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const bool conv = conv_w != nullptr;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(x, es) || !aligned(u_r, es) || !aligned(u_i, es) || !aligned(branch, es) || !aligned(out, es) ||
      !aligned(conv_state, es) || !aligned(lambda, 4) || !aligned(conv_w, 4) || !aligned(conv_b, 4) || !aligned(h0, 4) ||
      !aligned(h_last, 4) || !aligned(ws, 4))
    return RGLRU_ERR_MISALIGNED;
  if (ws && ws_bytes < rglru_workspace_bytes(B, T, D, io_dtype)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;

  ScanFwdArgs a = {};
  a.x = x; a.ur = u_r; a.ui = u_i; a.y = out; a.g = branch;
  a.lambda = lambda; a.h0 = h0; a.tok = tok; a.h_last = h_last;
  a.states = static_cast<float*>(ws);
  if (conv) { a.conv_w = conv_w; a.conv_b = conv_b; a.conv_state = conv_state; }
  {
    const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
    a.ticket = ws ? reinterpret_cast<unsigned*>(static_cast<float*>(ws) + static_cast<size_t>(B) * nsave * D +
                                               static_cast<size_t>(B) * D)
                  : nullptr;
  }
  a.B = B; a.T = T; a.D = D; a.c = c; a.status = status;

  FwdMaps maps;
  bool tma = tma_shape_ok(T, D, es) && aligned(x, 16) && aligned(u_r, 16) && aligned(u_i, 16) && aligned(branch, 16) &&
             aligned(out, 16);
  if (tma) {
    const int rows = scan_fwd_box_rows(0), cols = scan_fwd_box_cols(0);
    tma = make_map(&maps.x, x, bf16, B, T, D, rows + (conv ? 3 : 0), cols) &&
          make_map(&maps.ur, u_r, bf16, B, T, D, rows, cols) && make_map(&maps.ui, u_i, bf16, B, T, D, rows, cols) &&
          make_map(&maps.g, branch, bf16, B, T, D, rows, cols) && make_map(&maps.y, out, bf16, B, T, D, rows, cols);
  }
  const cudaError_t e = launch_merge_fwd(bf16, tma, conv, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_merge_bwd(const void* dout, const float* dh_last, const void* x, const float* conv_w, const float* conv_b,
                    const void* conv_state, const void* u_r, const void* u_i, const void* branch, const float* lambda,
                    const float* h0, const uint8_t* tok, void* ws, size_t ws_bytes, void* dx, void* du_r, void* du_i,
                    void* dbranch, float* dlambda, float* dh0, int B, int T, int D, float c, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!dout || !x || !u_r || !u_i || !branch || !lambda || !dx || !du_r || !du_i || !dbranch || !dlambda)
    return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const bool conv = conv_w != nullptr;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(dout, es) || !aligned(x, es) || !aligned(u_r, es) || !aligned(u_i, es) || !aligned(branch, es) ||
      !aligned(dx, es) || !aligned(du_r, es) || !aligned(du_i, es) || !aligned(dbranch, es) || !aligned(conv_state, es) ||
      !aligned(lambda, 4) || !aligned(conv_w, 4) || !aligned(conv_b, 4) || !aligned(h0, 4) || !aligned(dh_last, 4) ||
      !aligned(dlambda, 4) || !aligned(dh0, 4) || !aligned(ws, 4))
    return RGLRU_ERR_MISALIGNED;
  if (!ws || ws_bytes < rglru_workspace_bytes(B, T, D, io_dtype)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;

  const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
  ScanBwdArgs a = {};
  a.dy = dout; a.x = x; a.ur = u_r; a.ui = u_i; a.dx = dx; a.dur = du_r; a.dui = du_i; a.g = branch; a.dg = dbranch;
  a.lambda = lambda; a.h0 = h0; a.dh_last = dh_last; a.tok = tok;
  a.states = static_cast<const float*>(ws);
  a.dlam_part = static_cast<float*>(ws) + static_cast<size_t>(B) * nsave * D;
  a.dlambda = dlambda; a.dh0 = dh0;
  a.ticket = (B <= FUSED_DLAMBDA_MAX_B) ? reinterpret_cast<unsigned*>(a.dlam_part + static_cast<size_t>(B) * D) : nullptr;
  if (conv) { a.conv_w = conv_w; a.conv_b = conv_b; a.conv_state = conv_state; }
  a.B = B; a.T = T; a.D = D; a.c = c; a.status = status;

  BwdMaps maps;
  bool tma = tma_shape_ok(T, D, es) && aligned(dout, 16) && aligned(x, 16) && aligned(u_r, 16) && aligned(u_i, 16) &&
             aligned(branch, 16) && aligned(dx, 16) && aligned(du_r, 16) && aligned(du_i, 16) && aligned(dbranch, 16);
  if (tma) {
    const int rows = scan_bwd_box_rows(0), cols = scan_bwd_box_cols(0);
    tma = make_map(&maps.dy, dout, bf16, B, T, D, rows, cols) &&
          make_map(&maps.x, x, bf16, B, T, D, rows + (conv ? 3 : 0), cols) &&
          make_map(&maps.ur, u_r, bf16, B, T, D, rows, cols) && make_map(&maps.ui, u_i, bf16, B, T, D, rows, cols) &&
          make_map(&maps.g, branch, bf16, B, T, D, rows, cols) && make_map(&maps.dx, dx, bf16, B, T, D, rows, cols) &&
          make_map(&maps.dur, du_r, bf16, B, T, D, rows, cols) && make_map(&maps.dui, du_i, bf16, B, T, D, rows, cols) &&
          make_map(&maps.dg, dbranch, bf16, B, T, D, rows, cols);
  }
  const cudaError_t e = launch_merge_bwd(bf16, tma, conv, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

// Grouped gate layout: TMA staging only, so everything the copy engine touches must be 16-byte aligned and a
// channel tile must not straddle a gate head.
static int check_grouped(int D, int gate_width, size_t es) {
  if (gate_width <= 0 || D % gate_width != 0 || gate_width % grouped_box_cols() != 0) return RGLRU_ERR_BAD_SHAPE;
  if ((static_cast<size_t>(D) * es) % 16 != 0) return RGLRU_ERR_BAD_SHAPE;
  return RGLRU_OK;
}

int rglru_grouped_fwd(const void* x, const void* u, const float* gate_bias, const void* branch, const float* lambda,
                      const float* h0, const uint8_t* tok, void* out, float* h_last, void* ws, size_t ws_bytes, int B,
                      int T, int D, int gate_width, float c, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!x || !u || !lambda || !out) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const bool merge = branch != nullptr;
  const size_t es = bf16 ? 2 : 4;
  rc = check_grouped(D, gate_width, es);
  if (rc != RGLRU_OK) return rc;
  if (!aligned(x, 16) || !aligned(u, 16) || !aligned(branch, 16) || !aligned(out, 16) || !aligned(gate_bias, 16) ||
      !aligned(lambda, 4) || !aligned(h0, 4) || !aligned(h_last, 4) || !aligned(ws, 4))
    return RGLRU_ERR_MISALIGNED;
  if (ws && ws_bytes < rglru_workspace_bytes(B, T, D, io_dtype)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;

  ScanFwdArgs a = {};
  a.x = x; a.ur = u; a.ui = u; a.y = out; a.g = branch; a.gate_bias = gate_bias; a.gate_bw = gate_width;
  a.lambda = lambda; a.h0 = h0; a.tok = tok; a.h_last = h_last;
  a.states = static_cast<float*>(ws);
  {
    const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
    a.ticket = ws ? reinterpret_cast<unsigned*>(static_cast<float*>(ws) + static_cast<size_t>(B) * nsave * D +
                                               static_cast<size_t>(B) * D)
                  : nullptr;
  }
  a.B = B; a.T = T; a.D = D; a.c = c; a.status = status;

  FwdMaps maps;
  const int rows = scan_fwd_box_rows(0), cols = grouped_box_cols();
  bool ok = make_map(&maps.x, x, bf16, B, T, D, rows, cols) && make_map(&maps.ur, u, bf16, B, T, 2 * D, rows, cols) &&
            make_map(&maps.y, out, bf16, B, T, D, rows, cols);
  if (ok && merge) ok = make_map(&maps.g, branch, bf16, B, T, D, rows, cols);
  if (!ok) return RGLRU_ERR_UNSUPPORTED;
  maps.ui = maps.ur;
  const cudaError_t e = launch_grouped_fwd(bf16, merge, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_grouped_bwd(const void* dout, const float* dh_last, const void* x, const void* u, const float* gate_bias,
                      const void* branch, const float* lambda, const float* h0, const uint8_t* tok, void* ws,
                      size_t ws_bytes, void* dx, void* du, void* dbranch, float* dlambda, float* dh0, float* d_gate_bias,
                      int B, int T, int D, int gate_width, float c, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!dout || !x || !u || !lambda || !dx || !du || !dlambda || (branch && !dbranch)) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const bool merge = branch != nullptr;
  const size_t es = bf16 ? 2 : 4;
  rc = check_grouped(D, gate_width, es);
  if (rc != RGLRU_OK) return rc;
  if (!aligned(dout, 16) || !aligned(x, 16) || !aligned(u, 16) || !aligned(branch, 16) || !aligned(dx, 16) ||
      !aligned(du, 16) || !aligned(dbranch, 16) || !aligned(gate_bias, 16) || !aligned(d_gate_bias, 16) ||
      !aligned(lambda, 4) || !aligned(h0, 4) || !aligned(dh_last, 4) || !aligned(dlambda, 4) || !aligned(dh0, 4) ||
      !aligned(ws, 16))
    return RGLRU_ERR_MISALIGNED;
  if (!ws || ws_bytes < rglru_workspace_bytes(B, T, D, io_dtype)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;

  const size_t nsave = (static_cast<size_t>(T) + SAVE_EVERY - 1) / SAVE_EVERY;
  ScanBwdArgs a = {};
  a.dy = dout; a.x = x; a.ur = u; a.ui = u; a.dx = dx; a.dur = du; a.dui = du; a.g = branch; a.dg = dbranch;
  a.gate_bias = gate_bias; a.gate_bw = gate_width;
  a.lambda = lambda; a.h0 = h0; a.dh_last = dh_last; a.tok = tok;
  a.states = static_cast<const float*>(ws);
  a.dlam_part = static_cast<float*>(ws) + static_cast<size_t>(B) * nsave * D;
  a.dlambda = dlambda; a.dh0 = dh0;
  a.ticket = (B <= FUSED_DLAMBDA_MAX_B) ? reinterpret_cast<unsigned*>(a.dlam_part + static_cast<size_t>(B) * D) : nullptr;
  a.dgate_part = d_gate_bias ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a.dlam_part + static_cast<size_t>(B) * D) +
                                                         WS_TAIL_BYTES)
                             : nullptr;
  a.dgate = d_gate_bias;
  a.B = B; a.T = T; a.D = D; a.c = c; a.status = status;

  BwdMaps maps;
  const int rows = scan_bwd_box_rows(0), cols = grouped_box_cols();
  bool ok = make_map(&maps.dy, dout, bf16, B, T, D, rows, cols) && make_map(&maps.x, x, bf16, B, T, D, rows, cols) &&
            make_map(&maps.ur, u, bf16, B, T, 2 * D, rows, cols) && make_map(&maps.dx, dx, bf16, B, T, D, rows, cols) &&
            make_map(&maps.dur, du, bf16, B, T, 2 * D, rows, cols);
  if (ok && merge)
    ok = make_map(&maps.g, branch, bf16, B, T, D, rows, cols) && make_map(&maps.dg, dbranch, bf16, B, T, D, rows, cols);
  if (!ok) return RGLRU_ERR_UNSUPPORTED;
  maps.ui = maps.ur;
  maps.dui = maps.dur;
  const cudaError_t e = launch_grouped_bwd(bf16, merge, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_linear_scan_fwd(const float* decay, const float* drive, const float* h0, float* out, int B, int T, int D,
                          void* stream) {
  if (!decay || !drive || !out) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  if (!aligned(decay, 4) || !aligned(drive, 4) || !aligned(out, 4) || !aligned(h0, 4)) return RGLRU_ERR_MISALIGNED;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  RawScanArgs a = {};
  a.decay = decay; a.drive = drive; a.h0 = h0; a.out = out;
  a.B = B; a.T = T; a.D = D; a.status = status;
  RawFwdMaps maps;
  bool tma = tma_shape_ok(T, D, 4) && aligned(decay, 16) && aligned(drive, 16) && aligned(out, 16);
  if (tma) {
    const int rows = raw_box_rows(), cols = raw_box_cols();
    tma = make_map(&maps.drive, drive, false, B, T, D, rows, cols) && make_map(&maps.decay, decay, false, B, T, D, rows, cols) &&
          make_map(&maps.out, out, false, B, T, D, rows, cols);
  }
  const cudaError_t e = launch_raw_fwd(tma, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_linear_scan_bwd(const float* d_out, const float* decay, const float* h0, const float* out, float* d_decay,
                          float* d_drive, float* d_h0, int B, int T, int D, void* stream) {
  if (!d_out || !decay || !out || !d_decay || !d_drive) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  if (!aligned(d_out, 4) || !aligned(decay, 4) || !aligned(out, 4) || !aligned(d_decay, 4) || !aligned(d_drive, 4) ||
      !aligned(h0, 4) || !aligned(d_h0, 4))
    return RGLRU_ERR_MISALIGNED;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  RawScanArgs a = {};
  a.dout = d_out; a.decay = decay; a.h0 = h0; a.out_in = out; a.ddecay = d_decay; a.ddrive = d_drive; a.dh0 = d_h0;
  a.B = B; a.T = T; a.D = D; a.status = status;
  RawBwdMaps maps;
  bool tma = tma_shape_ok(T, D, 4) && aligned(d_out, 16) && aligned(decay, 16) && aligned(out, 16) &&
             aligned(d_decay, 16) && aligned(d_drive, 16);
  if (tma) {
    const int rows = raw_box_rows(), cols = raw_box_cols();
    tma = make_map(&maps.dout, d_out, false, B, T, D, rows, cols) && make_map(&maps.decay, decay, false, B, T, D, rows, cols) &&
          make_map(&maps.out, out, false, B, T, D, rows, cols) && make_map(&maps.ddecay, d_decay, false, B, T, D, rows, cols) &&
          make_map(&maps.ddrive, d_drive, false, B, T, D, rows, cols);
  }
  const cudaError_t e = launch_raw_bwd(tma, maps, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_conv_fwd(const void* x_in, const float* conv_w, const float* conv_b, const void* conv_state,
                   const uint8_t* tok, void* x_conv, void* new_state, int B, int T, int D, int io_dtype,
                   void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!x_in || !conv_w || !x_conv) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(x_in, es) || !aligned(x_conv, es) || !aligned(conv_state, es) || !aligned(new_state, es) ||
      !aligned(conv_w, 4) || !aligned(conv_b, 4))
    return RGLRU_ERR_MISALIGNED;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  ConvArgs a = {};
  a.x_in = x_in; a.w = conv_w; a.bias = conv_b; a.state = conv_state; a.tok = tok; a.out = x_conv;
  a.new_state = new_state; a.B = B; a.T = T; a.D = D;
  a.vector_ok = (static_cast<size_t>(D) * es) % 16 == 0 && aligned(x_in, 16) && aligned(x_conv, 16) &&
                aligned(conv_state, 16) && aligned(conv_w, 16);
  ConvMaps maps;
  a.maps = nullptr;
  a.status = status;
  if (conv_tma_pays(B, D) && tma_shape_ok(T, D, es) && aligned(x_in, 16) && aligned(x_conv, 16) &&
      make_map(&maps.in0, x_in, bf16, B, T, D, conv_tma_box_rows(), conv_tma_box_cols()) &&
      make_map(&maps.out0, x_conv, bf16, B, T, D, conv_tma_box_rows() - 3, conv_tma_box_cols()))
    a.maps = &maps;
  const cudaError_t e = launch_conv_fwd(bf16, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

size_t rglru_conv_bwd_workspace_bytes(int B, int T, int D) {
  if (B <= 0 || T <= 0 || D <= 0) return 0;
  return static_cast<size_t>(conv_bwd_partial_rows(B, T)) * 5 * D * sizeof(float);
}

int rglru_conv_bwd(const void* d_conv, const void* x_in, const float* conv_w, const void* conv_state,
                   const uint8_t* tok, void* dx_in, float* d_w, float* d_b, void* d_state, void* ws, size_t ws_bytes,
                   int B, int T, int D, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!d_conv || !x_in || !conv_w || !dx_in || !d_w) return RGLRU_ERR_NULL_POINTER;
  int rc = check_dims(B, T, D);
  if (rc != RGLRU_OK) return rc;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(d_conv, es) || !aligned(x_in, es) || !aligned(dx_in, es) || !aligned(conv_state, es) ||
      !aligned(d_state, es) || !aligned(conv_w, 4) || !aligned(d_w, 4) || !aligned(d_b, 4) || !aligned(ws, 4))
    return RGLRU_ERR_MISALIGNED;
  if (!ws || ws_bytes < rglru_conv_bwd_workspace_bytes(B, T, D)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  ConvBwdArgs a = {};
  a.d_conv = d_conv; a.x_in = x_in; a.w = conv_w; a.state = conv_state; a.tok = tok; a.dx_in = dx_in;
  a.d_w = d_w; a.d_b = d_b; a.d_state = d_state; a.part = static_cast<float*>(ws);
  a.B = B; a.T = T; a.D = D;
  a.vector_ok = (static_cast<size_t>(D) * es) % 16 == 0 && aligned(d_conv, 16) && aligned(x_in, 16) &&
                aligned(dx_in, 16) && aligned(conv_state, 16) && aligned(d_state, 16) && aligned(conv_w, 16);
  ConvMaps maps;
  a.maps = nullptr;
  a.status = status;
  if (conv_tma_pays(B, D) && tma_shape_ok(T, D, es) && aligned(d_conv, 16) && aligned(x_in, 16) && aligned(dx_in, 16) &&
      make_map(&maps.in0, d_conv, bf16, B, T, D, conv_tma_box_rows(), conv_tma_box_cols()) &&
      make_map(&maps.in1, x_in, bf16, B, T, D, conv_tma_box_rows(), conv_tma_box_cols()) &&
      make_map(&maps.out0, dx_in, bf16, B, T, D, conv_tma_box_rows() - 3, conv_tma_box_cols()))
    a.maps = &maps;
  const cudaError_t e = launch_conv_bwd(bf16, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

size_t rglru_column_sums_workspace_bytes(long long rows, int cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return static_cast<size_t>(colsum_row_blocks(rows, cols)) * cols * sizeof(float);
}

int rglru_column_sums(const void* src, float* out, void* ws, size_t ws_bytes, long long rows, int cols, int io_dtype,
                      void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!src || !out) return RGLRU_ERR_NULL_POINTER;
  if (rows <= 0 || cols <= 0 || rows > (1ll << 40)) return RGLRU_ERR_BAD_SHAPE;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(src, es) || !aligned(out, 4) || !aligned(ws, 4)) return RGLRU_ERR_MISALIGNED;
  if (!ws || ws_bytes < rglru_column_sums_workspace_bytes(rows, cols)) return RGLRU_ERR_WORKSPACE;
  int* status = nullptr;
  const int rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  const bool vector_ok = (static_cast<size_t>(cols) * es) % 16 == 0 && aligned(src, 16);
  const cudaError_t e = launch_column_sums(bf16, src, out, static_cast<float*>(ws), rows, cols, vector_ok,
                                           static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_decode_conv(const void* x_in, const float* conv_w, const float* conv_b, void* conv_state,
                      const uint8_t* tok, void* x_conv, int B, int D, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!x_in || !conv_w || !conv_state || !x_conv) return RGLRU_ERR_NULL_POINTER;
  if (B <= 0 || D <= 0) return RGLRU_ERR_BAD_SHAPE;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(x_in, es) || !aligned(x_conv, es) || !aligned(conv_state, es) || !aligned(conv_w, 4) ||
      !aligned(conv_b, 4))
    return RGLRU_ERR_MISALIGNED;
  int* status = nullptr;
  int rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  ConvArgs a = {};
  a.x_in = x_in; a.w = conv_w; a.bias = conv_b; a.state = nullptr; a.tok = tok; a.out = x_conv;
  a.new_state = conv_state; a.B = B; a.T = 1; a.D = D;
  a.vector_ok = (static_cast<size_t>(D) * es) % 16 == 0 && aligned(x_in, 16) && aligned(x_conv, 16) &&
                aligned(conv_state, 16);
  const cudaError_t e = launch_decode_conv(bf16, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

int rglru_decode_step(const void* x, const void* u_r, const void* u_i, const float* lambda, float* h,
                      const uint8_t* tok, void* y, int B, int D, float c, int io_dtype, void* stream) {
  if (io_dtype != RGLRU_F32 && io_dtype != RGLRU_BF16) return RGLRU_ERR_BAD_DTYPE;
  if (!x || !u_r || !u_i || !lambda || !h || !y) return RGLRU_ERR_NULL_POINTER;
  if (B <= 0 || D <= 0) return RGLRU_ERR_BAD_SHAPE;
  const bool bf16 = io_dtype == RGLRU_BF16;
  const size_t es = bf16 ? 2 : 4;
  if (!aligned(x, es) || !aligned(u_r, es) || !aligned(u_i, es) || !aligned(y, es) || !aligned(lambda, 4) ||
      !aligned(h, 4))
    return RGLRU_ERR_MISALIGNED;
  int* status = nullptr;
  int rc = device_setup(&status);
  if (rc != RGLRU_OK) return rc;
  DecodeArgs a;
  a.x = x; a.ur = u_r; a.ui = u_i; a.lambda = lambda; a.h = h; a.tok = tok; a.y = y;
  a.B = B; a.D = D; a.c = c;
  a.vector_ok = (static_cast<size_t>(D) * es) % 16 == 0 && aligned(x, 16) && aligned(u_r, 16) && aligned(u_i, 16) &&
                aligned(y, 16) && aligned(h, 16);
  const cudaError_t e = launch_decode_step(bf16, a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? RGLRU_OK : fail_cuda(e);
}

}  // extern "C"
