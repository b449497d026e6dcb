/*
 * rglru_b200.h -- C ABI of the B200 (sm_100a) RG-LRU kernels.
 *
 * Every entry point replaces one piece of the Griffin reference's RG-LRU path
 * (paths below are relative to the reference project root).  All pointers are
 * DEVICE pointers owned by the caller, tensors are dense row-major with the
 * channel axis fastest ([B, T, D] unless stated otherwise).  Functions never
 * throw and never synchronise; they enqueue work on `stream` (a cudaStream_t
 * passed as void*, NULL = legacy default stream) of the current device and
 * return an rglru_status.  Except where stated they allocate no device memory.
 *
 * io_dtype selects the element type of the [B,T,D] activations and their
 * gradients; the recurrent state, Lambda and every reduction are fp32.
 */
#ifndef RGLRU_B200_H
#define RGLRU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum rglru_dtype { RGLRU_F32 = 0, RGLRU_BF16 = 1 };

enum rglru_status {
  RGLRU_OK = 0,
  RGLRU_ERR_NULL_POINTER = 1,   /* a required pointer is NULL */
  RGLRU_ERR_BAD_DTYPE = 2,      /* io_dtype is not a member of rglru_dtype */
  RGLRU_ERR_BAD_SHAPE = 3,      /* a dimension is <= 0 or exceeds the supported range */
  RGLRU_ERR_MISALIGNED = 4,     /* a pointer is not aligned to its element size */
  RGLRU_ERR_WORKSPACE = 5,      /* workspace is missing or smaller than rglru_workspace_bytes() */
  RGLRU_ERR_LAUNCH = 6,         /* the CUDA runtime rejected a launch (see rglru_last_cuda_error) */
  RGLRU_ERR_DEVICE_TIMEOUT = 7, /* a bounded in-kernel wait expired (reported by rglru_device_status) */
  RGLRU_ERR_UNSUPPORTED = 8,    /* the device is not sm_100 or the driver lacks a required entry point */
  RGLRU_ERR_TOO_LARGE = 9       /* the problem exceeds a fixed capacity of the entry point (see rglru_conv_bwd_noalloc) */
};

/* Per-token flag byte shared by all kernels (one byte per (b, t), row-major [B, T]).
 * It packs what the reference passes as three tensors: `reset_mask`, `active_mask`
 * (griffin/griffin.py:195-196) and, for the convolution, the tap mask
 * `segment_pos >= lag` (griffin/griffin.py:485).  A zero byte is an ordinary token
 * (active, no reset, all four taps inside its document) and a NULL mask pointer
 * means "all zero". */
#define RGLRU_TOK_CUT_MASK 0x03u     /* 3 - min(segment_pos, 3): how many of the oldest taps fall outside the document */
#define RGLRU_TOK_RESET 0x04u        /* recurrence restarts here: a = 0, gamma = 1 */
#define RGLRU_TOK_INACTIVE 0x08u     /* right padding: a = 1, b = 0, conv emits 0 and keeps its history */
#define RGLRU_TOK_ZERO_HISTORY 0x10u /* conv history older than this token is returned as zeros in the next
                                        conv state (the variable-length path, griffin/griffin.py:495-496) */

const char* rglru_status_string(int status);
/* Text of the last CUDA runtime error seen by this library on the calling thread. */
const char* rglru_last_cuda_error(void);
int rglru_abi_version(void);

/* Reads (and clears) the device-side status word that kernels set when a bounded
 * wait expires.  Synchronises the current device.  Returns RGLRU_OK or
 * RGLRU_ERR_DEVICE_TIMEOUT; *detail receives a kernel-specific code. */
int rglru_device_status(int* detail);

/* Self-test of the bounded in-kernel wait (no reference counterpart; the reference's only runtime self-check is
 * the Triton validation of griffin/triton_scan.py:180-204).  Launches one small CTA that waits, for at most
 * `limit_us` microseconds (1 .. 100000), on a barrier that nothing completes.  The wait gives up, the kernel runs
 * to its end (writing 1 to *finished when `finished`, a device int, is non-NULL) and the next
 * rglru_device_status() reports RGLRU_ERR_DEVICE_TIMEOUT with detail 3.  The context stays usable. */
int rglru_selftest_wait_timeout(unsigned limit_us, int* finished, void* stream);

/* Time-steps between two saved recurrent states (the backward kernel rebuilds the
 * states inside one such chunk from its entry state). */
int rglru_chunk_steps(int io_dtype);

/* Bytes of caller-provided workspace shared by rglru_fwd and rglru_bwd of one call
 * pair: chunk-entry states [B, ceil(T/chunk), D] fp32, per-row dLambda partial sums
 * [B, D] fp32, and a 256-byte tail with a completion ticket that rglru_fwd zeroes.  Contents written by rglru_fwd must be left untouched
 * until the matching rglru_bwd has run. */
size_t rglru_workspace_bytes(int B, int T, int D, int io_dtype);

/* Forward: gate epilogue + linear scan.
 * Replaces RG_LRU.forward from the gate activations on: griffin/griffin.py:237-258
 * (sigmoid gates, a = exp(c r logsigmoid(Lambda)), gamma = sqrt(-expm1(2 log a)),
 * reset / active masking, b = gamma i x) and the scan griffin/griffin.py:273-286
 * (also griffin/triton_scan.py:31-60 fed by the eager epilogue).
 *   x, u_r, u_i : [B,T,D] io_dtype; u_r / u_i are the outputs of the recurrence and
 *                 input BlockDiagonalLinear gates (griffin/griffin.py:237-238) BEFORE the sigmoid
 *   lambda      : [D] fp32        h0 : [B,D] fp32 or NULL (zeros)
 *   tok         : [B,T] flag bytes or NULL
 *   y           : [B,T,D] io_dtype out      h_last : [B,D] fp32 out or NULL
 *   ws          : workspace or NULL; NULL skips saving chunk states (inference only)
 */
int rglru_fwd(const void* x, const void* u_r, const void* u_i, const float* lambda, const float* h0,
              const uint8_t* tok, void* y, float* h_last, void* ws, size_t ws_bytes, int B, int T,
              int D, float c, int io_dtype, void* stream);

/* rglru_fwd that also returns the product of the decays over the sequence, decay_prod [B,D] fp32 (with masks
 * applied: 0 through a reset, 1 through padding).  Together with h_last computed from h0 = 0 it is the affine
 * map  h_last(h0) = decay_prod * h0 + h_last(0)  of this call, which lets one sequence be split over several
 * calls, or over the GPUs of a box along TIME, with one small exchange of [B,D] pairs between the pieces
 * (the associative operator of griffin/griffin.py:291-306 applied to whole slices).  The reference has no
 * such entry point; griffin_b200/time_shard.py is its user.  h_last and decay_prod are required.
 * y may be NULL: a carry-only pass that reads its inputs and writes h_last and decay_prod only (pass ws = NULL
 * with it; a slice's first pass needs nothing else). */
int rglru_fwd_carry(const void* x, const void* u_r, const void* u_i, const float* lambda, const float* h0,
                    const uint8_t* tok, void* y, float* h_last, float* decay_prod, void* ws, size_t ws_bytes, int B,
                    int T, int D, float c, int io_dtype, void* stream);

/* Backward of rglru_fwd.  The reference obtains these gradients from autograd over
 * griffin/griffin.py:237-286 with the capped sqrt slope of griffin/griffin.py:59-65
 * and, for the scan itself, griffin/triton_scan.py:63-122.
 *   dy       : [B,T,D] io_dtype     dh_last : [B,D] fp32 or NULL (zeros)
 *   x,u_r,u_i,lambda,h0,tok : the forward inputs;  ws : the workspace rglru_fwd filled
 *   dx       : [B,T,D] io_dtype out -- the DIRECT path only (through b = gamma i x); the
 *              part through the gate projections is the caller's GEMM backward of du_r/du_i
 *   du_r,du_i: [B,T,D] io_dtype out     dlambda : [D] fp32 out     dh0 : [B,D] fp32 out or NULL
 * Carry-only form (no reference counterpart; the time split's first backward pass): dx, du_r, du_i and dlambda
 * ALL NULL and dh0 given -- the call reads its inputs and writes dh0 only.  Any other NULL among the four is an
 * error.
 */
int rglru_bwd(const void* dy, const float* dh_last, const void* x, const void* u_r, const void* u_i,
              const float* lambda, const float* h0, const uint8_t* tok, void* ws, size_t ws_bytes,
              void* dx, void* du_r, void* du_i, float* dlambda, float* dh0, int B, int T, int D,
              float c, int io_dtype, void* stream);

/* Conv folded into the scan's load stage.  rglru_conv_scan_fwd computes rglru_fwd(conv(x_in), u_r, u_i)
 * and rglru_conv_scan_bwd the matching rglru_bwd, both reading the conv INPUT x_in (the output of linear_x,
 * griffin/griffin.py:465) with a three-token halo and applying the four taps, bias and document-boundary
 * tap masks of griffin/griffin.py:474-486 while a chunk is loaded, so the conv output need not be kept for
 * the backward pass.  u_r / u_i are still the gate pre-activations of the conv OUTPUT (the gate GEMMs are
 * the caller's and need that tensor once, from rglru_conv_fwd).
 *   conv_w [D,4] fp32 (column 3 on the current token), conv_b [D] fp32 or NULL,
 *   conv_state [B,3,D] io_dtype history before t = 0 or NULL (zeros); other arguments as rglru_fwd / rglru_bwd.
 *   rglru_conv_scan_bwd writes dx_conv = the gradient with respect to the conv OUTPUT through b = gamma i x
 *   only; the caller adds the gate-projection path and runs rglru_conv_bwd once on the sum.
 * Inactive (padding) tokens are handled as in rglru_fwd; the tok bytes must carry the tap-cut bits. */
int rglru_conv_scan_fwd(const void* x_in, const float* conv_w, const float* conv_b, const void* conv_state,
                        const void* u_r, const void* u_i, const float* lambda, const float* h0, const uint8_t* tok,
                        void* y, float* h_last, void* ws, size_t ws_bytes, int B, int T, int D, float c, int io_dtype,
                        void* stream);
int rglru_conv_scan_bwd(const void* dy, const float* dh_last, const void* x_in, const float* conv_w, const float* conv_b,
                        const void* conv_state, const void* u_r, const void* u_i, const float* lambda, const float* h0,
                        const uint8_t* tok, void* ws, size_t ws_bytes, void* dx_conv, void* du_r, void* du_i,
                        float* dlambda, float* dh0, int B, int T, int D, float c, int io_dtype, void* stream);

/* Branch merge folded into the scan.  The recurrent block multiplies the RG-LRU output by the GeLU branch
 * before its output projection: linear_out(x_branch * gelu(linear_y(x), approximate="tanh")),
 * griffin/griffin.py:464 and :520.  rglru_merge_fwd is rglru_fwd (conv_w == NULL) or rglru_conv_scan_fwd
 * (conv_w != NULL; x is then the conv INPUT) whose store stage writes out = h * gelu(branch) instead of h;
 * rglru_merge_bwd takes dout = the gradient of that product, forms the gradient of h while loading, and also
 * writes dbranch = dout * h * gelu'(branch).  h_last, ws, dx, du_r, du_i, dlambda, dh0 as in the unmerged calls.
 *   branch  : [B,T,D] io_dtype, the PRE-activation linear_y(x)        dbranch : [B,T,D] io_dtype out
 * With bf16 I/O the gradient of h is rounded to bf16 once inside the kernel, as the unfused sequence would. */
int rglru_merge_fwd(const void* x, const float* conv_w, const float* conv_b, const void* conv_state, const void* u_r,
                    const void* u_i, const void* branch, const float* lambda, const float* h0, const uint8_t* tok,
                    void* out, float* h_last, void* ws, size_t ws_bytes, int B, int T, int D, float c, int io_dtype,
                    void* stream);
int rglru_merge_bwd(const void* dout, const float* dh_last, const void* x, const float* conv_w, const float* conv_b,
                    const void* conv_state, const void* u_r, const void* u_i, const void* branch, const float* lambda,
                    const float* h0, const uint8_t* tok, void* ws, size_t ws_bytes, void* dx, void* du_r, void* du_i,
                    void* dbranch, float* dlambda, float* dh0, int B, int T, int D, float c, int io_dtype, void* stream);

/* Grouped gate layout.  The reference computes the two gates with two block-diagonal projections of the same
 * input (BlockDiagonalLinear, griffin/griffin.py:129-154, called at :237-238).  Stacking the two weight blocks
 * of every gate head ([G, 2 bw, bw]) turns them into ONE grouped GEMM whose output, written straight into a
 * [B, T, G, 2 bw] tensor, holds per head the columns [u_r (bw) | u_i (bw)].  rglru_grouped_fwd / _bwd read (and
 * write the gradient of) that tensor directly and add the gate biases themselves, so neither a re-layout nor a
 * bias pass is needed.  branch / dbranch non-NULL additionally folds the branch merge (see rglru_merge_fwd).
 *   u, du     : [B,T,2D] io_dtype in the layout above      gate_bias : [2D] fp32, same column layout, or NULL
 *   gate_width: bw = D / G, a multiple of 64; D * sizeof(element) a multiple of 16 (else RGLRU_ERR_BAD_SHAPE)
 *   x, u, branch, out, dout, dx, du, dbranch and gate_bias must be 16-byte aligned (else RGLRU_ERR_MISALIGNED).
 *   d_gate_bias : [2D] fp32, same column layout, 16-byte aligned, or NULL.  When given, the backward kernel also
 *               returns the gradient of the gate biases (the sums of du over batch and time, taken from the
 *               fp32 values before they are rounded to io_dtype, rows folded in index order), which saves the
 *               caller a reduction pass over du.  The workspace must then be 16-byte aligned.
 * Everything else as rglru_fwd / rglru_bwd; the caller's GEMMs turn du into the input and weight gradients. */
int rglru_grouped_fwd(const void* x, const void* u, const float* gate_bias, const void* branch, const float* lambda,
                      const float* h0, const uint8_t* tok, void* out, float* h_last, void* ws, size_t ws_bytes, int B,
                      int T, int D, int gate_width, float c, int io_dtype, void* stream);
int rglru_grouped_bwd(const void* dout, const float* dh_last, const void* x, const void* u, const float* gate_bias,
                      const void* branch, const float* lambda, const float* h0, const uint8_t* tok, void* ws,
                      size_t ws_bytes, void* dx, void* du, void* dbranch, float* dlambda, float* dh0, float* d_gate_bias,
                      int B, int T, int D, int gate_width, float c, int io_dtype, void* stream);

/* Raw affine scan h_t = a_t h_{t-1} + b_t on fp32 tensors: the operator
 * fused_rglru_scan(decay, current_input, initial_state) of griffin/triton_scan.py:274-276
 * (forward kernel :31-60).  decay, drive, out: [B,T,D] fp32; h0: [B,D] fp32 or NULL. */
int rglru_linear_scan_fwd(const float* decay, const float* drive, const float* h0, float* out, int B,
                          int T, int D, void* stream);

/* Backward of the raw scan (griffin/triton_scan.py:63-122, 248-271): given the saved
 * decay, h0 and forward output, writes d_decay = g_t h_{t-1}, d_drive = g_t and
 * d_h0 = a_0 g_0 with g_t = d_out_t + a_{t+1} g_{t+1}.  d_h0 may be NULL. */
int rglru_linear_scan_bwd(const float* d_out, const float* decay, const float* h0, const float* out,
                          float* d_decay, float* d_drive, float* d_h0, int B, int T, int D,
                          void* stream);

/* Causal depthwise convolution, kernel width 4, with document-boundary tap masking:
 * griffin/griffin.py:474-487 (dense path) and, when tok carries RGLRU_TOK_INACTIVE
 * bytes, the right-padded path griffin/griffin.py:488-510.
 *   x_in       : [B,T,D] io_dtype (output of linear_x)
 *   conv_w     : [D,4] fp32, column 3 multiplies the current token (temporal_conv.weight[:,0,:])
 *   conv_b     : [D] fp32 or NULL
 *   conv_state : [B,3,D] io_dtype history before t = 0, or NULL (zeros)
 *   tok        : [B,T] flag bytes or NULL
 *   x_conv     : [B,T,D] io_dtype out
 *   new_state  : [B,3,D] io_dtype out or NULL
 */
int rglru_conv_fwd(const void* x_in, const float* conv_w, const float* conv_b, const void* conv_state,
                   const uint8_t* tok, void* x_conv, void* new_state, int B, int T, int D,
                   int io_dtype, void* stream);

/* Backward of rglru_conv_fwd for the dense (no padding) case: the reference gets it from
 * autograd over griffin/griffin.py:478-486.
 *   d_conv : [B,T,D] io_dtype gradient of x_conv;   x_in, conv_w, conv_state, tok as in forward
 *   dx_in  : [B,T,D] io_dtype out
 *   d_w    : [D,4] fp32 out   d_b : [D] fp32 out or NULL   d_state : [B,3,D] io_dtype out or NULL
 *   ws     : >= rglru_conv_bwd_workspace_bytes(B,T,D) bytes of scratch
 */
size_t rglru_conv_bwd_workspace_bytes(int B, int T, int D);
int rglru_conv_bwd(const void* d_conv, const void* x_in, const float* conv_w, const void* conv_state,
                   const uint8_t* tok, void* dx_in, float* d_w, float* d_b, void* d_state, void* ws,
                   size_t ws_bytes, int B, int T, int D, int io_dtype, void* stream);

/* Conv backward for callers that cannot allocate device memory.  (No counterpart in the reference:
 * it exists for hosts of this library that may not call cudaMalloc or any allocating routine at the
 * point where the backward runs -- a runtime that owns all device memory and lends none to plugins,
 * a serving loop whose memory plan is frozen, a callback in which an allocation would synchronise
 * the device.)  Same arguments and results as rglru_conv_bwd, minus the workspace: the partial sums
 * live in a fixed 4 MiB array inside the library image, which every GPU on which the library's device
 * code is loaded holds until the process exits.
 *   - Limit: B * ceil(T / 256) * 5 * D <= 1,048,576 floats (rglru_conv_bwd_noalloc_max_bytes() / 4);
 *     anything larger returns RGLRU_ERR_TOO_LARGE and launches nothing.
 *   - The first call on each device looks up the array's device address (with that device current)
 *     and, under CUDA's lazy module loading, is also what loads the kernels and the array: it may
 *     allocate and synchronise inside the driver.  Make one warm-up call per device BEFORE entering the
 *     region where allocation is forbidden, and outside any stream capture.
 *   - `stream` must belong to the device that is current at the call (the scratch address is that
 *     device's); a stream of another device fails with RGLRU_ERR_LAUNCH.
 *   - It always runs the kernels that split the time axis; the TMA-staged kernels that rglru_conv_bwd
 *     may pick for large batches are not used here (same results up to rounding, possibly slower).
 *   - All calls share the array.  Calls on one stream are ordered and safe; calls that can overlap
 *     on the GPU (different streams, several host threads) race on it and must be serialised by the
 *     caller.  Nothing needs clearing between calls: every entry read is written first by the same call.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine. */
size_t rglru_conv_bwd_noalloc_max_bytes(void);
int rglru_conv_bwd_noalloc(const void* d_conv, const void* x_in, const float* conv_w, const void* conv_state,
                           const uint8_t* tok, void* dx_in, float* d_w, float* d_b, void* d_state, int B, int T,
                           int D, int io_dtype, void* stream);

/* Column sums of a dense row-major matrix: out[c] = sum_r src[r, c], fp32 accumulation in a fixed order (two
 * launches, no atomics), at streaming bandwidth.  It serves the bias gradients of the three linear layers
 * around the recurrence (griffin/griffin.py:379-389: linear_x, linear_y, linear_out; the reference leaves them
 * to autograd's generic reduction), whose inputs are exactly the gradients this library's backward kernels
 * produce or consume.
 *   src : [rows, cols] io_dtype   out : [cols] fp32   ws : rglru_column_sums_workspace_bytes(rows, cols) bytes
 */
size_t rglru_column_sums_workspace_bytes(long long rows, int cols);
int rglru_column_sums(const void* src, float* out, void* ws, size_t ws_bytes, long long rows, int cols, int io_dtype,
                      void* stream);

/* Single-token decode update: the T = 1 case of RecurrentBlock.forward with a cache,
 * griffin/griffin.py:459-528, split at the gate projections (which stay ordinary GEMMs):
 *
 * rglru_decode_conv: x_conv = bias + sum_k w[:,k] * [conv_state; x_in][k] with tap masking,
 * then conv_state <- last 3 rows (griffin/griffin.py:478-487); inactive rows leave the
 * state unchanged and emit zeros (griffin/griffin.py:505-508).
 *   x_in : [B,D] io_dtype   conv_state : [B,3,D] io_dtype in/out   tok : [B] or NULL
 *   x_conv : [B,D] io_dtype out
 */
int rglru_decode_conv(const void* x_in, const float* conv_w, const float* conv_b, void* conv_state,
                      const uint8_t* tok, void* x_conv, int B, int D, int io_dtype, void* stream);

/* rglru_decode_step: h <- a h + b for one token and y = h (griffin/griffin.py:237-258 at T = 1,
 * the sequential branch :280-286 that decode always takes).
 *   x, u_r, u_i : [B,D] io_dtype   h : [B,D] fp32 in/out   tok : [B] or NULL   y : [B,D] io_dtype out
 */
int rglru_decode_step(const void* x, const void* u_r, const void* u_i, const float* lambda, float* h,
                      const uint8_t* tok, void* y, int B, int D, float c, int io_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RGLRU_B200_H */
