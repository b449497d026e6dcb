// Host-side declarations shared between the C ABI layer and the kernel files.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace rglru {

// Time-steps between saved recurrent states == chunk length of the backward kernel.
constexpr int SAVE_EVERY = 64;
// Largest batch for which the backward kernel folds the dLambda rows itself (one CTA walks B x D floats).
constexpr int FUSED_DLAMBDA_MAX_B = 64;
constexpr size_t WS_TAIL_BYTES = 256;  // completion ticket at the end of the workspace

struct ScanFwdArgs {
  const void* x;
  const void* ur;
  const void* ui;
  void* y;
  const float* lambda;
  const float* h0;
  const uint8_t* tok;
  float* h_last;
  float* decay_prod;  // [B, D] product of the (masked) decays over the whole sequence, or nullptr
  float* states;  // [B, ceil(T/SAVE_EVERY), D] or nullptr
  unsigned* ticket;  // completion counter of the workspace (zeroed here for the backward), or nullptr
  // conv-folded variant only: x is the conv INPUT; taps [D,4], bias [D] or nullptr, carried history [B,3,D] or nullptr
  const float* conv_w;
  const float* conv_b;
  const void* conv_state;
  const void* g;     // merged variant only: pre-activation of the GeLU branch [B, T, D]; y receives h * gelu(g)
  // grouped gate layout only: ur == ui == one [B, T, 2 D] tensor, gate_bw channels per gate head,
  // gate_bias [2 D] fp32 in the same column layout or nullptr
  const float* gate_bias;
  int gate_bw;
  bool paired;  // the four tensor maps are the 5-D paired-row form (32-channel bf16 forward without flags)
  int B, T, D;
  float c;
  int* status;
};

struct ScanBwdArgs {
  const void* dy;
  const void* x;
  const void* ur;
  const void* ui;
  void* dx;
  void* dur;
  void* dui;
  const float* lambda;
  const float* h0;
  const float* dh_last;
  const uint8_t* tok;
  const float* states;  // written by the forward kernel
  float* dlam_part;     // [B, D] per-row partial sums of dl * r
  float* dlambda;       // [D]
  float* dh0;           // [B, D] or nullptr
  unsigned* ticket;     // when set, the last CTA folds dlam_part into dlambda; else a second kernel does
  const float* conv_w;  // conv-folded variant only (see ScanFwdArgs)
  const float* conv_b;
  const void* conv_state;
  const void* g;        // merged variant only: dy is then the gradient of h * gelu(g), dg receives that of g
  void* dg;
  const float* gate_bias;   // grouped gate layout only (see ScanFwdArgs); dur / dui then share that layout too
  int gate_bw;
  // grouped gate layout only: per-row partial column sums of du [B, 2 D] (workspace) and, when the caller wants
  // the gate-bias gradient, their fold over the batch [2 D]; both in the gate tensor's column layout
  float* dgate_part;
  float* dgate;
  int B, T, D;
  float c;
  int* status;
};

struct FwdMaps {
  CUtensorMap x, ur, ui, y, g;
};
struct BwdMaps {
  CUtensorMap dy, x, ur, ui, dx, dur, dui, g, dg;
};

struct RawFwdMaps {
  CUtensorMap drive, decay, out;
};
struct RawBwdMaps {
  CUtensorMap dout, decay, out, ddecay, ddrive;
};
struct RawScanArgs {
  const float* dout;   // backward only
  const float* decay;
  const float* drive;  // forward only
  const float* h0;
  const float* out_in;  // backward: saved forward output
  float* out;           // forward output
  float* ddecay;
  float* ddrive;
  float* dh0;
  int B, T, D;
  int* status;
};

// TMA-staged conv kernels: forward uses in0 = input (box of 67 rows), out0 = result; backward uses
// in0 = upstream gradient (67 rows), in1 = input (67 rows), out0 = input gradient.
struct ConvMaps {
  CUtensorMap in0, in1, out0;
};
struct ConvTmaArgs {
  const float* w;
  const float* bias;
  const void* state;     // [B, 3, D] history before t = 0 or nullptr
  const uint8_t* tok;
  void* d_state;         // backward only: gradient of the history, or nullptr
  float* part;           // backward only: partial rows [B, 5, D]
  int B, T, D;
  int* status;
};

struct ConvArgs {
  const void* x_in;
  const float* w;
  const float* bias;
  const void* state;  // history before t = 0 (forward) or nullptr
  const uint8_t* tok;
  void* out;
  void* new_state;  // decode: the in/out state
  int B, T, D;
  bool vector_ok;   // D and all pointers allow 16-byte accesses
  const ConvMaps* maps;   // non-null: the shape is staged by TMA (see launch_conv_tma_fwd)
  int* status;
};
struct ConvBwdArgs {
  const void* d_conv;
  const void* x_in;
  const float* w;
  const void* state;
  const uint8_t* tok;
  void* dx_in;
  float* d_w;
  float* d_b;
  void* d_state;
  float* part;
  int B, T, D;
  bool vector_ok;
  const ConvMaps* maps;   // non-null: the shape is staged by TMA (see launch_conv_tma_bwd)
  int* status;
};
struct DecodeArgs {
  const void* x;
  const void* ur;
  const void* ui;
  const float* lambda;
  float* h;
  const uint8_t* tok;
  void* y;
  int B, D;
  float c;
  bool vector_ok;
};

cudaError_t launch_raw_fwd(bool use_tma, const RawFwdMaps& maps, const RawScanArgs& args, cudaStream_t s);
cudaError_t launch_raw_bwd(bool use_tma, const RawBwdMaps& maps, const RawScanArgs& args, cudaStream_t s);
int raw_box_rows();
cudaError_t launch_conv_fwd(bool bf16, const ConvArgs& a, cudaStream_t s);
cudaError_t launch_conv_bwd(bool bf16, const ConvBwdArgs& a, cudaStream_t s);
int conv_bwd_partial_rows(int B, int T);
cudaError_t launch_conv_tma_fwd(bool bf16, const ConvMaps& maps, const ConvTmaArgs& a, cudaStream_t s);
cudaError_t launch_conv_tma_bwd(bool bf16, const ConvMaps& maps, const ConvTmaArgs& a, cudaStream_t s);
int conv_tma_box_rows();
int conv_tma_box_cols();
cudaError_t launch_decode_conv(bool bf16, const ConvArgs& a, cudaStream_t s);
cudaError_t launch_decode_step(bool bf16, const DecodeArgs& a, cudaStream_t s);
int colsum_row_blocks(long long rows, int cols);   // partial rows a column-sum call leaves in its workspace
cudaError_t launch_column_sums(bool bf16, const void* src, float* out, float* part, long long rows, int cols,
                               bool vector_ok, cudaStream_t s);

// use_tma == false selects the bounds-checked plain-load staging path that accepts any D.
// `variant` picks the CTA shape (see scan_fwd_variant); the tensor maps must be encoded with its box rows.
cudaError_t launch_scan_fwd(bool bf16, bool use_tma, int variant, const FwdMaps& maps, const ScanFwdArgs& args,
                            cudaStream_t s);
cudaError_t launch_scan_bwd(bool bf16, bool use_tma, int variant, const BwdMaps& maps, const ScanBwdArgs& args,
                            cudaStream_t s);
cudaError_t launch_conv_scan_fwd(bool bf16, bool use_tma, const FwdMaps& maps, const ScanFwdArgs& args, cudaStream_t s);
cudaError_t launch_conv_scan_bwd(bool bf16, bool use_tma, const BwdMaps& maps, const ScanBwdArgs& args, cudaStream_t s);
cudaError_t launch_merge_fwd(bool bf16, bool use_tma, bool conv, const FwdMaps& maps, const ScanFwdArgs& args, cudaStream_t s);
cudaError_t launch_merge_bwd(bool bf16, bool use_tma, bool conv, const BwdMaps& maps, const ScanBwdArgs& args, cudaStream_t s);
cudaError_t launch_grouped_fwd(bool bf16, bool merge, const FwdMaps& maps, const ScanFwdArgs& args, cudaStream_t s);
cudaError_t launch_grouped_bwd(bool bf16, bool merge, const BwdMaps& maps, const ScanBwdArgs& args, cudaStream_t s);
int grouped_box_cols();
int scan_fwd_variant(int B, int T, int D, bool bf16);
int scan_bwd_variant(int B, int T, int D, bool bf16);
int scan_fwd_box_rows(int variant);
int scan_fwd_box_cols(int variant);
// True when the call takes the paired-row tile layout, whose tensor maps are 5-D (see rglru_fwd_body).
bool scan_fwd_paired(int variant, bool bf16, const void* tok, int T);
int scan_bwd_box_rows(int variant);
int scan_bwd_box_cols(int variant);
int raw_box_cols();

cudaError_t launch_wait_selftest(int* status, int* finished, long long limit_cycles, cudaStream_t s);

int* device_status_word();  // device address of the status word of the current device

// Remember a CUDA error for rglru_last_cuda_error() (per host thread) and return RGLRU_ERR_LAUNCH.
int record_cuda_error(cudaError_t e);

}  // namespace rglru
