// Interface of the tcgen05 (tensor-core) kernel family towards the C ABI dispatcher.
#pragma once
#include "common.cuh"

namespace pcb {

// True when a tensor-core kernel exists for this pass / dtype / variant / geometry.
bool tensor_path_supported(Pass pass, int dtype, int variant, const Geom& g);
// Scratch bytes (beyond the workspace header) the tensor-core kernel of this problem needs.
size_t tensor_scratch_bytes(Pass pass, int dtype, int variant, int engine, const Geom& g);
// Operand roles as for simt_launch. `status` is the device status word of the workspace header.
// A staged tensor that another pass already made: where it lies and how it is padded.
struct StagedView {
    const void* base = nullptr;
    int Hp = 0, Wp = 0, pad_top = 0, pad_left = 0;   // padded plane and the position of pixel (0, 0) inside it
};
// What a filter-gradient pass may take over from other passes instead of staging it again:
// `kept_x`: the staged copy of x that the forward call of the same layer left in ITS workspace scratch (see
//           forward_keeps_staged_input);
// `dy`:     the padded copy of dy that the backward-data pass of the same call staged (see backward_shares_staged_dy);
// `scratch_offset`: bytes of the workspace scratch to leave alone (they hold that copy).
struct PassExtras {
    const void* kept_x = nullptr;
    StagedView dy;
    size_t scratch_offset = 0;
};
int tensor_launch(Pass pass, int dtype, int variant, const Geom& g, const void* a, const void* b, const void* bias,
                  void* out, float* scratch, int* status, cudaStream_t stream, const PassExtras* extras = nullptr);
// True when the backward-data pass of this layer stages dy (at the start of its scratch, `bytes` long) in a layout its
// filter gradient can read through a tensor map: stride-1 layers on the narrow pair of kernels, or on the general pair with
// one channel block per component. `view` receives the padded geometry (its base is left null).
bool backward_shares_staged_dy(int dtype, int variant, const Geom& g, StagedView* view, size_t* bytes);
// True when the forward pass of this layer stages x, at the start of its scratch, in exactly the layout its filter
// gradient reads: a narrow forward with a narrow filter gradient, or the general pair with one channel block per component.
bool forward_keeps_staged_input(int dtype, int variant, const Geom& g);

// Persistent TMA-fed kernel for wide pointwise layers (forward and backward-data); see pointwise_tc.cu.
bool pointwise_tc_supported(Pass pass, int dtype, int variant, const Geom& g);
int pointwise_tc_launch(Pass pass, int dtype, const Geom& g, const void* w, const void* act, const void* bias, void* out,
                        int* status, cudaStream_t stream);

// The forward kernel on pairs of SMs (cta_group::2 MMAs) for layers with a multiple of 256 output channels; see pointwise2_tc.cu.
bool pointwise_pair_tc_supported(Pass pass, int dtype, int variant, const Geom& g);
int pointwise_pair_tc_launch(int dtype, const Geom& g, const void* w, const void* x, const void* bias, void* y, int* status, cudaStream_t stream);
bool pointwise_filter_pair_tc_supported(const Geom& g);
int pointwise_filter_pair_tc_launch(int fmt, const Geom& g, const void* dy, const void* x, float* scratch, int* status, cudaStream_t stream);

bool pointwise_filter_tc_supported(int dtype, int variant, const Geom& g);
int pointwise_filter_tc_launch(int dtype, const Geom& g, const void* dy, const void* x, void* dw, float* scratch, int* status,
                               cudaStream_t stream);

// The factorised 8-product form of pointwise layers (all three passes) with the lane sums formed in shared memory and the
// recombination in the epilogue; see pointwise8_tc.cu.
bool pointwise8_tc_supported(Pass pass, int dtype, int variant, const Geom& g);
size_t pointwise8_tc_scratch_bytes(Pass pass, const Geom& g);
int pointwise8_tc_launch(Pass pass, int dtype, const Geom& g, const void* a, const void* b, const void* bias, void* out,
                         float* scratch, int* status, cudaStream_t stream);

// General implicit-GEMM convolution (any taps / stride <= 2 / padding) on staged operands; see conv_tc.cu.
bool conv_tc_supported(Pass pass, int dtype, int variant, const Geom& g);
size_t conv_tc_scratch_bytes(Pass pass, const Geom& g);
int conv_tc_launch(Pass pass, int dtype, const Geom& g, const void* w, const void* act, const void* bias, void* out,
                   void* scratch, int* status, cudaStream_t stream);

bool conv_filter_tc_supported(int dtype, int variant, const Geom& g);
size_t conv_filter_tc_scratch_bytes(const Geom& g);
int conv_filter_tc_launch(int dtype, const Geom& g, const void* dy, const void* x, void* dw, void* scratch, int* status,
                          cudaStream_t stream, const void* kept_x = nullptr, const StagedView* kept_dy = nullptr);
// Geometry of the copy of dy that the general backward-data kernel stages; false when it inserts zeros (strided layers) or
// the filter gradient would block its channels.
bool conv_tc_staged_dy_view(const Geom& g, StagedView* view, size_t* bytes);
// The filter gradient stages x as [component][image][h][w][channels], the layout of the forward pass.
bool conv_filter_tc_stages_like_forward(const Geom& g);

// Narrow layers (<= 16 reduced channels, stride-1 correlation): halo tiles in shared memory serve every tap; see narrow_tc.cu.
bool narrow_tc_supported(Pass pass, int dtype, int variant, const Geom& g);
size_t narrow_tc_scratch_bytes(Pass pass, const Geom& g);
int narrow_tc_launch(Pass pass, int dtype, const Geom& g, const void* w, const void* act, const void* bias, void* out, void* scratch,
                     int* status, cudaStream_t stream);

bool narrow_filter_tc_supported(int dtype, int variant, const Geom& g);
size_t narrow_filter_tc_scratch_bytes(const Geom& g);
int narrow_filter_tc_launch(int dtype, const Geom& g, const void* dy, const void* x, void* dw, void* scratch, int* status, cudaStream_t stream,
                            const void* kept_x = nullptr, const StagedView* kept_dy = nullptr);
bool narrow_tc_staged_dy_view(const Geom& g, StagedView* view, size_t* bytes);

// fp32 tensors on the tensor cores with error-compensated TF32 (convolution and dense); see conv_tf32.cu.
bool conv_tf32_supported(Pass pass, int dtype, int variant, const Geom& g);
size_t conv_tf32_scratch_bytes(Pass pass, const Geom& g);
int conv_tf32_launch(Pass pass, const Geom& g, const void* a, const void* b, const void* bias, void* out, void* scratch, int* status,
                     cudaStream_t stream);

}  // namespace pcb
