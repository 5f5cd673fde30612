// Lowering of a scheduled Model to a list of kernel launches over one device arena.
//
// Replaces Graph::map / unmap and the per-operator map() methods of the reference
// (src/ios/ios_runtime.cu:1273-1285, 1318-1327, 263-307, 639-651, 700-717, 776-787), which issue
// one cudaMalloc per operator output and per assembled input:
//  * every tensor is a channel window of an NHWC buffer inside ONE arena, sized by a dry lowering
//    pass, so building a plan performs no allocation once the arena has grown;
//  * a value that is a channel slice is a pointer offset (at every batch size, not only batch 1);
//  * a concat whose terms are whole operator outputs is performed by placement: the producers are
//    given their window of the concat buffer as output, so no copy kernel runs;
//  * other assembled inputs (sums, partial slices) are built by one sum/copy launch per term,
//    fused with the consumer when the consumer is an element-wise operator.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "graph.h"
#include "kernels.h"

namespace ios {

struct Options {
    bool tf32 = true;           // precision: tensor cores (tf32x3 / tf32) or CUDA cores (fp32)
    bool three_pass = true;     // tf32x3: operands split into TF32 value + residual, fp32-grade products
    bool bf16 = false;          // precision "bf16": bfloat16 activations and weights, fp32 accumulation
    bool pdl = true;            // programmatic dependent launch between consecutive convolution kernels
    bool stage_barriers = true; // join all groups after every stage (the reference's semantics); false: data-flow edges
    bool use_graph = true;      // executor: CUDA graph or plain streams
    bool pdl_edges = false;     // captured graphs: every kernel -> kernel edge becomes a programmatic dependency
    bool allow_tc = true;       // conv: auto or direct
    int force_split_k = 0;      // testing aid: > 0 overrides the split-K choice
    int force_bn = 0;           // testing aid: > 0 overrides the output-channel tile width
    int force_stages = 0;       // testing aid: > 0 caps the depth of the shared-memory pipeline
    int producers = 0;          // testing aid: > 0 caps the lanes that issue TMA loads in the convolution kernel
    bool no_stem_kernel = false; // testing aid: convolutions over at most 4 input channels take the tensor-core kernel too
    bool no_half_rows = false;  // testing aid: bfloat16 layers of at most 32 input channels keep 128-byte operand rows
    int patch_issuers = 0;      // testing aid: > 0 caps the warps that issue tcgen05.mma in the patch convolution
    bool patch_bulk_store = false; // testing aid: patch convolutions store finished tiles with bulk tensor stores
    bool patch_all = false;     // testing aid: patch convolutions also for layers that stream their weights
    bool no_patch = false;      // testing aid: stride-1 windows load an activation tile per tap instead of one patch per tile
    bool no_weight_prefetch = false; // testing aid: a convolution does not ask the next one's weights into L2
    bool no_dual_issue = false; // testing aid: three-pass convolutions issue all their products from one thread
    bool no_cluster_push = false; // testing aid: split-K clusters exchange partial tiles through L2 instead of shared memory
    bool no_persistent = false; // testing aid: grids of several waves launch one CTA per tile instead of resident CTAs
    bool no_im2col = false;     // testing aid: windows with taps tile the image in boxes instead of the flat pixel axis
    bool no_bulk_store = false; // testing aid: the epilogue stores straight from registers
    bool timeline = false;      // diagnostics: the tensor-core kernel stamps its phases (see conv_tc.cu)
};

enum class StepKind { SumAct, Pool, ConvTc, ConvDirect, ConvDepthwise };

struct Step {
    StepKind kind;
    int stage = 0, group = 0;
    int op = -1;                // operator that caused the launch (reporting)
    bool vec4 = false;
    SumActParams sum;
    PoolParams pool;
    ConvDirectParams direct;
    ConvTcParams tc;
    ConvTcPlan tcplan;
};

struct ConvSlot {               // where a convolution's parameters live in the arena
    int op;
    StepKind impl;
    ConvGeom geom;
    ConvTcPlan tcplan;
    size_t weight_offset, weight_bytes;
    size_t bias_offset;
};

struct Plan {
    Model model;
    Options options;
    std::vector<Step> steps;               // in stage, group, launch order
    std::vector<ConvSlot> convs;
    std::vector<TensorRef> tensors;        // output window of every operator
    std::vector<size_t> input_offsets;     // arena offset of every placeholder buffer
    size_t arena_bytes = 0;                // activations + workspaces + weights + staging
    size_t zero_begin = 0, zero_bytes = 0; // split-K counters: must start at zero
    size_t staging_in_offset = 0, staging_out_offset = 0;   // NCHW staging for host transfers
    size_t error_flag_offset = 0;
    size_t workspace_bytes = 0;
    std::vector<size_t> group_workspace_bytes;   // split-K workspace shared by the convolutions of each group slot
    bool input_round_tf32 = false;
    int launches_per_forward = 0;
    int max_groups = 1;
};

// Two-pass construction: plan_layout() sizes the arena (no device access), plan_bind() lowers
// against the real base address, encodes tensor maps.  Both throw GraphError / std::runtime_error.
void plan_layout(Plan *plan, int sm_count);
void plan_bind(Plan *plan, char *arena_base, int sm_count);

}  // namespace ios
