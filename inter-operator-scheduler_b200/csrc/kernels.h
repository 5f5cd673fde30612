// Device-side operator library: parameter blocks and host launchers.
//
// Activations live in HBM as NHWC, float32 or (precision "bf16") bfloat16, with a per-pixel pitch
// in elements that keeps every pixel row on a 16-byte boundary (a multiple of 4 floats / 8 bf16).
// A TensorRef addresses a channel window of such a buffer: element (n, h, w, c) is
// ptr[((n*H + h)*W + w)*pitch + c] in units of its element size.  Channel slices, concat
// members and whole tensors are all TensorRefs, which is what lets a producer write straight into
// its slot of a consumer's concat buffer and a consumer read a slice of a merged convolution
// without the copy kernels of the reference (src/ios/ops.cu:6-24).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace ios {

struct TensorRef {
    void *ptr = nullptr;
    int N = 0, H = 0, W = 0, C = 0;
    int pitch = 0;   // elements between consecutive pixels
    int esize = 4;   // bytes per element: 4 = float32, 2 = bfloat16

    __host__ __device__ long pixels() const { return long(N) * H * W; }
    // May the kernels move 4 elements per access?  C need not be a multiple of 4: the last group of a
    // pixel is loaded whole (the bytes past the window belong to the same arena) and stored element by element.
    bool vec4() const {
        return (pitch % 4 == 0) && ((reinterpret_cast<uintptr_t>(ptr) % size_t(4 * esize)) == 0);
    }
    // the same tensor seen from `channels` further along the channel axis
    TensorRef shifted(int channels) const {
        TensorRef t = *this;
        t.ptr = static_cast<char *>(ptr) + size_t(channels) * esize;
        return t;
    }
    template <class T>
    __host__ __device__ T *as() const { return static_cast<T *>(ptr); }
};

#ifdef __CUDACC__
// First statement of every kernel that runs inside a schedule.  A captured schedule may connect kernels
// by programmatic dependencies: a kernel is then started before its predecessors have finished and must
// wait here before it reads or writes anything they touch; its own successors may be started at once.
// Without such a dependency both instructions do nothing.
__device__ __forceinline__ void grid_dependency_entry() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

constexpr int kMaxSumInputs = 8;

// out = act(in_0 (+|*) in_1 ... in_{k-1}); k = 1 with act = identity is a strided copy.
struct SumActParams {
    const void *in[kMaxSumInputs];
    int in_pitch[kMaxSumInputs];
    void *out;
    int out_pitch;
    int esize;       // element size of every operand (4 or 2)
    int k;
    int C;
    long pixels;
    int act;   // Act
    int mul;   // 1: product instead of sum
    int round_out;   // 1: round the stored result to TF32
};
void launch_sum_act(const SumActParams &p, bool vec4, cudaStream_t stream);

struct PoolParams {
    TensorRef in, out;
    int kh, kw, sh, sw, ph, pw;
    int is_max;
    int round_out;   // 1: round the stored result to TF32
};
void launch_pool(const PoolParams &p, cudaStream_t stream);

// NCHW dense <-> NHWC TensorRef
void launch_nchw_to_nhwc(const float *src, TensorRef dst, bool round_tf32, cudaStream_t stream);
void launch_nhwc_to_nchw(TensorRef src, float *dst, cudaStream_t stream);

// Deterministic pseudo-random fill in [-scale, scale] (synthetic weights / inputs for timing runs);
// esize 4 writes float32, esize 2 bfloat16.
void launch_fill(void *dst, long count, uint32_t seed, float scale, cudaStream_t stream, int esize = 4);

// ---- convolution ---------------------------------------------------------------------------
struct ConvGeom {
    int N, Cin, H, W;      // input
    int Cout, OH, OW;      // output
    int kh, kw, sh, sw, ph, pw, groups;
    int act;
    int pre_relu;          // apply ReLU to the input while reading it (fused ReLU -> conv)
    int round_out;         // round the stored result to TF32: every consumer is a tensor-core convolution
};

// CUDA-core convolution for every shape the tensor-core kernel does not take (grouped, unaligned
// views, precision "fp32").  Weights: [tap][Cin/groups][Cout] float32.
struct ConvDirectParams {
    TensorRef in, out;
    const float *weight;
    const float *bias;
    ConvGeom g;
};
void launch_conv_direct(const ConvDirectParams &p, cudaStream_t stream);
// Does launch_conv_direct have its fast form for this layer (at most 4 input channels, Cout % 4 == 0,
// 16-byte aligned pixels)?  Such layers are bound by the bytes they write and are kept off the tensor cores.
bool conv_few_channels_supported(const TensorRef &in, const TensorRef &out, const ConvGeom &g);
// Depthwise (groups == Cin == Cout).  Weights: [tap][C rounded up to 4] float32, zero padded.
void launch_conv_depthwise(const ConvDirectParams &p, cudaStream_t stream);

// Tensor-core implicit-GEMM convolution (tcgen05 + TMEM + TMA), groups == 1.
// Packed weights: [planes][Cout_pad][taps][cchunks*chunk], zero padded, chunk = one 128-byte row
// (32 float32 or 64 bfloat16); plane 0 holds the weights rounded to TF32 (or bfloat16), plane 1
// (three-pass mode only) the TF32-rounded residuals.
struct ConvTcPlan {
    // tile geometry chosen by conv_tc_plan()
    int box_w, box_h, box_n;       // output pixels covered by one M tile along W, H, batch
    int tiles_w, tiles_h, tiles_n; // number of M tiles along each
    int bn;                        // output channels per CTA (UMMA N)
    int n_tiles;                   // ceil(Cout / bn)
    int cchunks;                   // ceil(Cin / 32)
    int k_iters;                   // taps * cchunks
    int split_k;                   // CTAs sharing one output tile
    int stages;                    // smem pipeline depth
    int flat_1x1;                  // 1: pixels flattened into one axis (1x1, stride 1, no padding)
    int persistent;                // 1: CTAs stay resident and walk the tiles (grids of several waves, split_k == 1)
    int grid_ctas;                 // CTAs launched
    int no_persistent;             // testing aid: never use the persistent kernel
    int half_rows;                 // 1: bfloat16 layer of at most 32 input channels: 64-byte operand rows (32 K elements per step)
    int no_half_rows;              // testing aid: such layers use 128-byte rows like the rest
    int max_producers;             // testing aid: cap on the lanes that issue TMA loads (0: the default, 4)
    int im2col;                    // 1: pixels flattened into one axis, activations fetched by im2col-mode TMA
    int x3;                        // 1: three-pass TF32 (operands split into value + residual)
    int tma_store;                 // 1: the output window is 16-byte aligned, the epilogue uses bulk tensor stores
    int pdl;                       // 1: launch with programmatic stream serialization
    int cluster;                   // 1: a K split of up to 8 is reduced inside a thread-block cluster
    int push;                      // 1: (cluster) partial tiles are pushed into the shared memory of the CTA that finishes their rows
    int no_dual;                   // testing aid: three-pass mode issues all products from one thread
    int no_push;                   // testing aid: the cluster reduction always goes through the workspace in L2
    int recv_off;                  // byte offset of the area the pushes land in
    int bf16;                      // 1: bfloat16 operands and activations (kind::f16), 0: float32 storage (kind::tf32)
    int sm_count;                  // SMs of the device the tiling was chosen for
    size_t smem_bytes;
    size_t workspace_bytes;        // split-K partial tiles (0 when split_k == 1)
    size_t counter_bytes;          // split-K arrival counters
    int cout_pad;                  // rows of the packed weight matrix
    // patch convolution (conv_tc_patch.cu): stride-1 windows, every input pixel loaded once per tile
    int patch;                     // 1: this plan runs as a patch convolution
    int no_patch;                  // testing aid: never do
    int patch_all;                 // testing aid: every stride-1 window the cost model favours, not only resident-weight layers
    int patch_pw, patch_ph;        // patch extent per image (input pixels): tile outputs plus the window's halo
    int patch_a_rows;              // rows of one activation stage
    int patch_a_stages, patch_b_stages;
    int patch_b_resident;          // 1: the packed weights are loaded once per CTA and stay in shared memory
    int patch_merged;              // 1: one-row windows: images and rows are one axis
    int patch_issuers;             // warps that issue tcgen05.mma (1..4)
    int patch_b_depth;             // weight stages per issuer (every issuer has a ring of its own)
    int max_issuers;               // testing aid: cap on patch_issuers (0: none)
    int patch_bulk_store;          // testing aid: 1 = finished patch tiles leave through bulk tensor stores (one per row segment)
    int patch_staging;             // bytes of store staging in shared memory (0: finished tiles are stored from registers)
    alignas(64) unsigned char tmap_a[128];   // CUtensorMap over the input view
    alignas(64) unsigned char tmap_b[128];   // CUtensorMap over the packed weights
    alignas(64) unsigned char tmap_c[128];   // CUtensorMap over the output window (when tma_store)
};
struct ConvTcParams {
    TensorRef in, out;
    const void *weight_packed;
    const float *bias;
    float *workspace;
    unsigned int *counters;
    int *error_flag;               // device word set to non-zero when a bounded wait ran out
    long long *timeline;           // optional diagnostics: 16 SM-clock stamps written by CTA (0,0,0), or null
    const void *next_weights;      // packed weights of the tensor-core convolution launched after this one (or null) ...
    unsigned next_weight_bytes;    // ... and how many of their bytes to ask into L2 while this kernel runs
    ConvGeom g;
};
// Returns false when the shape / view cannot use the tensor-core kernel.
bool conv_tc_supported(const TensorRef &in, const ConvGeom &g);
// Chooses the tiling; sm_count and concurrency_hint (groups running beside this one) steer bn and
// split_k.  three_pass selects the fp32-grade 3xTF32 product.  Does not touch the device.
void conv_tc_choose(const ConvGeom &g, int sm_count, int concurrency_hint, bool three_pass, ConvTcPlan *plan,
                    int force_bn = 0, bool bf16 = false, bool allow_im2col = true);
// Overrides the K split (recomputes pipeline depth, shared memory and workspace sizes).
void conv_tc_set_split(ConvTcPlan *plan, int split);
// Encodes the two tensor maps (needs final device addresses).  Returns a CUDA driver error text or nullptr.
const char *conv_tc_encode(const ConvTcParams &p, ConvTcPlan *plan);
// Variant of conv_tc_encode for a 1x1 convolution whose weights stay in the caller's dense
// [Cout][Cin] float32 array (single-pass TF32 only: nothing is packed or split).
const char *conv_tc_encode_dense_weights(const ConvTcParams &p, ConvTcPlan *plan);
// Raises the kernel's dynamic shared-memory limit; call once per device before the first launch.
cudaError_t conv_tc_prepare();
void launch_conv_tc(const ConvTcParams &p, const ConvTcPlan &plan, cudaStream_t stream);
// Patch convolution: may take over a plan that conv_tc_choose gave to the resident-CTA kernel (call it right
// after conv_tc_choose / conv_tc_set_split and before the weights are sized and packed).
void conv_tc_patch_consider(const ConvGeom &g, int sm_count, ConvTcPlan *plan);
cudaError_t conv_tc_patch_prepare();
void launch_conv_tc_patch(const ConvTcParams &p, const ConvTcPlan &plan, cudaStream_t stream);
size_t conv_tc_packed_bytes(const ConvGeom &g, const ConvTcPlan &plan);
// Host-side packing of OIHW weights into the tensor-core layout (rounds to TF32 or bfloat16, nearest even).
void conv_tc_pack_weights(const float *oihw, const ConvGeom &g, const ConvTcPlan &plan, void *packed);
// Host-side packing for the CUDA-core kernels.
void conv_direct_pack_weights(const float *oihw, const ConvGeom &g, float *packed);   // [tap][Cin/g][Cout]
void conv_depthwise_pack_weights(const float *oihw, const ConvGeom &g, float *packed); // [tap][C rounded up to 4]

}  // namespace ios
