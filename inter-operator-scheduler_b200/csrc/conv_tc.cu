// Implicit-GEMM convolution on the 5th-generation tensor cores (sm_100a): tcgen05.mma with the
// accumulator in tensor memory, both operands staged in shared memory by TMA, one CTA per
// (pixel tile, output-channel tile, K split) -- or resident CTAs that walk the tiles.
//
// GEMM view of y = act(conv(x, w) + b), groups == 1:
//     D[pixel, cout] = sum over taps (r, s) and input channels c of  X[pixel @ tap, c] * Wp[cout, tap, c]
// * M (128 TMEM lanes) = 128 consecutive pixels of the flattened (n, oh, ow) axis.  A 1x1 stride-1
//   convolution fetches them with a plain tiled TMA box over the NHWC input; every other window with an
//   im2col-mode TMA load (bounding-box corners = -padding and the last window corner, element strides =
//   the convolution's stride, the tap is the instruction's im2col offset).  Positions outside the image
//   and channels beyond Cin read zeros, so K needs no padded activation copy.  (Option im2col=0 keeps the
//   older form: a box_w x box_h x box_n rectangle of output pixels per tile, one tiled load per tap.)
// * N = bn output channels (32..256), K advances one 128-byte swizzle row per step (32 floats, four
//   tcgen05.mma.kind::tf32 of K = 8; 64 bfloat16, four kind::f16 of K = 16; bfloat16 layers of at most 32
//   input channels use 64-byte rows, two instructions per step).  Three-pass TF32: the weight tile and its
//   residual lie behind one another, one instruction of width 2 bn forms a_hi*w_hi | a_hi*w_lo, a second
//   adds a_lo*w_hi; the activation residual is computed from the landed tile by warps of their own.
//   Two threads issue: in three-pass mode one the wide instructions (as soon as a tile has landed), the
//   other a_lo*w_hi (once the residual is written) into an accumulator of its own; in the single-pass
//   modes each takes half of a K step's instructions.  The epilogue adds the accumulator ranges in a fixed order.
// * split_k CTAs share an output tile when the layer is too small to fill 148 SMs (batch 1).  Up to 8
//   of them form a thread-block cluster and exchange their fp32 partial tiles through distributed shared
//   memory: the tile's valid rows are dealt to the CTAs, every epilogue thread pushes its row (st.async, 16
//   bytes at a time) into the receive area of the CTA that finishes it, the bytes are counted on that CTA's
//   mbarrier, and the finishing CTA adds the S slices in split order, applies bias and activation and
//   stores.  When the receive area does not fit, partial tiles go to a workspace (it stays in L2) and one
//   cluster barrier precedes the same row-wise reduction.  Larger splits (a testing aid, and the
//   allocation-free entry point) elect the last CTA to arrive by one atomic ticket per tile.  In every
//   form the result does not depend on timing.
// * Epilogue: tcgen05.ld (one thread per pixel row), + bias, activation, optional rounding to TF32 for a
//   consumer convolution, then the tile is staged in shared memory (128-byte swizzle) and leaves through
//   bulk tensor stores into a channel window of the destination (NHWC, pitch) -- which is how
//   concat-by-placement and merged convolutions are written without a copy; windows that are not 16-byte
//   aligned, and the rows of a cluster reduction, are stored from registers.
// * While a three-pass convolution waits for its first tile it asks the packed weights of the next
//   convolution into L2 (they are read once per forward and the networks' weights do not fit the L2 together).
//
// Warp roles of conv_tc_kernel: warp 0 = TMA producer lanes (and barrier set-up, first weight tiles),
// warp 1 = MMA issuer (and tensor-map prefetch, first activation tiles), warps 2..5 = epilogue (warp 2
// allocates and frees tensor memory), warp 6 = second MMA issuer; three-pass mode: warps 7..10 = residual
// of the landed activation tiles, then half of the rows of a cluster reduction (192 / 224 / 352 threads).
// conv_tc_persistent_kernel (320 threads): one issuer, eight epilogue warps (three-pass mode: four, and four
// for the residual) and two accumulators in tensor memory, for grids of several waves.  Every wait on an
// mbarrier is bounded: when the bound is hit the kernel records a code in *error_flag, drains its own loads,
// frees its tensor memory and returns.  Stride-1 windows whose weights fit in shared memory take
// conv_tc_patch.cu instead.
//
// Replaces cudnnConvolutionBiasActivationForward / cudnnConvolutionForward + cudnnAddTensor
// (reference src/ios/ios_runtime.cu:313-331) and the algorithm search of :150-205.
#include "kernels.h"
#include "tc_device.h"

#include <type_traits>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdio>
#include <cstring>
#include <cmath>
#include <algorithm>
#include <vector>

namespace ios {
namespace {


struct TileGeom {
    int box_w, box_h, box_n;
    int tiles_w, tiles_h;
    int bn, cchunks, k_iters, split_k, stages;
    int flat;         // 1: a tile is box_w consecutive pixels of the flattened (n, oh, ow) axis
    int im2col;       // 1: (flat only) the window has taps, padding or strides: im2col-mode loads
    int a_bytes;      // bytes one A load delivers
    int tmem_cols;
    int round_tf32;   // round the stored result to TF32 (the consumer is a single-pass tensor-core convolution)
    int x3;           // 1: three-pass TF32 (value + residual of both operands), fp32-grade products
    int cout_pad;     // rows of one plane of the packed weight matrix
    int tma_store;    // 1: the epilogue stages the tile in shared memory and stores it with bulk tensor stores
    int cluster;      // 1: the split_k CTAs of a tile form a thread-block cluster and reduce through shared memory
    int bf16;         // 1: bfloat16 operands / activations (kind::f16), 0: float32 storage (kind::tf32)
    int chunk;        // elements of K per pipeline step: 32 (float32), 64 (bfloat16) or 32 (bfloat16, 64-byte rows)
    int slab;         // output channels per 128-byte row of the store staging: 32 (float32) or 64 (bfloat16)
    int producers;    // lanes of warp 0 that issue TMA loads; divides `stages`
    int wide;         // 1: (three-pass mode, bn <= 128) one instruction of width 2 bn covers the weight tile and its
                      //    residual; the residual's products accumulate in columns [bn, 2 bn)
    int dual;         // 1: (three-pass mode, wide) a second thread issues the products with the activation residual into an
                      //    accumulator of its own, columns [2 bn, 3 bn)
                      // 2: (single-pass modes) a second thread issues the second half of every K step's instructions into an
                      //    accumulator of its own, columns [bn, 2 bn)
    int split_shift;  // log2(split_k) when it is a power of two, else -1
    unsigned magic_ow, magic_cc, magic_kw;   // division by OW / cchunks / kw as a multiplication (0: divide)
    int push;         // 1: (cluster) partial tiles are pushed into the shared memory of the CTA that finishes their rows
    int recv_off;     // byte offset of the area those pushes land in (behind the pipeline stages and barriers)
};

// n / d for 0 <= n with n * d < 2^32, by the multiplier the host worked out (floor(2^32 / d) + 1); a CTA runs its
// prologue once, one thread per scheduler, so a division there is 100-400 cycles that nothing hides.
__device__ __forceinline__ int div_by(int n, int d, unsigned magic) {
    if (d == 1) return n;
    return magic ? int(__umulhi(unsigned(n), magic)) : n / d;
}
// n / d for n >= 0, d > 0, where d is most often a power of two
__device__ __forceinline__ int div_pow2_likely(int n, int d) {
    return (d & (d - 1)) == 0 ? n >> (31 - __clz(d)) : n / d;
}

// Optional diagnostics: CTA (0,0,0) stamps the SM clock at fixed points of its life.  The stamps sit
// in the single-thread role loops, where the mere test for them was measured at 3 % of batch-1
// latency, so they exist only in the kTimeline instantiations (option "timeline").
#define STAMP(slot)                                                                     \
    do {                                                                                \
        if (kTimeline && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) p.timeline[slot] = clock64(); \
    } while (0)

// Element offset of the output pixel that row `row` of a boxed (not flattened) pixel tile holds, or -1.
__device__ __noinline__ long boxed_pixel_offset(int row, int box_w, int box_h, int box_n, int ow0, int oh0, int n0, int N, int OH,
                                                int OW, int pitch) {
    const int ww = row % box_w;
    const int hh = (row / box_w) % box_h;
    const int im = row / (box_w * box_h);
    const int ow = ow0 + ww, oh = oh0 + hh, n = n0 + im;
    return (im < box_n && ow < OW && oh < OH && n < N) ? ((long(n) * OH + oh) * OW + ow) * pitch : -1;
}

// The MMA issuer's K loop, one copy per operand mode (0: TF32, 1: three-pass TF32, 2: BF16) so that the
// (3: three-pass TF32 with the weight tile and its residual under one instruction of twice the width,
//  4: BF16 with 64-byte operand rows, two instructions per K step)
// loop body carries no mode tests: wait for the stage, issue its instructions, hand the stage back.
// Position of the MMA issuer in the ring of pipeline stages (it outlives a tile in the persistent kernel).
struct MmaRing {
    uint64_t da0, db0, dal0, dbl0, dstep;   // descriptors of stage 0 and their step per stage (16-byte units)
    uint64_t da, db, dal, dbl;
    uint32_t s, phase;
    __device__ __forceinline__ void start(uint32_t smem_base, uint32_t a_lo_off, uint32_t b_off, uint32_t b_lo_off, int stage_bytes,
                                          int row_bytes) {
        da0 = smem_desc_kmajor(smem_base, row_bytes);
        db0 = smem_desc_kmajor(smem_base + b_off, row_bytes);
        dal0 = smem_desc_kmajor(smem_base + a_lo_off, row_bytes);
        dbl0 = smem_desc_kmajor(smem_base + b_lo_off, row_bytes);
        dstep = uint64_t(stage_bytes >> 4);
        da = da0; db = db0; dal = dal0; dbl = dbl0;
        s = 0; phase = 0;
    }
};

template <int MODE, bool kTimeline>
__device__ __forceinline__ bool mma_loop(int n_it, int stages, uint32_t wait0, uint32_t landed0, uint32_t empty0, MmaRing &ring,
                                         uint32_t tmem_d, uint32_t idesc, uint32_t idesc_wide, const ConvTcParams &p) {
#pragma unroll 1
    for (int i = 0; i < n_it; ++i) {
        const uint64_t da = ring.da, db = ring.db, dal = ring.dal, dbl = ring.dbl;
        if (MODE == 1 || MODE == 3) {
            // Three-pass mode: the products of the first activation tile as it landed (its TF32 value) start while
            // the residual warps are still writing the tile's residual; only the residual's product waits for them.
            // (Later tiles have their residual written while the tensor core is busy with the tile before: one wait.)
            if (!mbar_wait((i == 0 ? landed0 : wait0) + 8u * ring.s, ring.phase, p.error_flag)) return false;
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                if (MODE == 3) {
                    // a_hi*[w_hi | w_lo]: one instruction of twice the width
                    umma_tf32(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc_wide, acc);
                } else {
                    umma_tf32(tmem_d, da + uint64_t(k * 2), dbl + uint64_t(k * 2), idesc, acc);
                    umma_tf32(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, 1u);
                }
            }
        }
        if (!(MODE == 1 || MODE == 3) || i == 0) {
            if (!mbar_wait(wait0 + 8u * ring.s, ring.phase, p.error_flag)) return false;
            tc_fence_after();
        }
        if (i == 0) STAMP(3);
#pragma unroll
        for (int k = 0; k < (MODE == 4 ? 2 : 4); ++k) {   // 32 bytes of K per instruction: 8 TF32 or 16 BF16; 64-byte rows: two
            const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
            if (MODE == 1 || MODE == 3) {
                // a_lo*w_hi
                umma_tf32(tmem_d, dal + uint64_t(k * 2), db + uint64_t(k * 2), idesc, 1u);
            } else if (MODE == 2 || MODE == 4) {
                umma_f16(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, acc);
            } else {
                umma_tf32(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, acc);
            }
        }
        umma_commit(empty0 + 8u * ring.s);   // frees the stage once these MMAs have read it
        ring.da += ring.dstep; ring.db += ring.dstep; ring.dal += ring.dstep; ring.dbl += ring.dstep;
        if (++ring.s == uint32_t(stages)) {
            ring.s = 0; ring.phase ^= 1u;
            ring.da = ring.da0; ring.db = ring.db0; ring.dal = ring.dal0; ring.dbl = ring.dbl0;
        }
    }
    return true;
}

// Three-pass mode with two issuing threads: each runs this loop over its own pair of operand planes and its own
// accumulator, so neither waits for the other's instructions to be issued (one thread gets a tcgen05.mma out
// about every 90 cycles, whatever its width).  Both hand a stage back; the producer waits for the two of them.
// (Single-pass modes use it too: there the two threads share the instructions of a K step, k in [k0, k1) each.)
template <bool kTimeline, bool kF16 = false>
__device__ __forceinline__ bool mma_loop_planes(int n_it, int stages, uint32_t wait0, uint32_t empty0, uint64_t da0, uint64_t db0,
                                                uint64_t dstep, uint32_t tmem_d, uint32_t idesc, const ConvTcParams &p, bool stamp,
                                                int k0 = 0, int k1 = 4) {
    uint64_t da = da0, db = db0;
    uint32_t s = 0, phase = 0;
#pragma unroll 1
    for (int i = 0; i < n_it; ++i) {
        if (!mbar_wait(wait0 + 8u * s, phase, p.error_flag)) return false;
        if (i == 0 && stamp) STAMP(3);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (k < k0 || k >= k1) continue;
            const uint32_t acc = (i > 0 || k > k0) ? 1u : 0u;
            if (kF16) umma_f16(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, acc);
            else umma_tf32(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, acc);
        }
        umma_commit(empty0 + 8u * s);
        da += dstep; db += dstep;
        if (++s == uint32_t(stages)) { s = 0; phase ^= 1u; da = da0; db = db0; }
    }
    return true;
}

// ---- the kernel ------------------------------------------------------------------------------
// One instantiation per operand mode (0: TF32, 1: three-pass TF32, 2: BF16, 4: BF16 with 64-byte operand rows)
// and per reduction form
// (kCluster: the split_k CTAs of a tile are a cluster): a CTA runs its code once, so what it does not
// need should not be in its instruction stream.
template <int MODE, bool kCluster, bool kTimeline>
__global__ void __launch_bounds__(kThreads, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, const ConvTcParams p, const TileGeom t) {
    constexpr bool kX3 = MODE == 1, kBf16 = MODE == 2 || MODE == 4;
    constexpr int kRow = MODE == 4 ? 64 : 128;          // bytes of K per operand row (MODE 4: bfloat16, 64-byte rows)
    extern __shared__ uint8_t smem_raw[];
    __shared__ float bias_s[256];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    constexpr int a_tile_bytes = kTileM * kRow;
    const int b_bytes = t.bn * kRow;
    const int passes = kX3 ? 2 : 1;                       // operand planes per stage: value (+ residual)
    const int stage_bytes = passes * (a_tile_bytes + b_bytes);
    // stage layout: A | A residual | B | B residual
    const uint32_t a_lo_off = uint32_t(a_tile_bytes);
    const uint32_t b_off = uint32_t(passes) * a_tile_bytes;
    const uint32_t b_lo_off = b_off + uint32_t(b_bytes);
    const uint32_t bars = smem_base + uint32_t(t.stages) * stage_bytes;
    const uint32_t full0 = bars, empty0 = bars + 8u * t.stages, ready0 = bars + 16u * t.stages;
    const uint32_t accum_bar = bars + 24u * t.stages;
    const uint32_t recv_bar = accum_bar + 16u;
    volatile uint32_t *tmem_slot =
        reinterpret_cast<volatile uint32_t *>(generic_base + size_t(t.stages) * stage_bytes + 24 * t.stages + 8);
    volatile int *ticket_slot = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const ConvGeom &g = p.g;
    if (threadIdx.x == 0) STAMP(0);
    {
        // Kernel parameters are new with every launch, so the first read of each of their cache lines misses.
        // One word of every line is asked for here, all at once, instead of one miss at a time where the
        // epilogue first needs them.
        const int touch = p.in.pitch ^ p.out.pitch ^ int(reinterpret_cast<uintptr_t>(p.bias)) ^ int(reinterpret_cast<uintptr_t>(p.error_flag)) ^
                          g.N ^ g.act ^ g.round_out ^ t.box_w ^ t.tmem_cols ^ t.wide ^ t.recv_off;
        asm volatile("" ::"r"(touch));
    }

    // tile coordinates
    const int m_tile = blockIdx.x, n_tile = blockIdx.y, split = blockIdx.z;
    int ow0 = 0, oh0 = 0, n0 = 0, im_w = 0, im_h = 0;
    if (t.flat) {
        ow0 = m_tile * t.box_w;
        if (t.im2col) {
            // the tile's first pixel, as the corner of its filter window in input coordinates
            const int per_image = g.OH * g.OW;
            n0 = g.N == 1 ? 0 : ow0 / per_image;
            const int rem = ow0 - n0 * per_image;
            oh0 = div_by(rem, g.OW, t.magic_ow);
            im_w = (rem - oh0 * g.OW) * g.sw - g.pw;
            im_h = oh0 * g.sh - g.ph;
        }
    } else {
        const int tw = m_tile % t.tiles_w;
        const int rest = m_tile / t.tiles_w;
        ow0 = tw * t.box_w;
        oh0 = (rest % t.tiles_h) * t.box_h;
        n0 = (rest / t.tiles_h) * t.box_n;
    }
    const int cout0 = n_tile * t.bn;
    // K steps [split * k_iters / split_k, (split + 1) * k_iters / split_k)
    const int it_begin = t.split_shift >= 0 ? (split * t.k_iters) >> t.split_shift : int(unsigned(split * t.k_iters) / unsigned(t.split_k));
    const int it_end = t.split_shift >= 0 ? ((split + 1) * t.k_iters) >> t.split_shift : int(unsigned((split + 1) * t.k_iters) / unsigned(t.split_k));
    const int n_it = it_end - it_begin;
    // Push form of the cluster reduction: the tile's valid rows (a prefix of the 128 when the tile is a run of
    // consecutive pixels) are dealt to the CTAs of the cluster, `push_rpr` rows each; this CTA finishes `push_rows`
    // of them and receives, from every CTA of the cluster, those rows of that CTA's partial tile.
    const bool push = kCluster && t.push != 0;
    int push_vrows = 0, push_rpr = 0, push_rows = 0;
    if (push) {
        const long total = long(g.N) * g.OH * g.OW;
        push_vrows = t.flat ? int(max(0l, min(long(min(t.box_w, kTileM)), total - ow0))) : kTileM;
        push_rpr = t.split_shift >= 0 ? (push_vrows + t.split_k - 1) >> t.split_shift : (push_vrows + t.split_k - 1) / t.split_k;
        push_rows = max(0, min(push_rpr, push_vrows - int(cluster_cta_rank()) * push_rpr));
    }

    // Push form: one "item" is four output channels of one of the rows this CTA finishes.  Its position in the
    // receive area, its place in the output and its bias are worked out ahead of time (prepare_item); once the
    // rows have been received, finish_item adds the cluster's partial sums in split order and stores.
    auto prepare_item = [&](int item, int &src, long &at, int &count, float4 &bias) {
        src = -1;
        at = -1;
        count = 0;
        bias = make_float4(0.f, 0.f, 0.f, 0.f);
        if (item >= push_rows * (t.bn >> 2)) return;
        const int r0 = int(cluster_cta_rank()) * push_rpr;
        const int valid = min(t.bn, g.Cout - cout0);
        const int q4 = div_pow2_likely(item, push_rows), lr = item - q4 * push_rows, c = q4 << 2;
        src = q4 * push_rpr + lr;
        const long pix = long(ow0) + r0 + lr;
        const long pix_off = t.flat ? ((r0 + lr < t.box_w && pix < long(g.N) * g.OH * g.OW) ? pix * p.out.pitch : -1)
                                    : boxed_pixel_offset(r0 + lr, t.box_w, t.box_h, t.box_n, ow0, oh0, n0, g.N, g.OH, g.OW, p.out.pitch);
        if (pix_off >= 0 && c < valid) {
            at = pix_off + cout0 + c;
            count = valid - c;
            // (straight from global memory: the loads are in flight until the sums need them)
            float b[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = (p.bias && c + j < valid) ? __ldg(p.bias + cout0 + c + j) : 0.0f;
            bias = make_float4(b[0], b[1], b[2], b[3]);
        }
    };
    auto finish_item = [&](auto split_tag, int src, long at, int count, const float4 &bias) {
        constexpr int S = decltype(split_tag)::value;
        const float4 *recv = reinterpret_cast<const float4 *>(generic_base + t.recv_off);
        const int plane = (t.bn >> 2) * push_rpr;           // float4 from one partial tile to the next
        float4 part[S];
#pragma unroll
        for (int sp = 0; sp < S; ++sp) part[sp] = recv[max(src, 0) + sp * plane];
        float4 acc = part[0];
#pragma unroll
        for (int sp = 1; sp < S; ++sp) {
            acc.x += part[sp].x; acc.y += part[sp].y; acc.z += part[sp].z; acc.w += part[sp].w;
        }
        float o[4] = {acc.x + bias.x, acc.y + bias.y, acc.z + bias.z, acc.w + bias.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            o[j] = act_apply(o[j], g.act);
            if (t.round_tf32) o[j] = round_tf32(o[j]);
        }
        if (at >= 0) store4_direct(p.out.ptr, kBf16, at, make_float4(o[0], o[1], o[2], o[3]), count);
    };
    // Splits of 2, 4 and 8 have an unrolled form; three-pass mode has four more warps (those of the residual) that
    // take the second 128 items, so that a thread of either group has one item.
    const bool fast_split = t.split_k == 8 || t.split_k == 4 || t.split_k == 2;

    // Set-up is spread over three warps so that none of its chains follows another: warp 0 initialises the barriers
    // and requests the weight tiles, warp 1 fetches the tensor maps and requests the activation tiles, warp 2
    // allocates tensor memory.  The tiles of the first `stages` K steps are requested here, one lane per step (at
    // batch 1 a CTA of a split-K cluster has no more steps than that); the rest of the set-up runs while they
    // are on their way.
    const int early = min(n_it, t.stages);
    const bool dual = kX3 && t.dual == 1;
    const bool halves = !kX3 && t.dual == 2;        // single-pass modes: the K step's instructions shared by two threads
    constexpr int kSteps = MODE == 4 ? 2 : 4;       // instructions per K step (32 bytes of K each)
    if (warp == 0) {
        // the barriers lie behind one another: full[stages], empty[stages], ready[stages], accumulator, (8 bytes
        // of other use), receive -- lane i initialises the i-th of them
        const int n_bars = 3 * t.stages + 3;
        if (lane < n_bars && lane != 3 * t.stages + 1 && (push || lane != 3 * t.stages + 2)) {
            // arrivals per phase: the split's 128 threads on `ready`; both issuers on `empty` and on the accumulator's
            const bool both = (dual || halves) && ((lane >= t.stages && lane < 2 * t.stages) || lane == 3 * t.stages);
            mbar_init(bars + 8u * lane, (lane >= 2 * t.stages && lane < 3 * t.stages) ? 128u : (both ? 2u : 1u));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.arrive 2, 64;" ::: "memory");         // warp 1 may use the barriers
        // Weights never depend on the previous kernel: no grid dependency is waited for.  (Their bytes may be
        // counted before warp 1 has announced them: the barrier's phase cannot end before that arrival.)
        if (lane < early) {
            const int it = it_begin + lane;
            const uint32_t stage = smem_base + uint32_t(lane) * stage_bytes;
            const uint32_t bar = full0 + 8u * lane;
            tma_load_2d(stage + b_off, &tmap_b, bar, it * t.chunk, cout0);
            if (kX3) tma_load_2d(stage + b_lo_off, &tmap_b, bar, it * t.chunk, t.cout_pad + cout0);
        }
        // the bytes this CTA will be sent: its rows of the partial tiles of all CTAs of the cluster
        if (lane == 3 * t.stages + 2 && push) mbar_expect_tx(recv_bar, uint32_t(t.split_k * push_rows * t.bn) * 4u);
    } else if (warp == 1) {
        if (lane == 31) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            if (t.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c) : "memory");
        }
        int cc = 0, r = 0, sx = 0;
        if (lane < early) {
            const int it = it_begin + lane;
            const int tap = div_by(it, t.cchunks, t.magic_cc);
            cc = it - tap * t.cchunks;
            r = div_by(tap, g.kw, t.magic_kw);
            sx = tap - r * g.kw;
        }
        asm volatile("bar.sync 2, 64;" ::: "memory");           // the barriers exist
        if (lane < early) {
            const uint32_t stage = smem_base + uint32_t(lane) * stage_bytes;
            const uint32_t bar = full0 + 8u * lane;
            mbar_expect_tx(bar, uint32_t(t.a_bytes + passes * b_bytes));
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (t.im2col) tma_load_im2col(stage, &tmap_a, bar, cc * t.chunk, im_w, im_h, n0, uint32_t(sx), uint32_t(r));
            else if (t.flat) tma_load_4d(stage, &tmap_a, bar, cc * t.chunk, ow0, 0, 0);
            else tma_load_4d(stage, &tmap_a, bar, cc * t.chunk, ow0 * g.sw - g.pw + sx, oh0 * g.sh - g.ph + r, n0);
            if (lane == 0) STAMP(2);
        }
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), uint32_t(t.tmem_cols));
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Nothing may be pushed into a CTA before its barrier exists: every thread of the cluster arrives here and
    // waits only where it needs the others (the epilogue before its first push, everyone else before leaving).
    if (push) cluster_arrive_relaxed();
    // The next kernel of the stream may start its prologue (on SMs this grid leaves free, or as CTAs leave) once
    // every CTA of this grid has got here; it reads nothing of ours before its own griddepcontrol.wait.  (At kernel
    // entry instead: the same for one stream, 2 % slower for schedules with concurrent groups, whose waiting
    // dependents then hold SMs that a sibling group's kernel could use.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) STAMP(1);
    // Warps 0 and 1 work through a few lanes only.  Their other lanes leave now: a lane that spins on a
    // barrier pays about 50 cycles per wait while the rest of its warp is parked at the reconvergence point.
    // (Not in a cluster: there every thread takes part in the cluster barriers below.)
    if (!kCluster && ((warp == 0 && lane >= t.producers) || (warp == 1 && lane != 0) || (warp == 6 && (lane != 0 || !(dual || halves))))) return;
    if (!kCluster && !kX3 && warp >= 7) return;

    if (warp == 0) {
        // ---------------- TMA producers ----------------
        // (the tiles of the first `stages` K steps were requested during set-up)
        if (lane < t.producers && n_it > t.stages) {
            // One thread gets through wait -> arm -> issue about once per 600-800 cycles, whatever the
            // tiles' size, so `producers` lanes share the remaining K steps: lane l serves steps l + stages,
            // l + stages + P, ... and, P dividing the pipeline depth, owns stages l, l + P, ... for itself.
            const int P = t.producers;
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            int next = lane + t.stages;     // this lane's first K step whose tiles are not requested yet
            // running position of this lane (divisions cost more than the loads they would steer):
            // stage s and its phase, channel chunk cc and filter tap (r, sx) of K step it_begin + i
            int s = lane, phase = 0;
            int cc, r, sx;
            {
                const int it = it_begin + next;
                const int tap = it / t.cchunks;
                cc = it - tap * t.cchunks;
                r = tap / g.kw;
                sx = tap - r * g.kw;
            }
#pragma unroll 1
            for (int i = next; i < n_it; i += P) {
                const uint32_t stage = smem_base + uint32_t(s) * stage_bytes;
                const uint32_t bar = full0 + 8u * s;
                ok = mbar_wait(empty0 + 8u * s, uint32_t(phase), p.error_flag);
                if (!ok) break;
                const int kcol = (it_begin + i) * t.chunk;
                mbar_expect_tx(bar, uint32_t(t.a_bytes + passes * b_bytes));
                tma_load_2d(stage + b_off, &tmap_b, bar, kcol, cout0);
                if (kX3) tma_load_2d(stage + b_lo_off, &tmap_b, bar, kcol, t.cout_pad + cout0);
                if (t.im2col) tma_load_im2col(stage, &tmap_a, bar, cc * t.chunk, im_w, im_h, n0, uint32_t(sx), uint32_t(r));
                else if (t.flat) tma_load_4d(stage, &tmap_a, bar, cc * t.chunk, ow0, 0, 0);
                else tma_load_4d(stage, &tmap_a, bar, cc * t.chunk, ow0 * g.sw - g.pw + sx, oh0 * g.sh - g.ph + r, n0);
                next = i + P;
                s += P;
                if (s >= t.stages) { s -= t.stages; phase ^= 1; }
                cc += P;
                while (cc >= t.cchunks) {
                    cc -= t.cchunks;
                    if (++sx == g.kw) { sx = 0; ++r; }
                }
            }
            if (!ok) {
                atomicExch(p.error_flag, 1);
                // drain: the loads already issued still land in this CTA's shared memory; the latest
                // armed step of each stage this lane owns is waited for
                for (int j = next - P, k = 0; j >= 0 && k < t.stages; j -= P, k += P)
                    mbar_wait(full0 + 8u * (j % t.stages), uint32_t((j / t.stages) & 1), nullptr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            // instruction descriptor: fp32 accumulator, A/B format (2 = TF32, 1 = BF16), K-major, N, M
            const uint32_t fmt = kBf16 ? 1u : 2u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(t.bn >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
            // three-pass mode: the weight tile and its residual lie behind one another, so one instruction
            // of twice the width forms a_hi*w_hi (columns [0, bn)) and a_hi*w_lo (columns [bn, 2 bn))
            const uint32_t idesc_wide = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(t.bn >> 2) << 17) | (uint32_t(kTileM >> 4) << 24);
            MmaRing ring;
            ring.start(smem_base, a_lo_off, b_off, b_lo_off, stage_bytes, kRow);
#define IOS_MMA_LOOP(FORM, WAIT) mma_loop<FORM, kTimeline>(n_it, t.stages, WAIT, full0, empty0, ring, tmem_base, idesc, idesc_wide, p)
            // (two issuers: this one forms a_hi*[w_hi | w_lo] from the tiles as they land)
            const bool ok = dual ? mma_loop_planes<kTimeline>(n_it, t.stages, full0, empty0, ring.da0, ring.db0, ring.dstep, tmem_base,
                                                              idesc_wide, p, true)
                            : halves ? mma_loop_planes<kTimeline, kBf16>(n_it, t.stages, full0, empty0, ring.da0, ring.db0, ring.dstep,
                                                                         tmem_base, idesc, p, true, 0, kSteps / 2)
                            : kX3 ? (t.wide ? IOS_MMA_LOOP(3, ready0) : IOS_MMA_LOOP(1, ready0))
                                  : (kBf16 ? IOS_MMA_LOOP(MODE, full0) : IOS_MMA_LOOP(0, full0));
#undef IOS_MMA_LOOP
            if (ok) umma_commit(accum_bar);
            else atomicExch(p.error_flag, 2);
            STAMP(4);
        }
    } else if (warp == 6) {
        if (lane == 0 && dual) {
            // ---------------- second MMA issuer (three-pass mode): a_lo*w_hi, once the residual of a tile is written ----------------
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(t.bn >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
            const bool ok = mma_loop_planes<kTimeline>(n_it, t.stages, ready0, empty0, smem_desc_kmajor(smem_base + a_lo_off, kRow),
                                                       smem_desc_kmajor(smem_base + b_off, kRow), uint64_t(stage_bytes >> 4),
                                                       tmem_base + 2u * uint32_t(t.bn), idesc, p, false);
            if (ok) umma_commit(accum_bar);
            else atomicExch(p.error_flag, 2);
        } else if (lane == 0 && halves) {
            // ---------------- second MMA issuer (single-pass modes): the second half of every K step ----------------
            const uint32_t fmt = kBf16 ? 1u : 2u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(t.bn >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
            const bool ok = mma_loop_planes<kTimeline, kBf16>(n_it, t.stages, full0, empty0, smem_desc_kmajor(smem_base, kRow),
                                                              smem_desc_kmajor(smem_base + b_off, kRow), uint64_t(stage_bytes >> 4),
                                                              tmem_base + uint32_t(t.bn), idesc, p, false, kSteps / 2, kSteps);
            if (ok) umma_commit(accum_bar);
            else atomicExch(p.error_flag, 2);
        }
    } else if (warp >= 7) {
        // ---------------- warps 7..10 (three-pass mode): the residual of every landed activation tile ----------------
        if (kX3) {
            const int tid = threadIdx.x - 224;          // 0..127
            // Nothing to do until the first tile lands: the CTAs of the grid share out the next convolution's
            // weights, one 128-byte line per request, and ask them into L2 (they are read once per forward and the
            // networks' weights do not fit the L2 together, so they would otherwise be met in DRAM).
            if (p.next_weights) {
                const unsigned ctas = gridDim.x * gridDim.y * gridDim.z;
                const unsigned cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
                const char *w = static_cast<const char *>(p.next_weights);
#pragma unroll 1
                for (unsigned off = (cta * 128u + unsigned(tid)) * 128u; off < p.next_weight_bytes; off += ctas * 128u * 128u)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(w + off) : "memory");
            }
            // The tensor core reads the 19 leading bits of an fp32 operand (sign, exponent, 10 mantissa
            // bits), so the landed activation tile serves as the TF32 value as it is.  What the hardware
            // drops -- x minus x with the low 13 bits cleared, exact in fp32 -- is written to the residual
            // tile here.  (Weights are split on the host into two planes; deriving their residual here too
            // was measured 7-15 % slower: this step sits on the latency chain TMA -> split -> MMA.)
            const int n_vec = t.a_bytes >> 4;
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
#pragma unroll 1
            for (int i = 0; i < n_it && ok; ++i) {
                ok = mbar_wait(full0 + 8u * s, phase, p.error_flag);
                if (!ok) break;
                uint8_t *stage = generic_base + size_t(s) * stage_bytes;
                const float4 *hi = reinterpret_cast<const float4 *>(stage);
                float4 *lo = reinterpret_cast<float4 *>(stage + a_lo_off);
#pragma unroll 2
                for (int v = tid; v < n_vec; v += 128) {
                    const float4 x = hi[v];
                    float4 l;
                    l.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
                    l.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
                    l.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
                    l.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
                    lo[v] = l;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready0 + 8u * s) : "memory");
                if (++s == t.stages) { s = 0; phase ^= 1u; }
            }
            ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
            if (!ok && lane == 0) atomicExch(p.error_flag, 5);
            if (kCluster && push) {
                // These warps are free now: each thread finishes one of the second 128 items of this CTA's rows.
                cluster_wait();                                 // (pairs with the arrival at set-up)
                int src, count;
                long at;
                float4 bias;
                prepare_item(128 + tid, src, at, count, bias);
                bool good = ok;
                if (good && fast_split && push_rows > 0)
                    good = __all_sync(0xffffffffu, mbar_wait_cluster(recv_bar, 0, p.error_flag) ? 1 : 0) != 0;
                if (good && fast_split && push_rows > 0) {
                    if (t.split_k == 8) finish_item(std::integral_constant<int, 8>(), src, at, count, bias);
                    else if (t.split_k == 4) finish_item(std::integral_constant<int, 4>(), src, at, count, bias);
                    else finish_item(std::integral_constant<int, 2>(), src, at, count, bias);
                }
                if (!good) {
                    // (as in the epilogue: a warp that gave up waits for the rest of the cluster to leave or give up)
                    if (lane == 0) atomicExch(p.error_flag, 4);
                    cluster_arrive();
                    cluster_wait();
                }
                return;
            }
        }
    } else {
        // ---------------- warps 2..5: the epilogue ----------------
        const int tid = threadIdx.x - 64;           // 0..127
        const int quad = warp & 3;                  // TMEM lane group this warp may read
        const int row = quad * 32 + lane;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // (the loads go out now; the values are put into shared memory further down, so that nothing waits for them here)
        float bias_early[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int j = tid + u * 128;
            bias_early[u] = (p.bias && j < t.bn && cout0 + j < g.Cout) ? __ldg(p.bias + cout0 + j) : 0.0f;
        }
        // Push form of the cluster reduction: everything that does not depend on the accumulator is worked out
        // now, while the first tiles are on their way.  After the accumulator there are four warps, one per
        // scheduler, each instruction waiting for the one before it: what is left on that path is the accumulator
        // load, the pushes, and for the rows this CTA finishes the loads, adds and stores.
        constexpr int kFast = kX3 ? 1 : 2;          // items per thread with everything precomputed (256 in all: 64 columns x 16 rows)
        uint32_t push_dst = 0, push_bar = 0, push_stride = 0;
        bool push_mine = false;
        int fast_src[kFast];                        // float4 index of partial tile 0 of the item in the receive area
        long fast_at[kFast];                        // element offset of the item's four outputs, or -1
        int fast_count[kFast];                      // valid outputs of the four
        float4 fast_bias[kFast];
        if (kCluster && push) {
            if (threadIdx.x == 64) STAMP(8);
            cluster_wait();                                     // every CTA of the cluster has its barrier set up
            if (threadIdx.x == 64) STAMP(13);
            push_mine = row < push_vrows;
            const int owner = push_mine ? div_pow2_likely(row, push_rpr) : 0;
            const int lrow = row - owner * push_rpr;
            push_dst = cluster_map(smem_base + uint32_t(t.recv_off) + uint32_t(split * (t.bn >> 2) * push_rpr + lrow) * 16u, uint32_t(owner));
            push_bar = cluster_map(recv_bar, uint32_t(owner));
            push_stride = uint32_t(push_rpr) * 16u;
            if (threadIdx.x == 64) STAMP(14);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (tid + u * 128 < t.bn) bias_s[tid + u * 128] = bias_early[u];
        // (the second half of the preparation: called once the operand work of the K loop is behind these warps)
        auto prepare_rows = [&]() {
#pragma unroll
            for (int k = 0; k < kFast; ++k) prepare_item(tid + k * 128, fast_src[k], fast_at[k], fast_count[k], fast_bias[k]);
            if (threadIdx.x == 64) STAMP(15);
        };
        bool ok = true;
        if (kCluster && push) prepare_rows();
        if (ok) ok = mbar_wait(accum_bar, 0, p.error_flag);
        ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
        if (!ok && lane == 0) atomicExch(p.error_flag, 3);
        if (threadIdx.x == 64) STAMP(5);
        tc_fence_after();
        if (!(kCluster && push)) asm volatile("bar.sync 1, 128;" ::: "memory");          // bias_s is complete
        if (threadIdx.x == 64) STAMP(9);
        const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16);
        const uint32_t pair = (t.wide || halves) ? uint32_t(t.bn) : 0u;
        const uint32_t third = dual ? 2u * uint32_t(t.bn) : 0u;
        const int tile_id = m_tile * gridDim.y + n_tile;
        bool finisher = true;
        if (kCluster && push) {
            // cluster reduction, push form: row r of this CTA's partial tile goes, 16 bytes at a time, into the
            // shared memory of the CTA that finishes row r, as recv[split][column quad][row of that CTA]; the
            // bytes are counted on that CTA's barrier as they land, so no cluster barrier and no trip through L2
            // follows.  (The accumulator load is warp-wide; rows past the tile's valid prefix are not sent.)
            finisher = false;
            if (ok) {
#pragma unroll 1
                for (int c = 0; c < t.bn; c += 32) {
                    float v[32];
                    acc_ld32_pair(taddr + c, pair, v, third);
                    if (push_mine) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            cluster_push16(push_dst + uint32_t((c + j) >> 2) * push_stride, push_bar, v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                }
            }
            if (threadIdx.x == 64) STAMP(6);
            asm volatile("bar.sync 1, 128;" ::: "memory");      // bias_s is complete (every epilogue thread gets here)
            // the rows this CTA finishes have landed once its barrier has counted their bytes
            bool good = ok;
            if (good && push_rows > 0) good = __all_sync(0xffffffffu, mbar_wait_cluster(recv_bar, 0, p.error_flag) ? 1 : 0) != 0;
            if (threadIdx.x == 64) STAMP(10);
            if (good) {
                // partial tiles are added in split order, so the result does not depend on timing
                const float4 *recv = reinterpret_cast<const float4 *>(generic_base + t.recv_off);
                const int plane = (t.bn >> 2) * push_rpr;           // float4 from one partial tile to the next
#pragma unroll
                for (int k = 0; k < kFast; ++k) {
                    if (t.split_k == 8) finish_item(std::integral_constant<int, 8>(), fast_src[k], fast_at[k], fast_count[k], fast_bias[k]);
                    else if (t.split_k == 4) finish_item(std::integral_constant<int, 4>(), fast_src[k], fast_at[k], fast_count[k], fast_bias[k]);
                    else if (t.split_k == 2) finish_item(std::integral_constant<int, 2>(), fast_src[k], fast_at[k], fast_count[k], fast_bias[k]);
                    if (k == 0 && threadIdx.x == 64) STAMP(12);
                }
                // items beyond the precomputed ones (wide tiles), and splits without a form of their own
                const int quads = t.bn >> 2;
                const int n_items = push_rows * quads;
                const int r0 = int(cluster_cta_rank()) * push_rpr;
                const int valid = min(t.bn, g.Cout - cout0);
#pragma unroll 1
                for (int item = tid + (fast_split ? 256 : 0); item < n_items; item += 128) {
                    const int q4 = item / push_rows, lr = item - q4 * push_rows, c = q4 << 2;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                    for (int sp = 0; sp < t.split_k; ++sp) {
                        const float4 x = recv[q4 * push_rpr + lr + sp * plane];
                        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
                    }
                    const long pix = long(ow0) + r0 + lr;
                    const long pix_off = t.flat ? ((r0 + lr < t.box_w && pix < long(g.N) * g.OH * g.OW) ? pix * p.out.pitch : -1)
                                                : boxed_pixel_offset(r0 + lr, t.box_w, t.box_h, t.box_n, ow0, oh0, n0, g.N, g.OH, g.OW, p.out.pitch);
                    if (pix_off < 0 || c >= valid) continue;
                    float o[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float z = act_apply(o[j] + bias_s[c + j], g.act);
                        o[j] = t.round_tf32 ? round_tf32(z) : z;
                    }
                    store4_direct(p.out.ptr, kBf16, pix_off + cout0 + c, make_float4(o[0], o[1], o[2], o[3]), valid - c);
                }
            }
            if (threadIdx.x == 64) STAMP(7);
            // the accumulator has been read by all four warps: TMEM goes back
            tc_fence_before();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == 2) {
                tc_fence_after();
                tmem_dealloc(tmem_base, uint32_t(t.tmem_cols));
            }
            if (!good) {
                // A warp that gave up stays until every other thread of the cluster has left or given up too:
                // a CTA must not vanish while others may still push into its shared memory.
                if (lane == 0) atomicExch(p.error_flag, 4);
                cluster_arrive();
                cluster_wait();
            }
            return;
        } else if (kCluster) {
            // cluster reduction through L2 (when the push form's receive area does not fit): this CTA's partial tile
            // goes to the workspace as ws[tile][split][column quad][row]
            // (float4 units; a warp writes 512 contiguous bytes).  It stays in L2: the CTAs of the cluster read it
            // back right after the cluster barrier below.  (Loads from another CTA's shared memory were measured
            // at a few bytes per cycle here, several times slower than this round trip through L2.)
            finisher = false;
            if (ok) {
                float4 *ws = reinterpret_cast<float4 *>(p.workspace) + (size_t(tile_id) * t.split_k + split) * size_t(t.bn >> 2) * kTileM + row;
#pragma unroll 1
                for (int c = 0; c < t.bn; c += 32) {
                    float v[32];
                    acc_ld32(taddr + c, pair, v, third);
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        ws[size_t((c + j) >> 2) * kTileM] = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
            }
            if (threadIdx.x == 64) STAMP(6);
        } else if (!kCluster && ok && t.split_k > 1) {
            // publish this CTA's partial tile: ws[tile][split][col][row], rows contiguous
            float *ws = p.workspace + (size_t(tile_id) * t.split_k + split) * size_t(t.bn) * kTileM;
#pragma unroll 1
            for (int c = 0; c < t.bn; c += 16) {
                float v[16];
                acc_ld16(taddr + c, pair, v, third);
#pragma unroll
                for (int j = 0; j < 16; ++j) ws[size_t(c + j) * kTileM + row] = v[j];
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) {
                const unsigned int prev = atomicAdd(p.counters + tile_id, 1u);
                *ticket_slot = int(prev);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            finisher = (*ticket_slot == t.split_k - 1);
            if (finisher) __threadfence();
            if (threadIdx.x == 64) STAMP(6);
        }
        if (ok && finisher) {
            // which output pixel does this row hold? (only the direct-store path needs it)
            long pix_off = -1;
            if (t.flat) {
                const long pix = long(ow0) + row;
                if (row < t.box_w && pix < long(g.N) * g.OH * g.OW) pix_off = pix * p.out.pitch;
            } else {
                pix_off = boxed_pixel_offset(row, t.box_w, t.box_h, t.box_n, ow0, oh0, n0, g.N, g.OH, g.OW, p.out.pitch);
            }
            const int valid = min(t.bn, g.Cout - cout0);
            const float *ws_tile = p.workspace + size_t(tile_id) * t.split_k * size_t(t.bn) * kTileM;
            // (loops that run a handful of times are kept rolled: the code of a CTA runs once, so its
            // cost is dominated by instruction fetch, not by loop overhead)
            if (t.split_k == 1 && t.tma_store) {
                // common case: 32 channels = one 128-byte staging row per TMEM round trip
#pragma unroll 1
                for (int c = 0; c < t.bn; c += 32) {
                    float v[32];
                    acc_ld32(taddr + c, pair, v, third);
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float o[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float z = act_apply(v[j + u] + bias_s[c + j + u], g.act);
                            o[u] = t.round_tf32 ? round_tf32(z) : z;
                        }
                        stage4(generic_base, row, c + j, make_float4(o[0], o[1], o[2], o[3]), kBf16);
                    }
                }
            } else
#pragma unroll 1
            for (int c = 0; c < t.bn; c += 16) {
                float v[16];
                if (t.split_k == 1) {
                    acc_ld16(taddr + c, pair, v, third);
                    if (c == 0 && threadIdx.x == 64) STAMP(13);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    // four partial tiles per round trip, added in split order
#pragma unroll 1
                    for (int s0 = 0; s0 < t.split_k; s0 += 4) {
                        float part[4][16];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float *src = ws_tile + size_t(min(s0 + u, t.split_k - 1)) * t.bn * kTileM + size_t(c) * kTileM + row;
#pragma unroll
                            for (int j = 0; j < 16; ++j) part[u][j] = __ldcg(src + size_t(j) * kTileM);
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (s0 + u < t.split_k) {
#pragma unroll
                                for (int j = 0; j < 16; ++j) v[j] += part[u][j];
                            }
                    }
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float o = act_apply(v[j] + bias_s[c + j], g.act);
                    v[j] = t.round_tf32 ? round_tf32(o) : o;
                }
                if (c == 0 && threadIdx.x == 64) STAMP(14);
                if (t.tma_store) {
                    // stage the tile as [slab][row][128 B], swizzled like a TMA box, for the bulk store
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        stage4(generic_base, row, c + j, make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]), kBf16);
                    if (c == 0 && threadIdx.x == 64) STAMP(15);
                    continue;
                }
                if (pix_off < 0 || c >= valid) continue;
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    if (c + j < valid)
                        store4_direct(p.out.ptr, kBf16, pix_off + cout0 + c + j, make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]),
                                      valid - (c + j));
            }
            if (threadIdx.x == 64) STAMP(10);
            if (t.tma_store) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    STAMP(11);
                    // one bulk tensor store per 128-byte slab; pixels and channels outside the tensor are clipped
                    for (int c = 0; c < valid; c += t.slab) {
                        const uint32_t src = smem_base + uint32_t(c / t.slab) * kATileBytes;
                        if (t.flat) tma_store_4d(&tmap_c, src, cout0 + c, ow0, 0, 0);
                        else tma_store_4d(&tmap_c, src, cout0 + c, ow0, oh0, n0);
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    STAMP(12);
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                }
            }
            if (t.split_k > 1 && threadIdx.x == 64) p.counters[tile_id] = 0;   // ready for the next launch
        }
        if (threadIdx.x == 64) STAMP(7);
        tc_fence_before();
        if (kCluster) {
            // the accumulator has been read: give TMEM back now, behind the cluster barrier's wait
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == 2) {
                tc_fence_after();
                tmem_dealloc(tmem_base, uint32_t(t.tmem_cols));
            }
        }
    }
    if (kCluster) {
        if (push) {
            // the warps of the single-thread roles pair their arrival at the set-up barrier with a wait and leave
            if (warp < 2 || warp >= 6) {
                __syncwarp();
                cluster_wait();
                return;
            }
            return;                 // (the epilogue warps have finished the tile inside their branch)
        } else {
            // Every thread of every CTA of the cluster passes this barrier, whatever happened before; its
            // release / acquire pair makes the partial tiles written above visible to the cluster.
            cluster_sync_all();
        }
        if (threadIdx.x == 64) STAMP(10);
        if (warp >= 2 && warp < 6) {
            // CTA r of the cluster finishes rows [r*128/S, (r+1)*128/S) of the tile: it adds the S partial
            // tiles in split order (so the result does not depend on timing), applies bias and activation
            // and writes its rows.  A thread puts all its loads in flight before it adds anything.
            const int tid = threadIdx.x - 64;
            const int rank = int(cluster_cta_rank());
            const int r0 = rank * kTileM / t.split_k;
            const int rows = (rank + 1) * kTileM / t.split_k - r0;
            const int quads = t.bn >> 2;
            const int valid = min(t.bn, g.Cout - cout0);
            const int n_items = rows * quads;
            const int tile_id = m_tile * gridDim.y + n_tile;
            // partial tile `sp`, column quad `q4`, row `lr` of this CTA's rows is at src0[(sp * quads + q4) * pitch + lr]
            const float4 *src0 = reinterpret_cast<const float4 *>(p.workspace) + size_t(tile_id) * t.split_k * size_t(quads) * kTileM + r0;
            const int pitch = kTileM;
            auto fetch = [&](const float4 *src) -> float4 { return __ldcg(src); };
            // offset of the output pixel held by tile row `row`, or -1
            auto pixel_offset = [&](int row) -> long {
                if (t.flat) {
                    const long pix = long(ow0) + row;
                    return (row < t.box_w && pix < long(g.N) * g.OH * g.OW) ? pix * p.out.pitch : -1;
                }
                return boxed_pixel_offset(row, t.box_w, t.box_h, t.box_n, ow0, oh0, n0, g.N, g.OH, g.OW, p.out.pitch);
            };
            auto finish = [&](int row, int c, float4 acc) {
                const long pix_off = pixel_offset(row);
                if (pix_off < 0 || c >= valid) return;
                float o[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float z = act_apply(o[j] + bias_s[c + j], g.act);
                    o[j] = t.round_tf32 ? round_tf32(z) : z;
                }
                store4_direct(p.out.ptr, kBf16, pix_off + cout0 + c, make_float4(o[0], o[1], o[2], o[3]), valid - c);
            };
            auto reduce = [&](auto split_tag) {
                constexpr int S = decltype(split_tag)::value;
                constexpr int kItems = 16 / S;
#pragma unroll 1
                for (int first = tid; first < n_items; first += 128 * kItems) {
                    float4 part[kItems][S];
#pragma unroll
                    for (int k = 0; k < kItems; ++k) {
                        const int item = min(first + k * 128, n_items - 1);
                        const int q4 = item / rows;
                        const float4 *src = src0 + size_t(q4) * pitch + (item - q4 * rows);
#pragma unroll
                        for (int sp = 0; sp < S; ++sp) part[k][sp] = fetch(src + size_t(sp) * quads * pitch);
                    }
#pragma unroll
                    for (int k = 0; k < kItems; ++k) {
                        const int item = first + k * 128;
                        if (item >= n_items) break;
                        const int q4 = item / rows;
                        float4 acc = part[k][0];
#pragma unroll
                        for (int sp = 1; sp < S; ++sp) {
                            acc.x += part[k][sp].x; acc.y += part[k][sp].y; acc.z += part[k][sp].z; acc.w += part[k][sp].w;
                        }
                        finish(r0 + (item - q4 * rows), q4 << 2, acc);
                    }
                }
            };
            if (t.split_k == 8) reduce(std::integral_constant<int, 8>());
            else if (t.split_k == 4) reduce(std::integral_constant<int, 4>());
            else if (t.split_k == 2) reduce(std::integral_constant<int, 2>());
            else
#pragma unroll 1
            for (int item = tid; item < n_items; item += 128) {
                const int q4 = item / rows;
                const float4 *src = src0 + size_t(q4) * pitch + (item - q4 * rows);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (int sp = 0; sp < t.split_k; ++sp) {
                    const float4 x = fetch(src + size_t(sp) * quads * pitch);
                    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
                }
                finish(r0 + (item - q4 * rows), q4 << 2, acc);
            }
            if (threadIdx.x == 64) STAMP(7);
        }
    }
    if (warp < 2 || warp >= 6 || kCluster) return;   // the producer lanes, the MMA issuers and the residual warps have nothing left to do
    // warps 0 and 1 are gone by now or on their way out; the warps that read the accumulator free it
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, uint32_t(t.tmem_cols));
        if (lane == 0) STAMP(8);
    }
}

// ---- the persistent kernel -------------------------------------------------------------------
// A grid of several waves spends most of its time outside the K loop when K is short (a 1x1
// convolution over 192 bfloat16 channels is three K steps): set-up and epilogue of a tile cost more
// than its tensor work.  Here a CTA stays on its SM and walks tiles blockIdx.x, blockIdx.x + gridDim.x,
// ...; barriers, tensor maps and TMEM are set up once, the accumulator is double-buffered in TMEM, and
// the epilogue warps finish tile i while the producer and the MMA issuer are already in tile i + 1.
//   warp 0     TMA producer lanes (ring of pipeline stages, running across tiles)
//   warp 1     MMA issuer: waits for a free accumulator, runs the tile's K loop, commits to acc_full
//   warps 2-9  epilogue: two warps per TMEM lane quarter, each half of the tile's columns
//              (three-pass mode: warps 2-5 are the epilogue, warps 6-9 compute the activation residual)
constexpr int kPersistThreads = 320;

struct PersistGeom {
    int n_tiles;        // output-channel tiles
    int total_tiles;    // pixel tiles * output-channel tiles, output-channel tile fastest
    int staging_off;    // byte offset of the store staging area (behind the pipeline stages)
    int acc_stride;     // TMEM columns from one accumulator to the other
};

struct TileCoord {
    int cout0, ow0, oh0, n0, im_w, im_h;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, const TileGeom &t, const PersistGeom &pg, const ConvGeom &g) {
    TileCoord c;
    const int m_tile = tile / pg.n_tiles;
    c.cout0 = (tile - m_tile * pg.n_tiles) * t.bn;
    c.ow0 = c.oh0 = c.n0 = c.im_w = c.im_h = 0;
    if (t.flat) {
        c.ow0 = m_tile * t.box_w;
        if (t.im2col) {
            const int per_image = g.OH * g.OW;
            c.n0 = c.ow0 / per_image;
            const int rem = c.ow0 - c.n0 * per_image;
            c.oh0 = rem / g.OW;
            c.im_w = (rem - c.oh0 * g.OW) * g.sw - g.pw;
            c.im_h = c.oh0 * g.sh - g.ph;
        }
    } else {
        const int tw = m_tile % t.tiles_w;
        const int rest = m_tile / t.tiles_w;
        c.ow0 = tw * t.box_w;
        c.oh0 = (rest % t.tiles_h) * t.box_h;
        c.n0 = (rest / t.tiles_h) * t.box_n;
    }
    return c;
}

template <int MODE>      // operand mode, as for conv_tc_kernel
__global__ void __launch_bounds__(kPersistThreads, 1)
conv_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_c, const ConvTcParams p, const TileGeom t,
                          const PersistGeom pg) {
    constexpr bool kX3 = MODE == 1, kBf16 = MODE == 2 || MODE == 4;
    constexpr int kRow = MODE == 4 ? 64 : 128;          // bytes of K per operand row (MODE 4: bfloat16, 64-byte rows)
    extern __shared__ uint8_t smem_raw[];
    __shared__ float bias_s[2][256];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    constexpr int a_tile_bytes = kTileM * kRow;
    const int b_bytes = t.bn * kRow;
    const int passes = kX3 ? 2 : 1;
    const int stage_bytes = passes * (a_tile_bytes + b_bytes);
    const uint32_t a_lo_off = uint32_t(a_tile_bytes);
    const uint32_t b_off = uint32_t(passes) * a_tile_bytes;
    const uint32_t b_lo_off = b_off + uint32_t(b_bytes);
    const int slabs = (t.bn + t.slab - 1) / t.slab;
    const uint32_t bars = smem_base + uint32_t(pg.staging_off) + (t.tma_store ? uint32_t(slabs) * kATileBytes : 0u);
    const uint32_t full0 = bars, empty0 = bars + 8u * t.stages, ready0 = bars + 16u * t.stages;
    const uint32_t acc_full0 = bars + 24u * t.stages, acc_empty0 = acc_full0 + 16u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(generic_base + (bars - smem_base) + 24 * t.stages + 32);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const ConvGeom &g = p.g;
    const int epi_warps = kX3 ? 4 : 8;
    const int my_tiles = (pg.total_tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);

    if (warp == 0) {
        if (lane < t.stages) {
            mbar_init(full0 + 8u * lane, 1);
            mbar_init(empty0 + 8u * lane, 1);
            mbar_init(ready0 + 8u * lane, 128);
        }
        if (lane >= 28) {
            const int a = lane & 1;
            if (lane < 30) mbar_init(acc_full0 + 8u * a, 1);
            else mbar_init(acc_empty0 + 8u * a, uint32_t(epi_warps));
        }
        if (lane == 27) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            if (t.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), uint32_t(t.tmem_cols));
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if ((warp == 0 && lane >= t.producers) || (warp == 1 && lane != 0)) return;

    if (warp == 0) {
        // ---------------- TMA producer lanes ----------------
        // Lane l serves K steps l, l + P, ... of the CTA's whole sequence of (tile, K step) pairs and owns
        // stages l, l + P, ... of the ring.  A fresh barrier lets a wait for parity 1 pass at once.
        const int P = t.producers;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        int tile = blockIdx.x, it = lane;
        while (it >= t.k_iters && tile < pg.total_tiles) { it -= t.k_iters; tile += gridDim.x; }
        int s = lane, phase = 1, armed = 0;
        bool ok = true;
#pragma unroll 1
        while (ok && tile < pg.total_tiles) {
            const TileCoord tc = tile_coord(tile, t, pg, g);
            int cc, r, sx;
            {
                const int tap = it / t.cchunks;
                cc = it - tap * t.cchunks;
                r = tap / g.kw;
                sx = tap - r * g.kw;
            }
#pragma unroll 1
            while (it < t.k_iters) {
                ok = mbar_wait(empty0 + 8u * s, uint32_t(phase), p.error_flag);
                if (!ok) break;
                const uint32_t stage = smem_base + uint32_t(s) * stage_bytes;
                const uint32_t bar = full0 + 8u * s;
                mbar_expect_tx(bar, uint32_t(t.a_bytes + passes * b_bytes));
                tma_load_2d(stage + b_off, &tmap_b, bar, it * t.chunk, tc.cout0);
                if (kX3) tma_load_2d(stage + b_lo_off, &tmap_b, bar, it * t.chunk, t.cout_pad + tc.cout0);
                if (t.im2col) tma_load_im2col(stage, &tmap_a, bar, cc * t.chunk, tc.im_w, tc.im_h, tc.n0, uint32_t(sx), uint32_t(r));
                else if (t.flat) tma_load_4d(stage, &tmap_a, bar, cc * t.chunk, tc.ow0, 0, 0);
                else tma_load_4d(stage, &tmap_a, bar, cc * t.chunk, tc.ow0 * g.sw - g.pw + sx, tc.oh0 * g.sh - g.ph + r, tc.n0);
                ++armed;
                s += P;
                if (s >= t.stages) { s -= t.stages; phase ^= 1; }
                it += P;
                cc += P;
                while (cc >= t.cchunks) {
                    cc -= t.cchunks;
                    if (++sx == g.kw) { sx = 0; ++r; }
                }
            }
            it -= t.k_iters;
            tile += gridDim.x;
            while (it >= t.k_iters && tile < pg.total_tiles) { it -= t.k_iters; tile += gridDim.x; }
        }
        if (!ok) {
            atomicExch(p.error_flag, 1);
            // drain: the loads this lane has issued still land in shared memory; wait for the latest
            // one of each stage it owns before the CTA may go
            const int owned = t.stages / P;
            for (int j = armed - 1, k = 0; j >= 0 && k < owned; --j, ++k)
                mbar_wait(full0 + 8u * (lane + (j % owned) * P), uint32_t((j / owned) & 1), nullptr);
        }
        return;
    }
    if (warp == 1) {
        // ---------------- MMA issuer ----------------
        const uint32_t fmt = kBf16 ? 1u : 2u;
        const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(t.bn >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
        const uint32_t idesc_wide = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(t.bn >> 2) << 17) | (uint32_t(kTileM >> 4) << 24);
        MmaRing ring;
        ring.start(smem_base, a_lo_off, b_off, b_lo_off, stage_bytes, kRow);
        bool ok = true;
#pragma unroll 1
        for (int ti = 0; ti < my_tiles && ok; ++ti) {
            const uint32_t a = uint32_t(ti) & 1u;
            // the epilogue must have emptied this accumulator (tiles 0 and 1 find it fresh: parity 1 passes)
            ok = mbar_wait(acc_empty0 + 8u * a, ((uint32_t(ti) >> 1) & 1u) ^ 1u, p.error_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + a * uint32_t(pg.acc_stride);
#define IOS_MMA_LOOP(FORM, WAIT) mma_loop<FORM, false>(t.k_iters, t.stages, WAIT, full0, empty0, ring, tmem_d, idesc, idesc_wide, p)
            ok = kX3 ? (t.wide ? IOS_MMA_LOOP(3, ready0) : IOS_MMA_LOOP(1, ready0))
                      : (kBf16 ? IOS_MMA_LOOP(MODE, full0) : IOS_MMA_LOOP(0, full0));
#undef IOS_MMA_LOOP
            if (ok) umma_commit(acc_full0 + 8u * a);
        }
        if (!ok) atomicExch(p.error_flag, 2);
        return;
    }
    if (kX3 && warp >= 6) {
        // ---------------- warps 6..9 (three-pass mode): residual of every landed activation tile ----------------
        const int tid = threadIdx.x - 192;
        const int n_vec = t.a_bytes >> 4;
        const long steps = long(my_tiles) * t.k_iters;
        int s = 0;
        uint32_t phase = 0;
#pragma unroll 1
        for (long i = 0; i < steps; ++i) {
            if (!mbar_wait(full0 + 8u * s, phase, p.error_flag)) {
                atomicExch(p.error_flag, 4);
                break;
            }
            uint8_t *stage = generic_base + size_t(s) * stage_bytes;
            const float4 *hi = reinterpret_cast<const float4 *>(stage);
            float4 *lo = reinterpret_cast<float4 *>(stage + a_lo_off);
#pragma unroll 2
            for (int v = tid; v < n_vec; v += 128) {
                const float4 x = hi[v];
                float4 l;
                l.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
                l.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
                l.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
                l.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
                lo[v] = l;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready0 + 8u * s) : "memory");
            if (++s == t.stages) { s = 0; phase ^= 1u; }
        }
        return;
    }
    // ---------------- epilogue warps ----------------
    const int e = warp - 2;                           // 0 .. epi_warps - 1
    const int etid = threadIdx.x - 64;                // 0 .. epi_warps * 32 - 1
    const int epi_threads = epi_warps * 32;
    const int quad = warp & 3;                        // TMEM lane quarter this warp may read
    const int row = quad * 32 + lane;
    const int cols_per_warp = epi_warps == 8 ? t.bn / 2 : t.bn;
    const int c_begin = (e >> 2) * cols_per_warp, c_end = c_begin + cols_per_warp;
    const uint32_t pair = t.wide ? uint32_t(t.bn) : 0u;
    uint8_t *staging = generic_base + pg.staging_off;
    const long total_pixels = long(g.N) * g.OH * g.OW;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the output window may still be read by the previous kernel
#pragma unroll 1
    for (int ti = 0; ti < my_tiles; ++ti) {
        const int tile = int(blockIdx.x) + ti * int(gridDim.x);
        const TileCoord tc = tile_coord(tile, t, pg, g);
        const uint32_t a = uint32_t(ti) & 1u;
        float *bias = bias_s[a];
        for (int j = etid; j < t.bn; j += epi_threads) bias[j] = (p.bias && tc.cout0 + j < g.Cout) ? p.bias[tc.cout0 + j] : 0.0f;
        bool ok = mbar_wait(acc_full0 + 8u * a, (uint32_t(ti) >> 1) & 1u, p.error_flag);
        ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
        if (!ok && lane == 0) atomicExch(p.error_flag, 3);
        tc_fence_after();
        // the bulk store of the previous tile must have read the staging area before it is written again
        if (t.tma_store && etid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");      // bias complete, staging free
        const int valid = min(t.bn, g.Cout - tc.cout0);
        if (ok) {
            long pix_off = -1;
            if (t.flat) {
                const long pix = long(tc.ow0) + row;
                if (row < t.box_w && pix < total_pixels) pix_off = pix * p.out.pitch;
            } else {
                pix_off = boxed_pixel_offset(row, t.box_w, t.box_h, t.box_n, tc.ow0, tc.oh0, tc.n0, g.N, g.OH, g.OW, p.out.pitch);
            }
            const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + a * uint32_t(pg.acc_stride);
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 16) {
                float v[16];
                acc_ld16(taddr + c, pair, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float z = act_apply(v[j] + bias[c + j], g.act);
                    v[j] = t.round_tf32 ? round_tf32(z) : z;
                }
                if (t.tma_store) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        stage4(staging, row, c + j, make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]), kBf16);
                } else if (pix_off >= 0 && c < valid) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        if (c + j < valid)
                            store4_direct(p.out.ptr, kBf16, pix_off + tc.cout0 + c + j, make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]),
                                          valid - (c + j));
                }
            }
        }
        // hand the accumulator back to the MMA issuer: one arrival per epilogue warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8u * a) : "memory");
        if (t.tma_store) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");  // the tile is staged
            if (ok && etid == 0) {
                for (int c = 0; c < valid; c += t.slab) {
                    const uint32_t src = smem_base + uint32_t(pg.staging_off) + uint32_t(c / t.slab) * kATileBytes;
                    if (t.flat) tma_store_4d(&tmap_c, src, tc.cout0 + c, tc.ow0, 0, 0);
                    else tma_store_4d(&tmap_c, src, tc.cout0 + c, tc.ow0, tc.oh0, tc.n0);
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
    }
    if (t.tma_store && etid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, uint32_t(t.tmem_cols));
    }
}


// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
    return fn;
}

typedef CUresult (*EncodeIm2colFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t, const cuuint32_t *,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeIm2colFn encode_im2col_fn() {
    static EncodeIm2colFn fn = nullptr;
    if (fn) return fn;
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeIm2colFn>(sym);
    return fn;
}

int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Corners of the im2col bounding box along one axis: the filter window's first corner sits at -pad,
// its last at (out - 1) * stride - pad, given relative to the last input element.
void im2col_corners(int in, int out, int stride, int pad, int *lower, int *upper) {
    *lower = -pad;
    *upper = (out - 1) * stride - pad - (in - 1);
}

float tf32_round_host(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return v;   // inf / nan
    u += 0x00000FFFu + ((u >> 13) & 1u);              // round to nearest even on the 13 dropped bits
    u &= 0xFFFFE000u;
    float r;
    std::memcpy(&r, &u, 4);
    return r;
}

}  // namespace

bool conv_tc_supported(const TensorRef &in, const ConvGeom &g) {
    if (g.groups != 1 || g.pre_relu) return false;
    if ((reinterpret_cast<uintptr_t>(in.ptr) & 15) != 0 || (size_t(in.pitch) * in.esize) % 16 != 0) return false;
    if (g.sw > 8 || g.sh > 8) return false;            // TMA element strides are at most 8
    if (g.kh * g.kw > 4096) return false;
    return true;
}

// Tile selection.  A CTA costs a fixed overhead plus a K loop whose steps are bound by the slowest of
// three things -- the wait/issue chain of its single-thread roles (about 450 cycles per step, 700 in
// three-pass mode, whatever the tile's size), the tensor pipe, the TMA unit -- so the choice is made
// with a small cost model (cycles, fitted to a sweep over the 43 distinct Inception-v3 layers on B200):
//     step = max(issue chain of one CTA, tensor time of the resident CTAs, bytes loaded by them / TMA fill rate)
//     cta  = fixed + k_steps_per_cta * step + epilogue(bn) + cluster_overhead
//     time = waves * cta,  waves = ceil(ctas / how many fit at once)
// over every pixel-tile shape, output-channel tile width and K split that the kernel supports.
// It replaces the reference's run-time algorithm search (src/ios/ios_runtime.cu:150-205).
void conv_tc_choose(const ConvGeom &g, int sm_count, int concurrency_hint, bool three_pass, ConvTcPlan *plan, int force_bn,
                    bool bf16, bool allow_im2col) {
    ConvTcPlan &q = *plan;
    q.bf16 = bf16 ? 1 : 0;
    q.sm_count = sm_count;
    q.x3 = (three_pass && !bf16) ? 1 : 0;
    q.cluster = 1;
    // K elements per pipeline step = one operand row: 128 bytes, except that bfloat16 layers of at most 32
    // input channels use 64-byte rows (64-byte swizzle) -- half-empty 128-byte rows would cost the TMA
    // unit and shared memory twice the bytes for the same work
    q.half_rows = (bf16 && g.Cin <= 32 && !q.no_half_rows) ? 1 : 0;
    const int row_bytes = q.half_rows ? 64 : 128;
    const int chunk = bf16 ? (q.half_rows ? 32 : 64) : 32;
    const int bn_step = bf16 ? 64 : 32;          // output channels per 128-byte row of the store staging
    const bool flat = g.kh == 1 && g.kw == 1 && g.sh == 1 && g.sw == 1 && g.ph == 0 && g.pw == 0;
    q.flat_1x1 = flat ? 1 : 0;
    q.cchunks = ceil_div(g.Cin, chunk);
    q.k_iters = g.kh * g.kw * q.cchunks;

    struct Shape { int box_w, box_h, box_n, tiles_w, tiles_h, tiles_n, im2col; };
    std::vector<Shape> shapes;
    // A window with taps, padding or strides still tiles the flattened pixel axis when the TMA unit
    // walks it in im2col mode; its bounding-box corners are 8-bit signed offsets.
    bool im2col = allow_im2col && !flat && long(g.N) * g.OH * g.OW < (1l << 31) - kTileM;
    if (im2col) {
        int lo_w, up_w, lo_h, up_h;
        im2col_corners(g.W, g.OW, g.sw, g.pw, &lo_w, &up_w);
        im2col_corners(g.H, g.OH, g.sh, g.ph, &lo_h, &up_h);
        for (int v : {lo_w, up_w, lo_h, up_h}) im2col = im2col && v >= -128 && v <= 127;
        im2col = im2col && g.kw <= 65535 && g.kh <= 65535;
    }
    if (flat || im2col) {
        const long pixels = long(g.N) * g.OH * g.OW;
        const long tiles = (pixels + kTileM - 1) / kTileM;
        Shape sh;
        sh.box_w = int((pixels + tiles - 1) / tiles);
        sh.box_h = sh.box_n = 1;
        sh.tiles_w = int((pixels + sh.box_w - 1) / sh.box_w);
        sh.tiles_h = sh.tiles_n = 1;
        sh.im2col = im2col ? 1 : 0;
        shapes.push_back(sh);
    } else {
        const int max_w = std::min(kTileM, 256 / g.sw);
        const int min_parts = ceil_div(g.OW, max_w);
        for (int parts = min_parts; parts < min_parts + 4; ++parts) {
            Shape sh;
            sh.box_w = ceil_div(g.OW, parts);
            if (sh.box_w < 8 && parts > min_parts) break;
            sh.tiles_w = ceil_div(g.OW, sh.box_w);
            sh.box_h = std::min({g.OH, std::max(1, kTileM / sh.box_w), std::max(1, 256 / g.sh)});
            sh.tiles_h = ceil_div(g.OH, sh.box_h);
            const bool whole_image = sh.tiles_w == 1 && sh.box_h == g.OH;
            sh.box_n = whole_image ? std::min(g.N, std::max(1, kTileM / (g.OH * g.OW))) : 1;
            sh.tiles_n = ceil_div(g.N, sh.box_n);
            sh.im2col = 0;
            shapes.push_back(sh);
        }
    }
    // cycles; fitted to a sweep of tile width x split over the 43 distinct Inception-v3 layers at batch 1 and 64
    const double kFixed = 3000.0, kIssue = 450.0, kIssueThreePass = 700.0, kFillBytesPerCycle = 60.0, kEpiloguePerColumn = 36.0,
                 kClusterOverhead = 2000.0, kTensorPerColumn = 2.1 * 1.15;
    const int planes = q.x3 ? 2 : 1;
    const int share = std::max(1, concurrency_hint);
    double best_cost = 1e30;
    Shape best_shape = shapes[0];
    int best_bn = 32, best_split = 1;
    static const int splits[] = {1, 2, 4, 8};
    for (const Shape &sh : shapes) {
        const int m_tiles = sh.tiles_w * sh.tiles_h * sh.tiles_n;
        const int rows = sh.box_w * sh.box_h * sh.box_n;
        int last_bn = 0;
        for (int n_tiles = 1; n_tiles <= ceil_div(g.Cout, bn_step); ++n_tiles) {
            const int bn_max = 256;
            int bn = std::min(bn_max, ceil_div(ceil_div(g.Cout, n_tiles), bn_step) * bn_step);
            if (force_bn > 0) bn = std::min(bn_max, ceil_div(force_bn, bn_step) * bn_step);
            if (bn == last_bn) continue;
            last_bn = bn;
            const int nt = ceil_div(g.Cout, bn);
            const double load_bytes = double(rows) * row_bytes + double(planes) * bn * row_bytes;
            const double stage_bytes = double(planes) * (kTileM + bn) * row_bytes;
            const bool wide = q.x3 && bn <= 128;
            const double tensor = bn * kTensorPerColumn * (q.x3 ? 3.0 : 1.0);
            const double epilogue = bn * kEpiloguePerColumn * (wide ? 1.3 : 1.0);
            for (int split : splits) {
                if (split > 1 && split * 2 > q.k_iters) break;
                const long ctas = long(m_tiles) * nt * split;
                // a grid of several waves keeps two CTAs on an SM when two stages of each fit (conv_tc_set_split)
                const int resident = (split == 1 && ctas > sm_count && 2.0 * stage_bytes <= 108.0 * 1024) ? 2 : 1;
                const int fit = std::max(1, (split == 1 ? sm_count * resident : 8 * (16 / split) * split) / share);
                const double waves = double((ctas + fit - 1) / fit);
                // a K step costs what its slowest part costs: the issue chain of one CTA, or the SM's tensor
                // pipe and TMA unit shared by the resident CTAs
                const double step = std::max({q.x3 ? kIssueThreePass : kIssue, resident * tensor, resident * load_bytes / kFillBytesPerCycle});
                const double cta = kFixed + ceil_div(q.k_iters, split) * step + epilogue + (split > 1 ? kClusterOverhead : 0.0);
                const double cost = waves * cta;
                if (cost < best_cost) {
                    best_cost = cost;
                    best_shape = sh;
                    best_bn = bn;
                    best_split = split;
                }
            }
            if (force_bn > 0) break;
        }
    }
    q.box_w = best_shape.box_w; q.box_h = best_shape.box_h; q.box_n = best_shape.box_n;
    q.tiles_w = best_shape.tiles_w; q.tiles_h = best_shape.tiles_h; q.tiles_n = best_shape.tiles_n;
    q.im2col = best_shape.im2col;
    q.bn = best_bn;
    q.n_tiles = ceil_div(g.Cout, q.bn);
    q.cout_pad = q.n_tiles * q.bn;
    conv_tc_set_split(&q, best_split);
}

void conv_tc_set_split(ConvTcPlan *plan, int split) {
    ConvTcPlan &q = *plan;
    split = std::max(1, std::min(split, q.k_iters));
    const int base = q.tiles_w * q.tiles_h * q.tiles_n * q.n_tiles;
    q.split_k = split;
    const int stage_bytes = (q.x3 ? 2 : 1) * (kTileM + q.bn) * (q.half_rows ? 64 : 128);
    const int slab_channels = q.bf16 ? 64 : 32;
    const int per_split = ceil_div(q.k_iters, split);
    q.stages = std::max(2, std::min({8, per_split, (200 * 1024) / stage_bytes}));
    // A grid of several waves runs faster with two CTAs per SM (one CTA's set-up and epilogue hide
    // behind the other's K loop) than with one CTA and a deeper pipeline: keep such CTAs under half
    // of an SM's shared memory, three stages if they fit.
    if (long(base) * split > (q.sm_count > 0 ? q.sm_count : 148)) {
        const int fit = (108 * 1024) / stage_bytes;
        q.stages = std::max(2, std::min(q.stages, std::max(fit, 2)));
    }
    if (q.stages == 5 || q.stages == 7) --q.stages;    // a depth that 2, 3 or 4 producer lanes can share evenly
    if (split > 8) q.cluster = 0;          // larger splits go through the global workspace
    // the store staging needs one 16 KiB slab per 32 output channels inside the pipeline buffers
    while (q.stages * stage_bytes < ceil_div(q.bn, slab_channels) * kATileBytes) ++q.stages;
    q.smem_bytes = size_t(q.stages) * stage_bytes + 24 * q.stages + 64 + 1024;
    // A cluster exchanges its partial tiles through shared memory when an area for the rows a CTA finishes --
    // one slice per CTA of the cluster -- fits behind the pipeline (at the price of a stage, down to three).
    q.push = 0;
    q.recv_off = 0;
    if (split > 1 && q.cluster && !q.no_push) {
        const int recv_bytes = split * ceil_div(kTileM, split) * q.bn * 4;
        const int limit = 225 * 1024;                       // what a CTA may have, less the kernel's static shared memory
        const int staging = ceil_div(q.bn, slab_channels) * kATileBytes;
        auto recv_off = [&](int stages) { return (stages * stage_bytes + 24 * stages + 64 + 15) & ~15; };
        int stages = q.stages;
        while (stages > 3 && recv_off(stages) + recv_bytes + 1024 > limit) --stages;
        if (stages == 5 || stages == 7) --stages;
        if (recv_off(stages) + recv_bytes + 1024 <= limit && stages * stage_bytes >= staging) {
            q.push = 1;
            q.stages = stages;
            q.recv_off = recv_off(stages);
            q.smem_bytes = size_t(q.recv_off) + recv_bytes + 1024;
        }
    }
    // More tiles than CTAs that fit at once: persistent CTAs with two accumulators in TMEM, the store
    // staging in an area of its own behind the pipeline stages.
    q.persistent = 0;
    q.grid_ctas = base * split;
    const int sms = q.sm_count > 0 ? q.sm_count : 148;
    const int acc_cols = ((q.x3 && q.bn <= 128) ? 2 : 1) * ceil_div(q.bn, 32) * 32;
    if (split == 1 && !q.no_persistent && 2 * acc_cols <= 512) {
        const int staging = ceil_div(q.bn, slab_channels) * kATileBytes;
        const int fixed = staging + 24 * 8 + 64 + 1024;
        const int resident = (4 * acc_cols <= 512 && 2 * stage_bytes + fixed <= 110 * 1024) ? 2 : 1;
        if (base > sms * resident && 2 * stage_bytes + fixed <= 210 * 1024) {
            q.persistent = 1;
            q.grid_ctas = sms * resident;
            const int budget = (resident == 2 ? 110 : 210) * 1024;
            q.stages = std::max(2, std::min(8, (budget - fixed) / stage_bytes));
            if (q.stages == 5 || q.stages == 7) --q.stages;
            q.smem_bytes = size_t(q.stages) * stage_bytes + fixed;
            // a CTA that must have the SM's TMEM to itself also takes more than half of its shared memory,
            // so that no second CTA can be placed beside it only to wait for TMEM
            if (resident == 1) q.smem_bytes = std::max(q.smem_bytes, size_t(120 * 1024));
        }
    }
    // partial tiles meet in a workspace (one region per tile and split); splits of more than 8, which no
    // cluster covers, also need an arrival counter per tile
    q.workspace_bytes = (split > 1 && !q.push) ? size_t(base) * split * q.bn * kTileM * sizeof(float) : 0;
    q.counter_bytes = (split > 1 && !q.cluster) ? size_t(base) * sizeof(unsigned int) : 0;
}

static uint16_t bf16_round_host(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return uint16_t(u >> 16);   // inf / nan
    u += 0x00007FFFu + ((u >> 16) & 1u);                                // round to nearest even
    return uint16_t(u >> 16);
}

size_t conv_tc_packed_bytes(const ConvGeom &g, const ConvTcPlan &plan) {
    const size_t elems = size_t(plan.x3 ? 2 : 1) * plan.cout_pad * g.kh * g.kw * plan.cchunks * (plan.bf16 && !plan.half_rows ? 64 : 32);
    return elems * (plan.bf16 ? 2 : 4);
}

void conv_tc_pack_weights(const float *oihw, const ConvGeom &g, const ConvTcPlan &plan, void *packed_out) {
    const int taps = g.kh * g.kw;
    const int chunk = (plan.bf16 && !plan.half_rows) ? 64 : 32;
    const size_t row = size_t(taps) * plan.cchunks * chunk;
    const size_t plane = size_t(plan.cout_pad) * row;
    std::memset(packed_out, 0, conv_tc_packed_bytes(g, plan));
    float *packed = static_cast<float *>(packed_out);
    uint16_t *packed16 = static_cast<uint16_t *>(packed_out);
    for (int o = 0; o < g.Cout; ++o)
        for (int c = 0; c < g.Cin; ++c)
            for (int tp = 0; tp < taps; ++tp) {
                const float w = oihw[(size_t(o) * g.Cin + c) * taps + tp];
                const size_t at = size_t(o) * row + size_t(tp) * plan.cchunks * chunk + c;
                if (plan.bf16) {
                    packed16[at] = bf16_round_host(w);
                    continue;
                }
                const float hi = tf32_round_host(w);
                packed[at] = hi;
                if (plan.x3) packed[plane + at] = tf32_round_host(w - hi);   // residual plane
            }
}

const char *conv_tc_encode(const ConvTcParams &p, ConvTcPlan *plan) {
    EncodeTiledFn encode = encode_fn();
    if (!encode) return "cuTensorMapEncodeTiled is not available from the driver";
    const ConvGeom &g = p.g;
    ConvTcPlan &q = *plan;
    static thread_local char msg[160];
    const CUtensorMapDataType dtype = q.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const cuuint64_t esize = q.bf16 ? 2 : 4;
    const cuuint32_t chunk = (q.bf16 && !q.half_rows) ? 64 : 32;     // K elements per operand row
    const cuuint32_t slab = q.bf16 ? 64 : 32;                          // output channels per staging row
    const CUtensorMapSwizzle k_swizzle = q.half_rows ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
    auto fail = [&](const char *what, CUresult r) {
        std::snprintf(msg, sizeof msg, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, int(r));
        return msg;
    };
    {
        cuuint64_t dims[4];
        cuuint64_t strides[3];
        cuuint32_t box[4], estr[4];
        const cuuint64_t pix_bytes = cuuint64_t(p.in.pitch) * esize;
        if (q.patch) {
            // the input as (C, W, H, N) -- one-row windows: (C, W, N*H, 1) -- and a box of one tile's patch;
            // coordinates outside the image read zeros, which is the padding
            const cuuint64_t rows = q.patch_merged ? cuuint64_t(g.N) * g.H : cuuint64_t(g.H);
            dims[0] = cuuint64_t(g.Cin); dims[1] = cuuint64_t(g.W); dims[2] = rows; dims[3] = q.patch_merged ? 1 : cuuint64_t(g.N);
            strides[0] = pix_bytes; strides[1] = pix_bytes * g.W; strides[2] = pix_bytes * g.W * rows;
            box[0] = chunk; box[1] = cuuint32_t(q.patch_pw); box[2] = cuuint32_t(q.patch_ph); box[3] = cuuint32_t(q.box_n);
            estr[0] = estr[1] = estr[2] = estr[3] = 1;
        } else if (q.flat_1x1) {
            dims[0] = cuuint64_t(g.Cin); dims[1] = cuuint64_t(g.N) * g.H * g.W; dims[2] = 1; dims[3] = 1;
            strides[0] = pix_bytes; strides[1] = pix_bytes * dims[1]; strides[2] = strides[1];
            box[0] = chunk; box[1] = cuuint32_t(q.box_w); box[2] = 1; box[3] = 1;
            estr[0] = estr[1] = estr[2] = estr[3] = 1;
        } else if (q.im2col) {
            EncodeIm2colFn encode_im2col = encode_im2col_fn();
            if (!encode_im2col) return "cuTensorMapEncodeIm2col is not available from the driver";
            dims[0] = cuuint64_t(g.Cin); dims[1] = cuuint64_t(g.W); dims[2] = cuuint64_t(g.H); dims[3] = cuuint64_t(g.N);
            strides[0] = pix_bytes; strides[1] = pix_bytes * g.W; strides[2] = pix_bytes * g.W * g.H;
            estr[0] = 1; estr[1] = cuuint32_t(g.sw); estr[2] = cuuint32_t(g.sh); estr[3] = 1;
            int lower[2], upper[2];                      // w, h
            im2col_corners(g.W, g.OW, g.sw, g.pw, &lower[0], &upper[0]);
            im2col_corners(g.H, g.OH, g.sh, g.ph, &lower[1], &upper[1]);
            CUresult r = encode_im2col(reinterpret_cast<CUtensorMap *>(q.tmap_a), dtype, 4, p.in.ptr, dims, strides, lower,
                                       upper, chunk, cuuint32_t(q.box_w), estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       k_swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail("activations, im2col", r);
        } else {
            dims[0] = cuuint64_t(g.Cin); dims[1] = cuuint64_t(g.W); dims[2] = cuuint64_t(g.H); dims[3] = cuuint64_t(g.N);
            strides[0] = pix_bytes; strides[1] = pix_bytes * g.W; strides[2] = pix_bytes * g.W * g.H;
            box[0] = chunk; box[1] = cuuint32_t(q.box_w * g.sw); box[2] = cuuint32_t(q.box_h * g.sh); box[3] = cuuint32_t(q.box_n);
            estr[0] = 1; estr[1] = cuuint32_t(g.sw); estr[2] = cuuint32_t(g.sh); estr[3] = 1;
        }
        if (!q.im2col) {
            CUresult r = encode(reinterpret_cast<CUtensorMap *>(q.tmap_a), dtype, 4, p.in.ptr, dims,
                                strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, k_swizzle,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail("activations", r);
        }
    }
    {
        const cuuint64_t krow = cuuint64_t(g.kh) * g.kw * q.cchunks * chunk;
        cuuint64_t dims[2] = {krow, cuuint64_t(q.cout_pad) * (q.x3 ? 2 : 1)};
        cuuint64_t strides[1] = {krow * esize};
        cuuint32_t box[2] = {chunk, cuuint32_t(q.bn)};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = encode(reinterpret_cast<CUtensorMap *>(q.tmap_b), dtype, 2,
                            const_cast<void *>(p.weight_packed), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            k_swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail("weights", r);
    }
    // the output window: bulk tensor stores need a 16-byte aligned base
    // and a window whose end is 16-byte aligned too, so that clipping never lands inside a 16-byte unit
    const int per16 = int(16 / esize);
    q.tma_store = ((reinterpret_cast<uintptr_t>(p.out.ptr) & 15) == 0 && p.out.pitch % per16 == 0 && g.Cout % per16 == 0) ? 1 : 0;
    if (q.patch && !q.patch_staging) q.tma_store = 0;   // (tiles of many short row segments are stored from registers)
    std::memcpy(q.tmap_c, q.tmap_a, sizeof q.tmap_c);
    if (q.tma_store && q.patch) {
        // one store per output row segment of a patch tile: a box of box_w pixels of one row, 128 bytes of channels
        const cuuint64_t rows = q.patch_merged ? cuuint64_t(g.N) * g.OH : cuuint64_t(g.OH);
        const cuuint64_t pix_bytes = cuuint64_t(p.out.pitch) * esize;
        cuuint64_t dims[4] = {cuuint64_t(g.Cout), cuuint64_t(g.OW), rows, q.patch_merged ? 1 : cuuint64_t(g.N)};
        cuuint64_t strides[3] = {pix_bytes, pix_bytes * g.OW, pix_bytes * g.OW * rows};
        cuuint32_t box[4] = {slab, cuuint32_t(q.box_w), 1, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = encode(reinterpret_cast<CUtensorMap *>(q.tmap_c), dtype, 4, p.out.ptr, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail("output, row segments", r);
    } else if (q.tma_store) {
        cuuint64_t dims[4];
        cuuint64_t strides[3];
        cuuint32_t box[4];
        cuuint32_t estr[4] = {1, 1, 1, 1};
        const cuuint64_t pix_bytes = cuuint64_t(p.out.pitch) * esize;
        if (q.flat_1x1 || q.im2col) {
            dims[0] = cuuint64_t(g.Cout); dims[1] = cuuint64_t(g.N) * g.OH * g.OW; dims[2] = 1; dims[3] = 1;
            strides[0] = pix_bytes; strides[1] = pix_bytes * dims[1]; strides[2] = strides[1];
            box[0] = slab; box[1] = cuuint32_t(q.box_w); box[2] = 1; box[3] = 1;
        } else {
            dims[0] = cuuint64_t(g.Cout); dims[1] = cuuint64_t(g.OW); dims[2] = cuuint64_t(g.OH); dims[3] = cuuint64_t(g.N);
            strides[0] = pix_bytes; strides[1] = pix_bytes * g.OW; strides[2] = pix_bytes * g.OW * g.OH;
            box[0] = slab; box[1] = cuuint32_t(q.box_w); box[2] = cuuint32_t(q.box_h); box[3] = cuuint32_t(q.box_n);
        }
        CUresult r = encode(reinterpret_cast<CUtensorMap *>(q.tmap_c), dtype, 4, p.out.ptr, dims,
                            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail("output", r);
    }
    return nullptr;
}

const char *conv_tc_encode_dense_weights(const ConvTcParams &p, ConvTcPlan *plan) {
    // same as conv_tc_encode, but the weight matrix is the caller's dense [Cout][Cin] array (a 1x1
    // convolution's OIHW weights): rows and columns beyond it are filled with zeros by the TMA unit
    const char *err = conv_tc_encode(p, plan);
    if (err) return err;
    EncodeTiledFn encode = encode_fn();
    const ConvGeom &g = p.g;
    cuuint64_t dims[2] = {cuuint64_t(g.Cin), cuuint64_t(g.Cout)};
    cuuint64_t strides[1] = {cuuint64_t(g.Cin) * 4};
    cuuint32_t box[2] = {kChunk, cuuint32_t(plan->bn)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(reinterpret_cast<CUtensorMap *>(plan->tmap_b), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                        const_cast<void *>(p.weight_packed), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? nullptr : "cuTensorMapEncodeTiled(dense weights) failed";
}

cudaError_t conv_tc_prepare() {
    const void *forms[] = {
#define IOS_FORMS(MODE)                                                                                          \
    reinterpret_cast<const void *>(conv_tc_kernel<MODE, false, false>), reinterpret_cast<const void *>(conv_tc_kernel<MODE, true, false>), \
    reinterpret_cast<const void *>(conv_tc_kernel<MODE, false, true>), reinterpret_cast<const void *>(conv_tc_kernel<MODE, true, true>)
        IOS_FORMS(0), IOS_FORMS(1), IOS_FORMS(2), IOS_FORMS(4)
#undef IOS_FORMS
    };
    for (const void *form : forms) {
        cudaError_t err = cudaFuncSetAttribute(form, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
        if (err != cudaSuccess) return err;
    }
    const void *resident[] = {reinterpret_cast<const void *>(conv_tc_persistent_kernel<0>), reinterpret_cast<const void *>(conv_tc_persistent_kernel<1>),
                              reinterpret_cast<const void *>(conv_tc_persistent_kernel<2>), reinterpret_cast<const void *>(conv_tc_persistent_kernel<4>)};
    for (const void *form : resident) {
        cudaError_t err = cudaFuncSetAttribute(form, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);
        if (err != cudaSuccess) return err;
    }
    return conv_tc_patch_prepare();
}

void launch_conv_tc(const ConvTcParams &p, const ConvTcPlan &q, cudaStream_t stream) {
    if (q.patch) {
        launch_conv_tc_patch(p, q, stream);
        return;
    }
    TileGeom t;
    t.box_w = q.box_w; t.box_h = q.box_h; t.box_n = q.box_n;
    t.tiles_w = q.tiles_w; t.tiles_h = q.tiles_h;
    t.bn = q.bn; t.cchunks = q.cchunks; t.k_iters = q.k_iters; t.split_k = q.split_k; t.stages = q.stages;
    t.producers = 1;
    // lanes run in lockstep, so every lane's stage must be free before any of them refills: at most half
    // of the stages are refilled together
    // (measured: two lanes pay off from six stages on; never in three-pass mode, whose stages pass through
    // the residual split on their way to the tensor core and are few)
    for (int cand = 2; cand <= (q.max_producers > 0 ? q.max_producers : 4) && cand <= 8 && cand * 3 <= q.stages && !q.x3; ++cand)
        if (q.stages % cand == 0) t.producers = cand;
    t.flat = (q.flat_1x1 || q.im2col) ? 1 : 0;
    t.im2col = q.im2col;
    const int row_bytes = q.half_rows ? 64 : 128;
    t.a_bytes = q.box_w * q.box_h * q.box_n * row_bytes;
    t.bf16 = q.bf16;
    t.chunk = (q.bf16 && !q.half_rows) ? 64 : 32;
    t.slab = q.bf16 ? 64 : 32;
    t.wide = (q.x3 && q.bn <= 128) ? 1 : 0;
    // two issuers (three accumulator ranges) when tensor memory has room: this kernel has the SM's to itself
    // unless a second CTA shares the SM, and then 3 x bn columns of each must fit side by side
    t.dual = (t.wide && !q.persistent && !q.no_dual && 3 * q.bn <= ((q.split_k > 1 && q.cluster) ? 512 : 256)) ? 1 : 0;
    if (!q.x3 && !q.persistent && !q.no_dual && 2 * q.bn <= ((q.split_k > 1 && q.cluster) ? 512 : 256)) t.dual = 2;
    int cols = 32;
    while (cols < (t.dual == 1 ? 3 : (t.wide || t.dual == 2) ? 2 : 1) * q.bn) cols *= 2;   // further accumulator ranges
    t.tmem_cols = cols;
    t.round_tf32 = p.g.round_out;
    t.x3 = q.x3;
    t.cout_pad = q.cout_pad;
    t.tma_store = q.tma_store;
    t.cluster = (q.split_k > 1 && q.cluster) ? 1 : 0;
    t.push = (t.cluster && q.push) ? 1 : 0;
    t.recv_off = q.recv_off;
    t.split_shift = -1;
    for (int sh = 0; sh < 8; ++sh)
        if ((1 << sh) == q.split_k) t.split_shift = sh;
    // multipliers for the prologue's divisions, where the dividend is small enough for them to be exact
    auto magic = [](long n_max, int d) -> unsigned {
        return (d > 1 && n_max * d < (1l << 32)) ? unsigned((1ull << 32) / unsigned(d)) + 1u : 0u;
    };
    t.magic_ow = magic(long(p.g.OH) * p.g.OW, p.g.OW);
    t.magic_cc = magic(long(q.k_iters) + 64, q.cchunks);
    t.magic_kw = magic(long(p.g.kh) * p.g.kw + 64, p.g.kw);
    cudaLaunchConfig_t cfg = {};
    PersistGeom pg = {};
    if (q.persistent) {
        pg.n_tiles = q.n_tiles;
        pg.total_tiles = q.tiles_w * q.tiles_h * q.tiles_n * q.n_tiles;
        pg.staging_off = q.stages * (q.x3 ? 2 : 1) * (kTileM + q.bn) * row_bytes;
        pg.acc_stride = (t.wide ? 2 : 1) * ceil_div(q.bn, 32) * 32;
        cols = 32;
        while (cols < 2 * pg.acc_stride) cols *= 2;
        t.tmem_cols = cols;
        cfg.gridDim = dim3(std::min(q.grid_ctas, pg.total_tiles));
        cfg.blockDim = dim3(kPersistThreads);
    } else {
        cfg.gridDim = dim3(q.tiles_w * q.tiles_h * q.tiles_n, q.n_tiles, q.split_k);
        cfg.blockDim = dim3(q.x3 ? kThreads : t.dual == 2 ? 224 : 192);     // (warp 6: second issuer; warps 7..10: three-pass mode only)
    }
    cfg.dynamicSmemBytes = q.smem_bytes;
    cfg.stream = stream;
    // programmatic dependent launch: this kernel's prologue may overlap the tail of its predecessor
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (q.pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (t.cluster) {                      // the split_k CTAs of one output tile form a cluster
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = unsigned(q.split_k);
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    const CUtensorMap &ma = *reinterpret_cast<const CUtensorMap *>(q.tmap_a), &mb = *reinterpret_cast<const CUtensorMap *>(q.tmap_b),
                      &mc = *reinterpret_cast<const CUtensorMap *>(q.tmap_c);
    const int mode = q.x3 ? 1 : (q.bf16 ? (q.half_rows ? 4 : 2) : 0);
    if (q.persistent) {
        if (mode == 1) cudaLaunchKernelEx(&cfg, conv_tc_persistent_kernel<1>, ma, mb, mc, p, t, pg);
        else if (mode == 2) cudaLaunchKernelEx(&cfg, conv_tc_persistent_kernel<2>, ma, mb, mc, p, t, pg);
        else if (mode == 4) cudaLaunchKernelEx(&cfg, conv_tc_persistent_kernel<4>, ma, mb, mc, p, t, pg);
        else cudaLaunchKernelEx(&cfg, conv_tc_persistent_kernel<0>, ma, mb, mc, p, t, pg);
        return;
    }
    const bool stamps = p.timeline != nullptr;
#define IOS_LAUNCH(MODE)                                                                                         \
    do {                                                                                                         \
        if (t.cluster) {                                                                                         \
            if (stamps) cudaLaunchKernelEx(&cfg, conv_tc_kernel<MODE, true, true>, ma, mb, mc, p, t);            \
            else cudaLaunchKernelEx(&cfg, conv_tc_kernel<MODE, true, false>, ma, mb, mc, p, t);                  \
        } else {                                                                                                 \
            if (stamps) cudaLaunchKernelEx(&cfg, conv_tc_kernel<MODE, false, true>, ma, mb, mc, p, t);           \
            else cudaLaunchKernelEx(&cfg, conv_tc_kernel<MODE, false, false>, ma, mb, mc, p, t);                 \
        }                                                                                                        \
    } while (0)
    if (mode == 1) IOS_LAUNCH(1);
    else if (mode == 2) IOS_LAUNCH(2);
    else if (mode == 4) IOS_LAUNCH(4);
    else IOS_LAUNCH(0);
#undef IOS_LAUNCH
}

}  // namespace ios
