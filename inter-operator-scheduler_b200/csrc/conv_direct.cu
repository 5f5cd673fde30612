// CUDA-core convolutions: the general grouped kernel (exact fp32 products; used for shapes and
// views the tensor-core kernel does not take) and the depthwise kernel.
//
// Depthwise 3x3 (groups == Cin == Cout; 96 of the 195 convolutions of RandWire) has one
// multiply-add per loaded weight and nine per loaded activation: it is bound by HBM/L2 bandwidth,
// not by a contraction, so it runs on CUDA cores with 16-byte accesses along the channel axis and
// can fold the ReLU that precedes it in a ReluSepConv (python/ios/models/common.py:406-444).
// Both replace cudnnConvolutionForward / cudnnConvolutionBiasActivationForward call sites
// (src/ios/ios_runtime.cu:313-331) for their shapes.
#include "kernels.h"
#include <cstdlib>

#include <cuda_bf16.h>

#include <algorithm>
#include <cstring>

namespace ios {
namespace {

// sigmoid / tanh are rare; inlined, their code would be executed under predication by every thread
__device__ __noinline__ float act_slow(float v, int act) {
    return act == 2 ? 1.0f / (1.0f + __expf(-v)) : tanhf(v);
}
__device__ __forceinline__ float act_only(float v, int act) {
    if (act == 1) return fmaxf(v, 0.0f);
    if (act == 0) return v;
    return act_slow(v, act);
}
__device__ __forceinline__ float to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}
// activation, then the optional rounding for a tensor-core consumer
#define act_apply(v, act) finish_value((v), (act), g.round_out)
__device__ __forceinline__ float finish_value(float v, int act, int round_out) {
    v = act_only(v, act);
    return round_out ? to_tf32(v) : v;
}

// ---- element access (activations are float32 or bfloat16; weights, bias and arithmetic float32) ----
__device__ __forceinline__ float load1(const float *p) { return *p; }
__device__ __forceinline__ float load1(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
__device__ __forceinline__ void store1(float *p, float v) { *p = v; }
__device__ __forceinline__ void store1(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float4 load4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16 *p) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t *>(&lo);
    raw.y = *reinterpret_cast<const uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(p) = raw;
}

// One thread per (pixel, 4 consecutive output channels of one group); consecutive threads take
// consecutive channel quads, so weight reads are coalesced and the activation read is a broadcast.
constexpr int kCoPerThread = 4;

template <typename T>
__global__ void __launch_bounds__(128) conv_direct_kernel(const ConvDirectParams p) {
    grid_dependency_entry();
    const ConvGeom &g = p.g;
    const int cin_g = g.Cin / g.groups, cout_g = g.Cout / g.groups;
    const int quads_g = (cout_g + kCoPerThread - 1) / kCoPerThread;
    const int quads = quads_g * g.groups;
    const long total = long(g.N) * g.OH * g.OW * quads;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        long pix = i / quads;
        const int q = static_cast<int>(i - pix * quads);
        const int grp = q / quads_g;
        const int co0 = grp * cout_g + (q - grp * quads_g) * kCoPerThread;   // first output channel
        const int co_end = min(co0 + kCoPerThread, (grp + 1) * cout_g);
        const int ow = static_cast<int>(pix % g.OW);
        pix /= g.OW;
        const int oh = static_cast<int>(pix % g.OH);
        const int n = static_cast<int>(pix / g.OH);
        float acc[kCoPerThread] = {0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < g.kh; ++r) {
            const int h = oh * g.sh - g.ph + r;
            if (h < 0 || h >= g.H) continue;
            for (int s = 0; s < g.kw; ++s) {
                const int w = ow * g.sw - g.pw + s;
                if (w < 0 || w >= g.W) continue;
                const T *x = p.in.as<const T>() + ((long(n) * g.H + h) * g.W + w) * p.in.pitch + grp * cin_g;
                const float *wt = p.weight + (long(r * g.kw + s) * cin_g) * g.Cout;
                for (int c = 0; c < cin_g; ++c) {
                    float xv = load1(x + c);
                    if (g.pre_relu) xv = fmaxf(xv, 0.0f);
                    const float *wrow = wt + long(c) * g.Cout;
#pragma unroll
                    for (int j = 0; j < kCoPerThread; ++j)
                        if (co0 + j < co_end) acc[j] = fmaf(xv, wrow[co0 + j], acc[j]);
                }
            }
        }
        T *y = p.out.as<T>() + ((long(n) * g.OH + oh) * g.OW + ow) * p.out.pitch;
#pragma unroll
        for (int j = 0; j < kCoPerThread; ++j)
            if (co0 + j < co_end) store1(y + co0 + j, act_apply(acc[j] + (p.bias ? p.bias[co0 + j] : 0.0f), g.act));
    }
}

// ---- few input channels (the 3-channel stem of every network) ---------------------------------
// With 3 input channels an implicit-GEMM K step is one filter tap of a 128-byte row that is 90 %
// padding, and the layer is bound by the bytes it writes, not by a contraction.  Here a thread owns
// CG output channels (32 if Cout allows) of 2 output pixels: per tap it reads each pixel once (16
// bytes) and every weight as part of a float4 broadcast from shared memory, so that four of five
// instructions are multiply-adds.  The filter sits in shared memory as [tap][cin][CG/4][Cout/CG]
// float4 -- the threads of one pixel, which differ in their channel group, read neighbouring words --
// and the threads of a pixel together write its channels as one contiguous span.  Products and sums
// are float32.  KH, KW: the window if known at compile time (3x3: fully unrolled), else 0; kPadded:
// windows may reach outside the image.
template <typename T, int CG, int PX, int KH, int KW, bool kPadded>
__global__ void __launch_bounds__(128, 4) conv_few_channels_kernel(const ConvDirectParams p, int pixels_per_block) {
    grid_dependency_entry();
    extern __shared__ float4 w_s4[];
    constexpr int Q = CG / 4;
    const ConvGeom &g = p.g;
    const int kh = KH ? KH : g.kh, kw = KW ? KW : g.kw;
    const int groups = g.Cout / CG;
    {
        // global [tap][cin][Cout] -> shared [tap][cin][k][group] float4, Cout index = group * CG + 4 k + e
        const int n4 = (kh * kw * g.Cin * g.Cout) >> 2;
        const float4 *src = reinterpret_cast<const float4 *>(p.weight);
        const int per_row = g.Cout >> 2;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const int row = i / per_row, co4 = i - row * per_row;      // row = tap * Cin + cin
            const int j = co4 / Q, k = co4 - j * Q;
            w_s4[(row * Q + k) * groups + j] = src[i];
        }
    }
    __syncthreads();
    const int j = threadIdx.x % groups, lp = threadIdx.x / groups;
    const int per_image = g.OH * g.OW;
    const int total = g.N * per_image;
    const T *in = p.in.as<const T>();
    T *out = p.out.as<T>();
    const int row_step = g.W * p.in.pitch;              // elements from one input row to the next
    const float4 *wj = w_s4 + j;
    // PX pixels per thread, pixels_per_block apart: they share every weight load
    for (int pix0 = blockIdx.x * PX * pixels_per_block + lp; pix0 < total; pix0 += gridDim.x * PX * pixels_per_block) {
        const T *corner[PX];                             // input pixel under the window's first tap
        int h0[PX], w0[PX];
        bool live[PX];
#pragma unroll
        for (int u = 0; u < PX; ++u) {
            const int pix = pix0 + u * pixels_per_block;
            live[u] = pix < total;
            const int pc = live[u] ? pix : pix0;
            const int n = pc / per_image;
            const int rem = pc - n * per_image;
            const int oh = rem / g.OW;
            h0[u] = oh * g.sh - g.ph;
            w0[u] = (rem - oh * g.OW) * g.sw - g.pw;
            corner[u] = in + (size_t(n) * g.H + h0[u]) * row_step + w0[u] * p.in.pitch;
        }
        float acc[PX][CG];
#pragma unroll
        for (int u = 0; u < PX; ++u)
#pragma unroll
            for (int e = 0; e < CG; ++e) acc[u][e] = 0.0f;
        auto tap = [&](int r, int s) {
            float x[PX][4];
#pragma unroll
            for (int u = 0; u < PX; ++u) {
                const bool inside = !kPadded || (h0[u] + r >= 0 && h0[u] + r < g.H && w0[u] + s >= 0 && w0[u] + s < g.W);
                const float4 v = inside ? load4(corner[u] + r * row_step + s * p.in.pitch) : make_float4(0.f, 0.f, 0.f, 0.f);
                x[u][0] = v.x; x[u][1] = v.y; x[u][2] = v.z; x[u][3] = v.w;
            }
            const float4 *wt = wj + (r * kw + s) * g.Cin * Q * groups;
            // channels beyond Cin are padding of the pixel pitch and never enter a product
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (c < g.Cin) {
#pragma unroll
                    for (int k = 0; k < Q; ++k) {
                        const float4 wv = wt[(c * Q + k) * groups];
#pragma unroll
                        for (int u = 0; u < PX; ++u) {
                            acc[u][4 * k + 0] = fmaf(x[u][c], wv.x, acc[u][4 * k + 0]);
                            acc[u][4 * k + 1] = fmaf(x[u][c], wv.y, acc[u][4 * k + 1]);
                            acc[u][4 * k + 2] = fmaf(x[u][c], wv.z, acc[u][4 * k + 2]);
                            acc[u][4 * k + 3] = fmaf(x[u][c], wv.w, acc[u][4 * k + 3]);
                        }
                    }
                }
            }
        };
        if (KH && KW) {
#pragma unroll
            for (int r = 0; r < (KH ? KH : 1); ++r)
#pragma unroll
                for (int s = 0; s < (KW ? KW : 1); ++s) tap(r, s);
        } else {
#pragma unroll 1
            for (int r = 0; r < kh; ++r)
#pragma unroll 1
                for (int s = 0; s < kw; ++s) tap(r, s);
        }
        const float *bias = p.bias ? p.bias + j * CG : nullptr;
#pragma unroll
        for (int u = 0; u < PX; ++u) {
            if (!live[u]) continue;
            T *dst = out + size_t(pix0 + u * pixels_per_block) * p.out.pitch + j * CG;
#pragma unroll
            for (int k = 0; k < Q; ++k) {
                const float4 b = bias ? *reinterpret_cast<const float4 *>(bias + 4 * k) : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 o;
                o.x = act_apply(acc[u][4 * k + 0] + b.x, g.act); o.y = act_apply(acc[u][4 * k + 1] + b.y, g.act);
                o.z = act_apply(acc[u][4 * k + 2] + b.z, g.act); o.w = act_apply(acc[u][4 * k + 3] + b.w, g.act);
                store4(dst + 4 * k, o);
            }
        }
    }
}

template <typename T, int CG, int PX>
void launch_few_channels_cg(const ConvDirectParams &p, cudaStream_t stream) {
    const ConvGeom &g = p.g;
    const int groups = g.Cout / CG;
    const int pixels_per_block = std::max(1, 128 / groups);
    const size_t smem = size_t(g.kh) * g.kw * g.Cin * g.Cout * sizeof(float);
    const long spans = (long(g.N) * g.OH * g.OW + PX * pixels_per_block - 1) / (PX * pixels_per_block);
    const int grid = int(std::min<long>(spans, 148L * 16));
    const int threads = groups * pixels_per_block;
    const bool padded = g.ph > 0 || g.pw > 0 || (g.OH - 1) * g.sh + g.kh > g.H || (g.OW - 1) * g.sw + g.kw > g.W;
    static bool raised = false;               // filters above 48 KiB need the opt-in limit
    if (!raised) {
        cudaFuncSetAttribute(conv_few_channels_kernel<T, CG, PX, 0, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        cudaFuncSetAttribute(conv_few_channels_kernel<T, CG, PX, 3, 3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        cudaFuncSetAttribute(conv_few_channels_kernel<T, CG, PX, 3, 3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        raised = true;
    }
    if (g.kh == 3 && g.kw == 3 && !padded) conv_few_channels_kernel<T, CG, PX, 3, 3, false><<<grid, threads, smem, stream>>>(p, pixels_per_block);
    else if (g.kh == 3 && g.kw == 3) conv_few_channels_kernel<T, CG, PX, 3, 3, true><<<grid, threads, smem, stream>>>(p, pixels_per_block);
    else conv_few_channels_kernel<T, CG, PX, 0, 0, true><<<grid, threads, smem, stream>>>(p, pixels_per_block);
}

template <typename T>
void launch_few_channels(const ConvDirectParams &p, cudaStream_t stream) {
    const int cout = p.g.Cout;
    // (measured on B200, 3 -> 32 channels, 3x3 stride 2 at 299 x 299: 8 channels x 4 pixels per thread -- 32 accumulators,
    //  every weight read from shared memory used for four pixels, no register spills -- beats 32 x 2 by 10-17 %)
    if (cout % 8 == 0) launch_few_channels_cg<T, 8, 4>(p, stream);
    else launch_few_channels_cg<T, 4, 2>(p, stream);
}

template <typename T, bool kVec>
__global__ void __launch_bounds__(256) conv_depthwise_kernel(const ConvDirectParams p) {
    grid_dependency_entry();
    const ConvGeom &g = p.g;
    const int lanes = kVec ? (g.Cout + 3) / 4 : g.Cout;   // the last group may be partial: stored element by element
    const int wrow = (g.Cout + 3) / 4 * 4;                // packed weight rows are padded to a multiple of 4
    const long total = long(g.N) * g.OH * g.OW * lanes;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        long pix = i / lanes;
        const int c = static_cast<int>(i - pix * lanes);
        const int ow = static_cast<int>(pix % g.OW);
        pix /= g.OW;
        const int oh = static_cast<int>(pix % g.OH);
        const int n = static_cast<int>(pix / g.OH);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < g.kh; ++r) {
            const int h = oh * g.sh - g.ph + r;
            if (h < 0 || h >= g.H) continue;
            for (int s = 0; s < g.kw; ++s) {
                const int w = ow * g.sw - g.pw + s;
                if (w < 0 || w >= g.W) continue;
                const T *x = p.in.as<const T>() + ((long(n) * g.H + h) * g.W + w) * p.in.pitch;
                const float *wt = p.weight + long(r * g.kw + s) * wrow;
                if (kVec) {
                    float4 xv = load4(x + 4 * c);
                    const float4 wv = *reinterpret_cast<const float4 *>(wt + 4 * c);
                    if (g.pre_relu) {
                        xv.x = fmaxf(xv.x, 0.f); xv.y = fmaxf(xv.y, 0.f); xv.z = fmaxf(xv.z, 0.f); xv.w = fmaxf(xv.w, 0.f);
                    }
                    acc.x = fmaf(xv.x, wv.x, acc.x); acc.y = fmaf(xv.y, wv.y, acc.y);
                    acc.z = fmaf(xv.z, wv.z, acc.z); acc.w = fmaf(xv.w, wv.w, acc.w);
                } else {
                    float xv = load1(x + c);
                    if (g.pre_relu) xv = fmaxf(xv, 0.f);
                    acc.x = fmaf(xv, wt[c], acc.x);
                }
            }
        }
        T *y = p.out.as<T>() + ((long(n) * g.OH + oh) * g.OW + ow) * p.out.pitch;
        if (kVec) {
            float4 b = p.bias ? *reinterpret_cast<const float4 *>(p.bias + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 o;
            o.x = act_apply(acc.x + b.x, g.act); o.y = act_apply(acc.y + b.y, g.act);
            o.z = act_apply(acc.z + b.z, g.act); o.w = act_apply(acc.w + b.w, g.act);
            if (4 * c + 4 <= g.Cout) {
                store4(y + 4 * c, o);
            } else {
                const float a[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (4 * c + j < g.Cout) store1(y + 4 * c + j, a[j]);
            }
        } else {
            store1(y + c, act_apply(acc.x + (p.bias ? p.bias[c] : 0.f), g.act));
        }
    }
}

inline int blocks_for(long work, int threads) {
    long b = (work + threads - 1) / threads;
    if (b < 1) b = 1;
    if (b > 148L * 64) b = 148L * 64;
    return static_cast<int>(b);
}

}  // namespace

bool conv_few_channels_supported(const TensorRef &in, const TensorRef &out, const ConvGeom &g) {
    const size_t filter_bytes = size_t(g.kh) * g.kw * g.Cin * g.Cout * sizeof(float);
    return g.groups == 1 && g.Cin <= 4 && !g.pre_relu && g.Cout % 4 == 0 && g.Cout >= 4 && g.Cout <= 512 &&
           filter_bytes <= 96 * 1024 && in.vec4() && out.vec4() && long(g.N) * g.OH * g.OW < (1l << 30);
}

void launch_conv_direct(const ConvDirectParams &p, cudaStream_t stream) {
    const ConvGeom &g = p.g;
    if (conv_few_channels_supported(p.in, p.out, g) && (reinterpret_cast<uintptr_t>(p.weight) & 15) == 0 &&
        (!p.bias || (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0)) {
        if (p.in.esize == 2) launch_few_channels<__nv_bfloat16>(p, stream);
        else launch_few_channels<float>(p, stream);
        return;
    }
    const int cout_g = g.Cout / g.groups;
    const long work = long(g.N) * g.OH * g.OW * ((cout_g + kCoPerThread - 1) / kCoPerThread) * g.groups;
    if (p.in.esize == 2) conv_direct_kernel<__nv_bfloat16><<<blocks_for(work, 128), 128, 0, stream>>>(p);
    else conv_direct_kernel<float><<<blocks_for(work, 128), 128, 0, stream>>>(p);
}

void launch_conv_depthwise(const ConvDirectParams &p, cudaStream_t stream) {
    const ConvGeom &g = p.g;
    const bool vec = p.in.vec4() && p.out.vec4() &&
                     ((reinterpret_cast<uintptr_t>(p.weight) & 15) == 0) &&
                     (!p.bias || (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0);
    const long work = long(g.N) * g.OH * g.OW * (vec ? (g.Cout + 3) / 4 : g.Cout);
    if (p.in.esize == 2) {
        if (vec) conv_depthwise_kernel<__nv_bfloat16, true><<<blocks_for(work, 256), 256, 0, stream>>>(p);
        else conv_depthwise_kernel<__nv_bfloat16, false><<<blocks_for(work, 256), 256, 0, stream>>>(p);
    } else {
        if (vec) conv_depthwise_kernel<float, true><<<blocks_for(work, 256), 256, 0, stream>>>(p);
        else conv_depthwise_kernel<float, false><<<blocks_for(work, 256), 256, 0, stream>>>(p);
    }
}

void conv_direct_pack_weights(const float *oihw, const ConvGeom &g, float *packed) {
    const int cin_g = g.Cin / g.groups, taps = g.kh * g.kw;
    for (int o = 0; o < g.Cout; ++o)
        for (int c = 0; c < cin_g; ++c)
            for (int t = 0; t < taps; ++t)
                packed[(size_t(t) * cin_g + c) * g.Cout + o] = oihw[(size_t(o) * cin_g + c) * taps + t];
}

void conv_depthwise_pack_weights(const float *oihw, const ConvGeom &g, float *packed) {
    const int taps = g.kh * g.kw;
    const int wrow = (g.Cout + 3) / 4 * 4;
    std::memset(packed, 0, size_t(taps) * wrow * sizeof(float));
    for (int o = 0; o < g.Cout; ++o)
        for (int t = 0; t < taps; ++t) packed[size_t(t) * wrow + o] = oihw[size_t(o) * taps + t];
}

}  // namespace ios
