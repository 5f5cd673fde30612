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

#include <cuda_bf16.h>

#include <cstring>

namespace ios {
namespace {

__device__ __forceinline__ float act_only(float v, int act) {
    switch (act) {
        case 1: return fmaxf(v, 0.0f);
        case 2: return 1.0f / (1.0f + __expf(-v));
        case 3: return tanhf(v);
        default: return v;
    }
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

template <typename T, bool kVec>
__global__ void __launch_bounds__(256) conv_depthwise_kernel(const ConvDirectParams p) {
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

void launch_conv_direct(const ConvDirectParams &p, cudaStream_t stream) {
    const ConvGeom &g = p.g;
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
