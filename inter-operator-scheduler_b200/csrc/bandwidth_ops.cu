// HBM-bound operators: k-way sum / product with activation (also the strided copy), window and
// global pooling, NCHW <-> NHWC layout changes, synthetic fill.
//
// They replace the reference's scalar grid-stride kernels (src/ios/ops.cu:6-48), its cudnnAddTensor
// loop for terms of six or more values (src/ios/ios_runtime.cu:746-751), cudnnPoolingForward
// (:565), cudnnActivationForward (:427) and cudnnOpTensor (:479).  Every kernel moves four elements
// per thread per access when the channel window allows it (16 bytes of float32, 8 of bfloat16),
// with consecutive threads on consecutive channels of one pixel (NHWC), so a warp touches one
// contiguous span.  Arithmetic is float32 whatever the storage type.
#include "kernels.h"

#include <cuda_bf16.h>

#include <cfloat>

namespace ios {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// sigmoid / tanh are rare; keeping them out of line keeps the hot loops short
__device__ __noinline__ float act_slow(float v, int act) {
    return act == 2 ? 1.0f / (1.0f + __expf(-v)) : tanhf(v);
}
__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == 1) return fmaxf(v, 0.0f);
    if (act == 0) return v;
    return act_slow(v, act);
}

// ---- element access: one or four consecutive elements as float ----------------------------
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
// store the first `count` (1..4) of four values
template <typename T>
__device__ __forceinline__ void store_some(T *p, float4 v, int count) {
    const float a[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (j < count) store1(p + j, a[j]);
}
__device__ __forceinline__ void store4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t *>(&lo);
    raw.y = *reinterpret_cast<const uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(p) = raw;
}

inline int grid_for(long work, int threads, int max_blocks = 148 * 32) {
    long blocks = (work + threads - 1) / threads;
    if (blocks < 1) blocks = 1;
    if (blocks > max_blocks) blocks = max_blocks;
    return static_cast<int>(blocks);
}

// ---------------------------------------------------------------------------------------------
template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads) sum_act_kernel(const SumActParams p) {
    const int lanes = kVec ? (p.C + 3) / 4 : p.C;      // work items per pixel
    const long total = p.pixels * lanes;
    T *out = static_cast<T *>(p.out);
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        const long pix = i / lanes;
        const int c = static_cast<int>(i - pix * lanes);
        if (kVec) {
            float4 acc = load4(static_cast<const T *>(p.in[0]) + pix * p.in_pitch[0] + 4 * c);
#pragma unroll
            for (int j = 1; j < kMaxSumInputs; ++j) {
                if (j < p.k) {
                    const float4 v = load4(static_cast<const T *>(p.in[j]) + pix * p.in_pitch[j] + 4 * c);
                    if (p.mul) {
                        acc.x *= v.x; acc.y *= v.y; acc.z *= v.z; acc.w *= v.w;
                    } else {
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                }
            }
            acc.x = apply_act(acc.x, p.act);
            acc.y = apply_act(acc.y, p.act);
            acc.z = apply_act(acc.z, p.act);
            acc.w = apply_act(acc.w, p.act);
            if (p.round_out) {
                acc.x = to_tf32(acc.x); acc.y = to_tf32(acc.y); acc.z = to_tf32(acc.z); acc.w = to_tf32(acc.w);
            }
            if (4 * c + 4 <= p.C) store4(out + pix * p.out_pitch + 4 * c, acc);
            else store_some(out + pix * p.out_pitch + 4 * c, acc, p.C - 4 * c);
        } else {
            float acc = load1(static_cast<const T *>(p.in[0]) + pix * p.in_pitch[0] + c);
#pragma unroll
            for (int j = 1; j < kMaxSumInputs; ++j) {
                if (j < p.k) {
                    const float v = load1(static_cast<const T *>(p.in[j]) + pix * p.in_pitch[j] + c);
                    acc = p.mul ? acc * v : acc + v;
                }
            }
            acc = apply_act(acc, p.act);
            store1(out + pix * p.out_pitch + c, p.round_out ? to_tf32(acc) : acc);
        }
    }
}

// ---------------------------------------------------------------------------------------------
template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads) pool_kernel(const PoolParams p) {
    const int lanes = kVec ? (p.in.C + 3) / 4 : p.in.C;
    const long total = p.out.pixels() * lanes;
    const float inv_window = 1.0f / float(p.kh * p.kw);   // padding counts (CUDNN_POOLING_AVERAGE_COUNT_INCLUDE_PADDING)
    const T *in = p.in.as<const T>();
    T *out = p.out.as<T>();
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        long pix = i / lanes;
        const int c = static_cast<int>(i - pix * lanes);
        const int ow = static_cast<int>(pix % p.out.W);
        pix /= p.out.W;
        const int oh = static_cast<int>(pix % p.out.H);
        const int n = static_cast<int>(pix / p.out.H);
        const int h0 = oh * p.sh - p.ph, w0 = ow * p.sw - p.pw;
        float4 acc = p.is_max ? make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX) : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < p.kh; ++r) {
            const int h = h0 + r;
            if (h < 0 || h >= p.in.H) continue;
            for (int s = 0; s < p.kw; ++s) {
                const int w = w0 + s;
                if (w < 0 || w >= p.in.W) continue;
                const T *src = in + ((long(n) * p.in.H + h) * p.in.W + w) * p.in.pitch;
                if (kVec) {
                    const float4 v = load4(src + 4 * c);
                    if (p.is_max) {
                        acc.x = fmaxf(acc.x, v.x); acc.y = fmaxf(acc.y, v.y);
                        acc.z = fmaxf(acc.z, v.z); acc.w = fmaxf(acc.w, v.w);
                    } else {
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                } else {
                    const float v = load1(src + c);
                    acc.x = p.is_max ? fmaxf(acc.x, v) : acc.x + v;
                }
            }
        }
        if (!p.is_max) {
            acc.x *= inv_window; acc.y *= inv_window; acc.z *= inv_window; acc.w *= inv_window;
        }
        if (p.round_out) {
            acc.x = to_tf32(acc.x); acc.y = to_tf32(acc.y); acc.z = to_tf32(acc.z); acc.w = to_tf32(acc.w);
        }
        T *dst = out + ((long(n) * p.out.H + oh) * p.out.W + ow) * p.out.pitch;
        if (!kVec) store1(dst + c, acc.x);
        else if (4 * c + 4 <= p.in.C) store4(dst + 4 * c, acc);
        else store_some(dst + 4 * c, acc, p.in.C - 4 * c);
    }
}

// One block per (image, 32-channel slab): 8 warps stride over the pixels, lanes over channels, so
// each warp reads one contiguous span per pixel; partial results meet in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) global_pool_kernel(const PoolParams p) {
    __shared__ float part[8][33];
    const int slabs = (p.in.C + 31) / 32;
    const int n = blockIdx.x / slabs;
    const int c = (blockIdx.x % slabs) * 32 + (threadIdx.x & 31);
    const int warp = threadIdx.x >> 5;
    const int hw = p.in.H * p.in.W;
    float acc = p.is_max ? -FLT_MAX : 0.0f;
    if (c < p.in.C) {
        const T *src = p.in.as<const T>() + long(n) * hw * p.in.pitch + c;
        for (int i = warp; i < hw; i += 8) {
            const float v = load1(src + long(i) * p.in.pitch);
            acc = p.is_max ? fmaxf(acc, v) : acc + v;
        }
    }
    part[warp][threadIdx.x & 31] = acc;
    __syncthreads();
    if (warp == 0 && c < p.in.C) {
        float total = part[0][threadIdx.x];
        for (int w = 1; w < 8; ++w) total = p.is_max ? fmaxf(total, part[w][threadIdx.x]) : total + part[w][threadIdx.x];
        if (!p.is_max) total *= 1.0f / float(hw);
        store1(p.out.as<T>() + long(n) * p.out.pitch + c, p.round_out ? to_tf32(total) : total);
    }
}

// ---------------------------------------------------------------------------------------------
// Layout changes go through a 32x33 shared tile so that both the global read and the global write
// run along the respective fastest axis.  The NCHW side is always float32 (the API boundary).
template <typename T>
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const float *__restrict__ src, TensorRef dst, int round_out) {
    __shared__ float tile[32][33];
    const int hw = dst.H * dst.W;
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 32; j += 8) {
        const int c = c0 + j, px = p0 + tx;
        tile[j][tx] = (c < dst.C && px < hw) ? src[(long(n) * dst.C + c) * hw + px] : 0.0f;
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int px = p0 + j, c = c0 + tx;
        if (px < hw && c < dst.C)
            store1(dst.as<T>() + (long(n) * hw + px) * dst.pitch + c, round_out ? to_tf32(tile[tx][j]) : tile[tx][j]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) nhwc_to_nchw_kernel(TensorRef src, float *__restrict__ dst) {
    __shared__ float tile[32][33];
    const int hw = src.H * src.W;
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 32; j += 8) {
        const int px = p0 + j, c = c0 + tx;
        tile[j][tx] = (px < hw && c < src.C) ? load1(src.as<const T>() + (long(n) * hw + px) * src.pitch + c) : 0.0f;
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int c = c0 + j, px = p0 + tx;
        if (c < src.C && px < hw) dst[(long(n) * src.C + c) * hw + px] = tile[tx][j];
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) fill_kernel(T *dst, long count, uint32_t seed, float scale) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < count; i += long(gridDim.x) * blockDim.x) {
        uint32_t x = static_cast<uint32_t>(i) * 2654435761u + seed;
        x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
        store1(dst + i, (float(x >> 8) * (1.0f / 8388608.0f) - 1.0f) * scale);
    }
}

}  // namespace

void launch_sum_act(const SumActParams &p, bool vec4, cudaStream_t stream) {
    if (p.pixels <= 0 || p.C <= 0) return;
    const int grid = grid_for(p.pixels * (vec4 ? (p.C + 3) / 4 : p.C), kThreads);
    if (p.esize == 2) {
        if (vec4) sum_act_kernel<__nv_bfloat16, true><<<grid, kThreads, 0, stream>>>(p);
        else sum_act_kernel<__nv_bfloat16, false><<<grid, kThreads, 0, stream>>>(p);
    } else {
        if (vec4) sum_act_kernel<float, true><<<grid, kThreads, 0, stream>>>(p);
        else sum_act_kernel<float, false><<<grid, kThreads, 0, stream>>>(p);
    }
}

void launch_pool(const PoolParams &p, cudaStream_t stream) {
    const bool bf16 = p.in.esize == 2;
    const bool global = p.out.H == 1 && p.out.W == 1 && p.kh == p.in.H && p.kw == p.in.W && p.ph == 0 && p.pw == 0;
    if (global) {
        const int slabs = (p.in.C + 31) / 32;
        if (bf16) global_pool_kernel<__nv_bfloat16><<<p.in.N * slabs, 256, 0, stream>>>(p);
        else global_pool_kernel<float><<<p.in.N * slabs, 256, 0, stream>>>(p);
        return;
    }
    const bool vec = p.in.vec4() && p.out.vec4();
    const int grid = grid_for(p.out.pixels() * (vec ? (p.in.C + 3) / 4 : p.in.C), kThreads);
    if (bf16) {
        if (vec) pool_kernel<__nv_bfloat16, true><<<grid, kThreads, 0, stream>>>(p);
        else pool_kernel<__nv_bfloat16, false><<<grid, kThreads, 0, stream>>>(p);
    } else {
        if (vec) pool_kernel<float, true><<<grid, kThreads, 0, stream>>>(p);
        else pool_kernel<float, false><<<grid, kThreads, 0, stream>>>(p);
    }
}

void launch_nchw_to_nhwc(const float *src, TensorRef dst, bool round_tf32, cudaStream_t stream) {
    const int hw = dst.H * dst.W;
    dim3 grid((hw + 31) / 32, (dst.C + 31) / 32, dst.N);
    if (dst.esize == 2) nchw_to_nhwc_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(src, dst, 0);
    else nchw_to_nhwc_kernel<float><<<grid, 256, 0, stream>>>(src, dst, round_tf32 ? 1 : 0);
}

void launch_nhwc_to_nchw(TensorRef src, float *dst, cudaStream_t stream) {
    const int hw = src.H * src.W;
    dim3 grid((hw + 31) / 32, (src.C + 31) / 32, src.N);
    if (src.esize == 2) nhwc_to_nchw_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(src, dst);
    else nhwc_to_nchw_kernel<float><<<grid, 256, 0, stream>>>(src, dst);
}

void launch_fill(void *dst, long count, uint32_t seed, float scale, cudaStream_t stream, int esize) {
    if (count <= 0) return;
    if (esize == 2) fill_kernel<<<grid_for(count, kThreads), kThreads, 0, stream>>>(static_cast<__nv_bfloat16 *>(dst), count, seed, scale);
    else fill_kernel<<<grid_for(count, kThreads), kThreads, 0, stream>>>(static_cast<float *>(dst), count, seed, scale);
}

}  // namespace ios
