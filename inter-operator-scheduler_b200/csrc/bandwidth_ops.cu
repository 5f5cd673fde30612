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
    grid_dependency_entry();
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
    grid_dependency_entry();
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

// ---- 3x3 windows: a thread walks down a column of output pixels ------------------------------
// V consecutive channels as float: one 16-byte access of float32 (V = 4) or bfloat16 (V = 8), or 8 bytes of bfloat16 (V = 4).
template <typename T, int V> struct VecIo;
template <> struct VecIo<float, 4> {
    typedef float4 Raw;
    static __device__ __forceinline__ void unpack(const Raw &x, float (&v)[4]) { v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; }
    static __device__ __forceinline__ void load(const float *p, float (&v)[4]) {
        const float4 x = *reinterpret_cast<const float4 *>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float *p, const float (&v)[4]) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct VecIo<__nv_bfloat16, 4> {
    typedef uint2 Raw;
    static __device__ __forceinline__ void unpack(const Raw &raw, float (&v)[4]) {
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
        v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[4]) {
        const float4 x = load4(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&v)[4]) { store4(p, make_float4(v[0], v[1], v[2], v[3])); }
};
template <> struct VecIo<__nv_bfloat16, 8> {
    typedef uint4 Raw;
    static __device__ __forceinline__ void unpack(const Raw &raw, float (&v)[8]) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[j]));
            v[2 * j] = f.x; v[2 * j + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[j]));
            v[2 * j] = f.x; v[2 * j + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// A thread owns V channels of one output column and walks `rows_per_thread` output rows down it.  It
// reads every input row of its span once: the three pixels of the window's width (the pixels its
// neighbours in the warp read at the same moment, so two of three come from L1) are reduced to one
// value per row, the last three rows' values sit in registers, and an output row is emitted whenever
// the window is complete -- 3 loads per output for a stride-1 window instead of 9, 6 for stride 2.
// Rows are fetched two at a time, and the next pair is requested before the current one is reduced (6 to 12
// independent 16-byte loads in flight per thread at any time): a thread's rows depend on one another only
// through registers, and with two blocks of 256 threads per SM it is the bytes in flight that feed the memory.
// Average pooling divides by 9 whatever the padding (CUDNN_POOLING_AVERAGE_COUNT_INCLUDE_PADDING,
// the reference's mode, src/ios/ios_runtime.cu:546-553).
template <typename T, int V, bool kMax>
__global__ void __launch_bounds__(kThreads) pool3x3_kernel(const PoolParams p, int rows_per_thread) {
    grid_dependency_entry();
    typedef typename VecIo<T, V>::Raw Raw;
    constexpr int kRows = 4;
    // grid: x covers (output column, channel group), y the row segments, z the images -- no 64-bit index arithmetic
    const int groups = (p.in.C + V - 1) / V;
    const int idx = blockIdx.x * kThreads + threadIdx.x;
    if (idx >= p.out.W * groups) return;
    const int ow = idx / groups;
    const int c = (idx - ow * groups) * V;
    const int n = blockIdx.z;
    const int oh_begin = blockIdx.y * rows_per_thread, oh_end = min(p.out.H, oh_begin + rows_per_thread);
    const float identity = kMax ? -FLT_MAX : 0.0f;
    const int w0 = ow * p.sw - p.pw;
    const bool w_ok[3] = {w0 >= 0 && w0 < p.in.W, w0 + 1 >= 0 && w0 + 1 < p.in.W, w0 + 2 >= 0 && w0 + 2 < p.in.W};
    const size_t row_pitch = size_t(p.in.W) * p.in.pitch;
    const T *image = p.in.as<const T>() + size_t(n) * p.in.H * row_pitch + size_t(max(w0, 0)) * p.in.pitch + c;
    const int first = w0 < 0 ? -w0 : 0;          // window column that `image` points at
    T *dst = p.out.as<T>() + ((size_t(n) * p.out.H + oh_begin) * p.out.W + ow) * p.out.pitch + c;
    const size_t dst_step = size_t(p.out.W) * p.out.pitch;
    const bool whole = c + V <= p.in.C;

    const int h_first = oh_begin * p.sh - p.ph, h_last = (oh_end - 1) * p.sh - p.ph + 2;
    int next_emit = h_first + 2;                 // the input row that completes the next output row
    float r1[V], r2[V];
#pragma unroll
    for (int j = 0; j < V; ++j) r1[j] = r2[j] = identity;
    // Two rows per request, two requests in flight: while one pair of rows is reduced, the next pair is on its way.
    constexpr int kPair = kRows / 2;
    auto fetch = [&](Raw (&raw)[kPair][3], int hb) {
#pragma unroll
        for (int r = 0; r < kPair; ++r) {
            const int h = hb + r;
            const bool row_ok = h >= 0 && h < p.in.H && h <= h_last;
            const T *src = image + size_t(max(h, 0)) * row_pitch;
#pragma unroll
            for (int s = 0; s < 3; ++s)
                if (row_ok && w_ok[s]) raw[r][s] = *reinterpret_cast<const Raw *>(src + (s - first) * p.in.pitch);
        }
    };
    auto reduce = [&](const Raw (&raw)[kPair][3], int hb) {
#pragma unroll
        for (int r = 0; r < kPair; ++r) {
            const int h = hb + r;
            if (h > h_last) break;
            const bool row_ok = h >= 0 && h < p.in.H;
            float acc[V];
#pragma unroll
            for (int j = 0; j < V; ++j) acc[j] = identity;
#pragma unroll
            for (int s = 0; s < 3; ++s) {
                if (!(row_ok && w_ok[s])) continue;
                float v[V];
                VecIo<T, V>::unpack(raw[r][s], v);
#pragma unroll
                for (int j = 0; j < V; ++j) acc[j] = kMax ? fmaxf(acc[j], v[j]) : acc[j] + v[j];
            }
            if (h == next_emit) {
                float o[V];
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const float z = kMax ? fmaxf(fmaxf(r1[j], r2[j]), acc[j]) : (r1[j] + r2[j] + acc[j]) * (1.0f / 9.0f);
                    o[j] = p.round_out ? to_tf32(z) : z;
                }
                if (whole) {
                    VecIo<T, V>::store(dst, o);
                } else {
#pragma unroll
                    for (int j = 0; j < V; ++j)
                        if (c + j < p.in.C) store1(dst + j, o[j]);
                }
                dst += dst_step;
                next_emit += p.sh;
            }
#pragma unroll
            for (int j = 0; j < V; ++j) { r1[j] = r2[j]; r2[j] = acc[j]; }
        }
    };
    Raw even[kPair][3], odd[kPair][3];
    fetch(even, h_first);
    for (int hb = h_first; hb <= h_last; hb += kRows) {
        fetch(odd, hb + kPair);
        reduce(even, hb);
        fetch(even, hb + kRows);
        reduce(odd, hb + kPair);
    }
}

template <typename T, int V>
void launch_pool3x3(const PoolParams &p, cudaStream_t stream) {
    const int groups = (p.in.C + V - 1) / V;
    // long columns reuse the most rows; short ones give a small batch enough threads to fill the GPU
    int rows = p.out.H;
    auto threads_for = [&](int r) { return long(p.out.N) * ((p.out.H + r - 1) / r) * p.out.W * groups; };
    while (rows > 4 && threads_for(rows) < 148L * 1024) rows = (rows + 1) / 2;
    const int segments = (p.out.H + rows - 1) / rows;
    const dim3 grid((p.out.W * groups + kThreads - 1) / kThreads, segments, p.out.N);
    if (p.is_max) pool3x3_kernel<T, V, true><<<grid, kThreads, 0, stream>>>(p, rows);
    else pool3x3_kernel<T, V, false><<<grid, kThreads, 0, stream>>>(p, rows);
}

// One block per (image, 32-channel slab): 8 warps stride over the pixels, lanes over channels, so
// each warp reads one contiguous span per pixel; partial results meet in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) global_pool_kernel(const PoolParams p) {
    grid_dependency_entry();
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
    grid_dependency_entry();
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

// At most four channels (a network's input image): a 32-channel tile would be nine tenths idle.  One thread per
// pixel reads its channels from the planes -- consecutive threads read consecutive addresses of each plane -- and
// writes them as one 4-element group (16 bytes of float32, 8 of bfloat16); lanes beyond C are written as zeros.
template <typename T>
__global__ void __launch_bounds__(256) nchw_to_nhwc_few_kernel(const float *__restrict__ src, TensorRef dst, int round_out) {
    grid_dependency_entry();
    const long hw = long(dst.H) * dst.W;
    const long total = hw * dst.N;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        const long n = i / hw, px = i - n * hw;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (c < dst.C) {
                const float x = src[(n * dst.C + c) * hw + px];
                v[c] = round_out ? to_tf32(x) : x;
            }
        store4(dst.as<T>() + i * dst.pitch, make_float4(v[0], v[1], v[2], v[3]));
    }
}

template <typename T>
__global__ void __launch_bounds__(256) nhwc_to_nchw_kernel(TensorRef src, float *__restrict__ dst) {
    grid_dependency_entry();
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
    if (vec && p.kh == 3 && p.kw == 3 && p.out.N <= 65535) {
        const bool wide = bf16 && p.in.pitch % 8 == 0 && p.out.pitch % 8 == 0 &&
                          (reinterpret_cast<uintptr_t>(p.in.ptr) | reinterpret_cast<uintptr_t>(p.out.ptr)) % 16 == 0;
        if (!bf16) launch_pool3x3<float, 4>(p, stream);
        else if (wide) launch_pool3x3<__nv_bfloat16, 8>(p, stream);
        else launch_pool3x3<__nv_bfloat16, 4>(p, stream);
        return;
    }
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
    if (dst.C <= 4 && dst.vec4()) {
        const int blocks = grid_for(long(hw) * dst.N, 256);
        if (dst.esize == 2) nchw_to_nhwc_few_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(src, dst, 0);
        else nchw_to_nhwc_few_kernel<float><<<blocks, 256, 0, stream>>>(src, dst, round_tf32 ? 1 : 0);
        return;
    }
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
