// Device-side building blocks shared by the tensor-core convolution kernels (sm_100a): mbarrier, TMA,
// tensor-memory and tcgen05.mma wrappers, the shared-memory operand descriptor, activation and store
// helpers.  Everything here is inline; the file is included by the translation units that hold kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace ios {
namespace {

constexpr int kTileM = 128;          // TMEM lanes = pixel rows per CTA
constexpr int kRowBytes = 128;       // K bytes per pipeline step = one 128-byte swizzle row (32 floats or 64 bf16)
constexpr int kChunk = 32;           // float32 elements per row
constexpr int kATileBytes = kTileM * kRowBytes;    // 16 KiB
constexpr int kThreads = 352;          // producer warp, MMA issuer, four epilogue warps; three-pass mode: second MMA issuer, four residual warps
constexpr uint64_t kWaitBudgetNs = 2000000000ull;  // 2 s per wait

// ---- PTX wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false when the budget ran out, or when another CTA of the grid has already
// reported a wait that ran out (so that one stuck tile does not cost the budget once per CTA).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const int *error_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 0) {
            if (global_ns() - t0 > kWaitBudgetNs) return false;
            if (error_flag && *reinterpret_cast<const volatile int *>(error_flag) != 0) return false;
        }
    }
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void *tmap, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// im2col mode: the box is `pixels per column` consecutive positions of the filter window's corner,
// walked along w, then h, then n inside the bounding box of the tensor map, starting at (w, h, n);
// (off_w, off_h) selects the filter tap.  Positions outside the image read zeros (the padding).
__device__ __forceinline__ void tma_load_im2col(uint32_t dst, const void *tmap, uint32_t bar, int c, int w, int h, int n,
                                                uint32_t off_w, uint32_t off_h) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(uint16_t(off_w)), "h"(uint16_t(off_h))
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void *tmap, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(tmap), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
// (relaxed: orders nothing by itself; barrier initialisation is published by fence.mbarrier_init before it)
__device__ __forceinline__ void cluster_arrive_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of `addr` (a shared-memory address of this CTA) in the CTA of rank `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// 16 bytes into another CTA's shared memory; the bytes are counted on that CTA's barrier `bar` when they land.
__device__ __forceinline__ void cluster_push16(uint32_t dst, uint32_t bar, float a, float b, float c, float d) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(dst), "f"(a), "f"(b), "f"(c), "f"(d), "r"(bar)
                 : "memory");
}
// Bounded wait on a barrier whose bytes come from other CTAs of the cluster.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, const int *error_flag) {
    const uint64_t t0 = global_ns();
    for (uint32_t spin = 1;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 1023u) == 0) {
            if (global_ns() - t0 > kWaitBudgetNs) return false;
            if (error_flag && *reinterpret_cast<const volatile int *>(error_flag) != 0) return false;
        }
    }
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// two 16-column loads in flight, one wait
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float *v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// Accumulator columns [c, c + N) of this thread's lane; in three-pass mode the products with the weight
// residual accumulate in a second column range `pair` columns further on and are added here.
// (`third`: a further range at that offset, where the products with the activation residual have an accumulator
// of their own because a second thread issues them)
__device__ __forceinline__ void acc_ld32(uint32_t taddr, uint32_t pair, float *v, uint32_t third = 0) {
    tmem_ld32(taddr, v);
    if (pair) {
        float w[32];
        tmem_ld32(taddr + pair, w);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += w[i];
    }
    if (third) {
        float w[32];
        tmem_ld32(taddr + third, w);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += w[i];
    }
}
// The same with both column ranges requested before either is waited for.
__device__ __forceinline__ void acc_ld32_pair(uint32_t taddr, uint32_t pair, float *v, uint32_t third = 0) {
    if (!pair) {
        tmem_ld32(taddr, v);
        return;
    }
    if (third) {
        // three ranges: all requested before any is waited for; added in a fixed order
        uint32_t r[32], w[32], x[32];
#define IOS_LD32(dst, addr)                                                                                              \
        asm volatile(                                                                                                    \
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, " \
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                 \
            : "=r"(dst[0]), "=r"(dst[1]), "=r"(dst[2]), "=r"(dst[3]), "=r"(dst[4]), "=r"(dst[5]), "=r"(dst[6]), "=r"(dst[7]), \
              "=r"(dst[8]), "=r"(dst[9]), "=r"(dst[10]), "=r"(dst[11]), "=r"(dst[12]), "=r"(dst[13]), "=r"(dst[14]), "=r"(dst[15]), \
              "=r"(dst[16]), "=r"(dst[17]), "=r"(dst[18]), "=r"(dst[19]), "=r"(dst[20]), "=r"(dst[21]), "=r"(dst[22]), "=r"(dst[23]), \
              "=r"(dst[24]), "=r"(dst[25]), "=r"(dst[26]), "=r"(dst[27]), "=r"(dst[28]), "=r"(dst[29]), "=r"(dst[30]), "=r"(dst[31]) \
            : "r"(addr))
        IOS_LD32(r, taddr);
        IOS_LD32(w, taddr + pair);
        IOS_LD32(x, taddr + third);
#undef IOS_LD32
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = (__uint_as_float(r[i]) + __uint_as_float(w[i])) + __uint_as_float(x[i]);
        return;
    }
    uint32_t r[32], w[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]),
          "=r"(w[8]), "=r"(w[9]), "=r"(w[10]), "=r"(w[11]), "=r"(w[12]), "=r"(w[13]), "=r"(w[14]), "=r"(w[15]),
          "=r"(w[16]), "=r"(w[17]), "=r"(w[18]), "=r"(w[19]), "=r"(w[20]), "=r"(w[21]), "=r"(w[22]), "=r"(w[23]),
          "=r"(w[24]), "=r"(w[25]), "=r"(w[26]), "=r"(w[27]), "=r"(w[28]), "=r"(w[29]), "=r"(w[30]), "=r"(w[31])
        : "r"(taddr + pair));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) + __uint_as_float(w[i]);
}
__device__ __forceinline__ void acc_ld16(uint32_t taddr, uint32_t pair, float *v, uint32_t third = 0) {
    tmem_ld16(taddr, v);
    if (pair) {
        float w[16];
        tmem_ld16(taddr + pair, w);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += w[i];
    }
    if (third) {
        float w[16];
        tmem_ld16(taddr + third, w);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += w[i];
    }
}
// K-major operand tile with 128-byte swizzle: rows are 128 bytes, groups of 8 rows are 1024 bytes apart.
// (row_bytes 64: the same with the 64-byte swizzle, rows are 64 bytes and groups of 8 rows 512 bytes apart)
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t addr, int row_bytes) {
    uint64_t d = 0;
    d |= uint64_t((addr & 0x3FFFF) >> 4);    // start address, 16-byte units
    d |= uint64_t(1) << 16;                  // leading-dimension byte offset (unused for swizzled K-major)
    d |= uint64_t((8 * row_bytes) >> 4) << 32;   // stride-dimension byte offset: 8 rows
    d |= uint64_t(1) << 46;                  // descriptor version for sm_100
    d |= uint64_t(row_bytes == 128 ? 2 : 4) << 61;   // SWIZZLE_128B / SWIZZLE_64B
    return d;
}
// sigmoid / tanh are rare; keeping them out of line keeps the unrolled epilogue small
__device__ __noinline__ float act_slow(float v, int act) {
    return act == 2 ? 1.0f / (1.0f + __expf(-v)) : tanhf(v);
}
__device__ __forceinline__ float act_apply(float v, int act) {
    if (act == 1) return fmaxf(v, 0.0f);
    if (act == 0) return v;
    return act_slow(v, act);
}
__device__ __forceinline__ float round_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// Byte offset of 16-byte column `c4` of row `row` inside a [rows][128 B] tile with the 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128_offset(int row, int c4) {
    return uint32_t(row) * 128u + (uint32_t(c4 ^ (row & 7)) << 4);
}

// Stage four finished values (tile channels cc..cc+3 of `row`) for the bulk store: the staging area
// is [slab][row][128 B] with the TMA swizzle, a slab being 32 float32 or 64 bfloat16 channels.
__device__ __forceinline__ void stage4(uint8_t *staging, int row, int cc, float4 o, int bf16) {
    if (!bf16) {
        *reinterpret_cast<float4 *>(staging + size_t(cc >> 5) * kATileBytes + sw128_offset(row, (cc & 31) >> 2)) = o;
    } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t *>(&lo);
        raw.y = *reinterpret_cast<const uint32_t *>(&hi);
        *reinterpret_cast<uint2 *>(staging + size_t(cc >> 6) * kATileBytes + sw128_offset(row, (cc & 63) >> 3) + ((cc & 7) << 1)) = raw;
    }
}
// Store up to four finished values straight to the output window at element offset `at`.  The whole,
// aligned group is the common case; everything else goes element by element, out of line.
__device__ __noinline__ void store_some_direct(void *out, int bf16, long at, float4 o, int count) {
    const float v[4] = {o.x, o.y, o.z, o.w};
    if (!bf16) {
        float *dst = static_cast<float *>(out) + at;
        for (int j = 0; j < 4; ++j)
            if (j < count) dst[j] = v[j];
    } else {
        __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(out) + at;
        for (int j = 0; j < 4; ++j)
            if (j < count) dst[j] = __float2bfloat16_rn(v[j]);
    }
}
__device__ __forceinline__ void store4_direct(void *out, int bf16, long at, float4 o, int count) {
    if (!bf16) {
        float *dst = static_cast<float *>(out) + at;
        if (count >= 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) *reinterpret_cast<float4 *>(dst) = o;
        else store_some_direct(out, bf16, at, o, count);
    } else {
        __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(out) + at;
        if (count >= 4 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
            uint2 raw;
            raw.x = *reinterpret_cast<const uint32_t *>(&lo);
            raw.y = *reinterpret_cast<const uint32_t *>(&hi);
            *reinterpret_cast<uint2 *>(dst) = raw;
        } else {
            store_some_direct(out, bf16, at, o, count);
        }
    }
}
// Store eight finished values (bfloat16: one 16-byte access when the address allows) at element offset `at`.
__device__ __forceinline__ void store8_direct(void *out, int bf16, long at, const float *v, int count) {
    if (bf16) {
        __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(out) + at;
        if (count >= 8 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            uint4 raw;
            const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
            const __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
            raw.x = *reinterpret_cast<const uint32_t *>(&a);
            raw.y = *reinterpret_cast<const uint32_t *>(&b);
            raw.z = *reinterpret_cast<const uint32_t *>(&c);
            raw.w = *reinterpret_cast<const uint32_t *>(&d);
            *reinterpret_cast<uint4 *>(dst) = raw;
            return;
        }
    }
    store4_direct(out, bf16, at, make_float4(v[0], v[1], v[2], v[3]), count);
    if (count > 4) store4_direct(out, bf16, at + 4, make_float4(v[4], v[5], v[6], v[7]), count - 4);
}

}  // namespace
}  // namespace ios
