// Stride-1 convolutions with a window (3x3, 5x5, 1x7, 7x1 ...) on the tensor cores, every input pixel
// fetched ONCE per tile instead of once per filter tap.
//
// The implicit-GEMM kernel of conv_tc.cu loads, for each of the kh*kw taps, a fresh 128-pixel activation
// tile through the TMA unit; on B200 that unit, not the tensor pipe, bounds such layers (about 1.2
// cycles per 128-byte row plus 1 cycle per 100 bytes, measured).  Here a tile's input PATCH -- ph x pw
// pixels per image, the tile's outputs plus the window's halo -- lands in shared memory once per channel
// chunk as rows in (image, row, column) order, and GEMM row m is the output pixel
//     m = (image * ph + y) * pw + x,
// so that tap (r, s) of EVERY output pixel of the tile is patch row m + r*pw + s: the A operand of tap
// (r, s) is the same shared-memory tile read from a start address (r*pw + s) rows further on.  (The
// 128-byte swizzle is a function of the shared-memory address, so an operand may start at any row.)
// Rows whose x >= box_w or y >= box_h are halo positions: their accumulators are garbage and are simply
// not stored.  Padding is the zero fill of the TMA unit for coordinates outside the image.
//
// A tile therefore costs ph*pw rows of activations (instead of taps*128) plus taps*bn rows of weights per
// channel chunk; when the whole packed weight matrix is small (the first layers of a network) it is
// loaded once per CTA and stays resident.  In three-pass TF32 mode the residual of the activations is
// computed once per patch instead of once per tap.
//
// Persistent CTAs (one or two per SM) walk the tiles; warp 0 lane 0 loads patches, lane 1 weight tiles,
// the other warps finish the previous tile (bias, activation, stores of the valid rows) while up to four
// ISSUER warps (warp 1 and warps 10..12) feed the tensor pipe: one thread gets a tcgen05.mma out about
// every 140 cycles (measured: whatever its shape), the pipe takes one of N <= 128 every 60, so the taps
// of a tile are dealt round-robin to the issuers.  Every issuer has an accumulator of its own in tensor
// memory and the epilogue adds them in a fixed order: instructions of different warps are not ordered
// among themselves, so a shared accumulator would make the result depend on timing in its last bits.
// Two sets of accumulators alternate between tiles.  Every wait is bounded.
//
// Replaces cudnnConvolutionBiasActivationForward (reference src/ios/ios_runtime.cu:313-331) for these shapes.
#include "kernels.h"
#include "tc_device.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace ios {
namespace {

constexpr int kPatchThreads = 416;       // 13 warps: producers, issuer, 8 epilogue / split warps, 3 more issuers
constexpr int kMaxIssuers = 4;

struct PatchGeom {
    int bn, cchunks, taps, kw, chunk;
    int pw, ph;                       // patch extent per image, input pixels
    int box_w, box_h, box_n;          // valid output extent of a tile
    int tiles_w, tiles_h, n_tiles, total_tiles;
    int a_rows;                       // rows of one plane of an activation stage (multiple of 8)
    int a_stages, b_stages;
    int a_tx_bytes;                   // bytes one patch load delivers
    int b_resident;                   // 1: every weight tile is loaded once and kept (b_stages = taps * cchunks)
    int tmem_cols, acc_stride;
    int wide, round_tf32, cout_pad;
    int pad_w, pad_h;
    int issuers;                      // warps that issue tcgen05.mma: tap i of every chunk belongs to issuer i % issuers
    int tma_store;                    // 1: finished tiles leave through bulk tensor stores, one per output row segment
    int slab;                         // output channels per 128-byte staging row: 32 (float32) or 64 (bfloat16)
    int b_depth;                      // weight stages per issuer: issuer w owns stages [w * b_depth, (w + 1) * b_depth), so that
                                      // every stage has ONE consumer, which sees each of its phases (b_stages = issuers * b_depth)
};

template <int MODE>      // 0: TF32, 1: three-pass TF32, 2: BF16, 4: BF16 with 64-byte operand rows (at most 32 input channels)
__global__ void __launch_bounds__(kPatchThreads, 2)
conv_tc_patch_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_c, const ConvTcParams p, const PatchGeom t) {
    constexpr bool kX3 = MODE == 1, kBf16 = MODE == 2 || MODE == 4;
    constexpr int kRow = MODE == 4 ? 64 : 128;           // bytes of K per operand row; 32 bytes of it per instruction
    extern __shared__ uint8_t smem_raw[];
    __shared__ float bias_s[2][256];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const int planes = kX3 ? 2 : 1;
    const int a_plane = t.a_rows * kRow;
    const int a_stage_bytes = planes * a_plane;
    const int b_bytes = t.bn * kRow;
    const int b_stage_bytes = planes * b_bytes;
    const uint32_t a0 = smem_base;
    const uint32_t b0 = a0 + uint32_t(t.a_stages) * a_stage_bytes;
    // store staging: [slab][128 rows][128 B], swizzled like a TMA box; pw is a multiple of 8, so that every output row
    // segment of a tile starts on a 1024-byte boundary of it
    const int slabs = (t.bn + t.slab - 1) / t.slab;
    const uint32_t staging0 = b0 + uint32_t(t.b_stages) * b_stage_bytes;
    const uint32_t bars = staging0 + (t.tma_store ? uint32_t(slabs) * kATileBytes : 0u);
    const uint32_t a_full0 = bars, a_empty0 = a_full0 + 8u * t.a_stages, a_ready0 = a_empty0 + 8u * t.a_stages;
    const uint32_t b_full0 = a_ready0 + 8u * t.a_stages, b_empty0 = b_full0 + 8u * t.b_stages;
    const uint32_t acc_full0 = b_empty0 + 8u * t.b_stages, acc_empty0 = acc_full0 + 16u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(generic_base + (acc_empty0 + 16u - smem_base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const ConvGeom &g = p.g;
    const int epi_warps = kX3 ? 4 : 8;
    const int my_tiles = (t.total_tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);

    if (warp == 0) {
        for (int i = lane; i < t.a_stages; i += 32) {
            mbar_init(a_full0 + 8u * i, 1);
            mbar_init(a_empty0 + 8u * i, uint32_t(t.issuers));
            mbar_init(a_ready0 + 8u * i, 128);
        }
        for (int i = lane; i < t.b_stages; i += 32) {
            mbar_init(b_full0 + 8u * i, 1);
            mbar_init(b_empty0 + 8u * i, 1);
        }
        if (lane < 2) {
            mbar_init(acc_full0 + 8u * lane, uint32_t(t.issuers));
            mbar_init(acc_empty0 + 8u * lane, uint32_t(epi_warps));
        }
        if (lane == 31) {
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
    const int issuer = warp == 1 ? 0 : warp - 9;          // warps 10, 11, 12 are issuers 1, 2, 3
    if ((warp == 0 && lane >= 1 + t.issuers) || ((warp == 1 || warp >= 10) && (lane != 0 || issuer >= t.issuers))) return;

    // where a role gave up (read back by the host beside the time-out word): word 1 + role = tile | chunk << 12 | tap << 18 | wait << 26
    auto gave_up = [&](int role, int ti, int cc, int tap, int wait) {
        p.error_flag[1 + role] = (ti & 0xFFF) | ((cc & 63) << 12) | ((tap & 255) << 18) | (wait << 26);
    };
    // tile -> coordinates: output-channel tile fastest, then tiles along w, h, n
    auto decode = [&](int tile, int &cout0, int &ow0, int &oh0, int &n0) {
        const int m_tile = tile / t.n_tiles;
        cout0 = (tile - m_tile * t.n_tiles) * t.bn;
        const int tw = m_tile % t.tiles_w;
        const int rest = m_tile / t.tiles_w;
        ow0 = tw * t.box_w;
        oh0 = (rest % t.tiles_h) * t.box_h;
        n0 = (rest / t.tiles_h) * t.box_n;
    };

    if (warp == 0 && lane == 0) {
        // ---------------- activation patches: one load per (tile, channel chunk) ----------------
        asm volatile("griddepcontrol.wait;" ::: "memory");
        int s = 0, phase = 1, issued = 0;
        bool ok = true;
#pragma unroll 1
        for (int ti = 0; ti < my_tiles && ok; ++ti) {
            int cout0, ow0, oh0, n0;
            decode(int(blockIdx.x) + ti * int(gridDim.x), cout0, ow0, oh0, n0);
#pragma unroll 1
            for (int cc = 0; cc < t.cchunks; ++cc) {
                ok = mbar_wait(a_empty0 + 8u * s, uint32_t(phase), p.error_flag);
                if (!ok) { gave_up(0, ti, cc, 0, 1); break; }
                const uint32_t bar = a_full0 + 8u * s;
                mbar_expect_tx(bar, uint32_t(t.a_tx_bytes));
                tma_load_4d(a0 + uint32_t(s) * a_stage_bytes, &tmap_a, bar, cc * t.chunk, ow0 - t.pad_w, oh0 - t.pad_h, n0);
                ++issued;
                if (++s == t.a_stages) { s = 0; phase ^= 1; }
            }
        }
        if (!ok) {
            atomicCAS(p.error_flag, 0, 11);
            // the loads already issued still land here: wait for the latest one of every stage
            for (int j = issued - 1, k = 0; j >= 0 && k < t.a_stages; --j, ++k)
                mbar_wait(a_full0 + 8u * (j % t.a_stages), uint32_t((j / t.a_stages) & 1), nullptr);
        }
        return;
    }
    if (warp == 0) {
        // ---------------- weight tiles: lane 1 + w loads the taps of issuer w (w, w + W, ... of every chunk) into that
        // issuer's ring -- or, when the weights stay resident, once into stage chunk * taps + tap.  One thread gets a load
        // out every few hundred cycles (wait, arm, issue), so every ring has a lane of its own.
        const int W = t.issuers, w = lane - 1;
        int s = 0, phase = 1, issued = 0;
        bool ok = true;
        const int rounds = t.b_resident ? 1 : my_tiles;
#pragma unroll 1
        for (int ti = 0; ti < rounds && ok; ++ti) {
            int cout0, ow0, oh0, n0;
            decode(int(blockIdx.x) + ti * int(gridDim.x), cout0, ow0, oh0, n0);
#pragma unroll 1
            for (int cc = 0; cc < t.cchunks && ok; ++cc) {
#pragma unroll 1
                for (int tap = w; tap < t.taps; tap += W) {
                    int slot;
                    if (t.b_resident) {
                        slot = cc * t.taps + tap;
                    } else {
                        slot = w * t.b_depth + s;
                        ok = mbar_wait(b_empty0 + 8u * slot, uint32_t(phase), p.error_flag);
                        if (!ok) { gave_up(1, ti, cc, tap, 2); break; }
                        if (++s == t.b_depth) { s = 0; phase ^= 1; }
                    }
                    const uint32_t bar = b_full0 + 8u * slot, dst = b0 + uint32_t(slot) * b_stage_bytes;
                    const int kcol = (tap * t.cchunks + cc) * t.chunk;
                    mbar_expect_tx(bar, uint32_t(b_stage_bytes));
                    tma_load_2d(dst, &tmap_b, bar, kcol, cout0);
                    if (kX3) tma_load_2d(dst + uint32_t(b_bytes), &tmap_b, bar, kcol, t.cout_pad + cout0);
                    ++issued;
                }
            }
        }
        if (!ok) {
            atomicCAS(p.error_flag, 0, 12);
            // the loads this lane has issued still land here: wait for the latest one of each of its stages
            if (!t.b_resident)
                for (int j = issued - 1, k = 0; j >= 0 && k < t.b_depth; --j, ++k)
                    mbar_wait(b_full0 + 8u * (w * t.b_depth + j % t.b_depth), uint32_t((j / t.b_depth) & 1), nullptr);
        }
        if (t.b_resident && issued > 0) {
            // (resident stages are waited for by the issuers; on a failure elsewhere this lane still owes the CTA the
            //  arrival of what it asked for before the shared memory may be given up)
            for (int cc = 0; cc < t.cchunks; ++cc)
                for (int tap = w; tap < t.taps; tap += W) mbar_wait(b_full0 + 8u * (cc * t.taps + tap), 0u, nullptr);
        }
        return;
    }
    if (warp == 1 || warp >= 10) {
        // ---------------- MMA issuers: taps issuer, issuer + W, ... of every channel chunk ----------------
        const int W = t.issuers;
        const uint32_t fmt = kBf16 ? 1u : 2u;
        const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(t.bn >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
        const uint32_t idesc_wide = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(t.bn >> 2) << 17) | (uint32_t(kTileM >> 4) << 24);
        const uint32_t a_wait0 = kX3 ? a_ready0 : a_full0;
        int sa = 0, sb = 0;
        uint32_t pa = 0, pb = 0;
        bool ok = true;
#pragma unroll 1
        for (int ti = 0; ti < my_tiles && ok; ++ti) {
            const uint32_t a = uint32_t(ti) & 1u;
            const uint32_t tile_parity = (uint32_t(ti) >> 1) & 1u;
            // the epilogue must have emptied this set of accumulators (sets 0 and 1 start out free: parity 1 passes)
            ok = mbar_wait(acc_empty0 + 8u * a, tile_parity ^ 1u, p.error_flag);
            if (!ok) { gave_up(2 + issuer, ti, 0, 0, 3); break; }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + (a * uint32_t(t.issuers) + uint32_t(issuer)) * uint32_t(t.acc_stride);
            uint32_t first = 0u;                            // 0 until this issuer's first instruction of the tile is out
#pragma unroll 1
            for (int cc = 0; cc < t.cchunks && ok; ++cc) {
                ok = mbar_wait(a_wait0 + 8u * sa, pa, p.error_flag);
                if (!ok) { gave_up(2 + issuer, ti, cc, 0, 4); break; }
                tc_fence_after();
                const uint32_t a_hi = a0 + uint32_t(sa) * a_stage_bytes;
                int r = issuer / t.kw, sx = issuer - r * t.kw;
#pragma unroll 1
                for (int tap = issuer; tap < t.taps; tap += W) {
                    // resident weights: a stage per (chunk, tap), filled once; else this issuer's own ring
                    const int slot = t.b_resident ? cc * t.taps + tap : issuer * t.b_depth + sb;
                    ok = mbar_wait(b_full0 + 8u * slot, t.b_resident ? 0u : pb, p.error_flag);
                    if (!ok) { gave_up(2 + issuer, ti, cc, tap, 5); break; }
                    tc_fence_after();
                    const uint32_t a_tap = a_hi + uint32_t(r * t.pw + sx) * kRow;
                    const uint64_t da = smem_desc_kmajor(a_tap, kRow), dal = smem_desc_kmajor(a_tap + uint32_t(a_plane), kRow);
                    const uint32_t b_hi = b0 + uint32_t(slot) * b_stage_bytes;
                    const uint64_t db = smem_desc_kmajor(b_hi, kRow), dbl = smem_desc_kmajor(b_hi + uint32_t(b_bytes), kRow);
#pragma unroll
                    for (int k = 0; k < kRow / 32; ++k) {
                        const uint32_t acc = first | (k > 0 ? 1u : 0u);
                        if (kX3 && t.wide) {
                            umma_tf32(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc_wide, acc);
                            umma_tf32(tmem_d, dal + uint64_t(k * 2), db + uint64_t(k * 2), idesc, 1u);
                        } else if (kX3) {
                            umma_tf32(tmem_d, dal + uint64_t(k * 2), db + uint64_t(k * 2), idesc, acc);
                            umma_tf32(tmem_d, da + uint64_t(k * 2), dbl + uint64_t(k * 2), idesc, 1u);
                            umma_tf32(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, 1u);
                        } else if (kBf16) {
                            umma_f16(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, acc);
                        } else {
                            umma_tf32(tmem_d, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, acc);
                        }
                        first = 1u;
                    }
                    if (!t.b_resident) {
                        umma_commit(b_empty0 + 8u * slot);
                        if (++sb == t.b_depth) { sb = 0; pb ^= 1u; }
                    }
                    sx += W;
                    while (sx >= t.kw) { sx -= t.kw; ++r; }
                }
                if (!ok) break;
                umma_commit(a_empty0 + 8u * sa);          // one arrival per issuer: the patch is free once all have read it
                if (++sa == t.a_stages) { sa = 0; pa ^= 1u; }
            }
            if (ok) umma_commit(acc_full0 + 8u * a);
        }
        if (!ok) atomicCAS(p.error_flag, 0, 20 + issuer);
        return;
    }
    if (kX3 && warp >= 6) {
        // ---------------- warps 6..9 (three-pass mode): residual of every landed patch ----------------
        const int tid = threadIdx.x - 192;
        const int n_vec = t.a_tx_bytes >> 4;
        const long steps = long(my_tiles) * t.cchunks;
        int s = 0;
        uint32_t phase = 0;
#pragma unroll 1
        for (long i = 0; i < steps; ++i) {
            if (!mbar_wait(a_full0 + 8u * s, phase, p.error_flag)) {
                atomicCAS(p.error_flag, 0, 50);
                break;
            }
            uint8_t *stage = generic_base + size_t(s) * a_stage_bytes;
            const float4 *hi = reinterpret_cast<const float4 *>(stage);
            float4 *lo = reinterpret_cast<float4 *>(stage + a_plane);
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
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a_ready0 + 8u * s) : "memory");
            if (++s == t.a_stages) { s = 0; phase ^= 1u; }
        }
        return;
    }
    // ---------------- epilogue warps ----------------
    const int e = warp - 2;
    const int etid = threadIdx.x - 64;
    const int epi_threads = epi_warps * 32;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int cols_per_warp = epi_warps == 8 ? t.bn / 2 : t.bn;
    const int c_begin = (e >> 2) * cols_per_warp, c_end = c_begin + cols_per_warp;
    const uint32_t pair = t.wide ? uint32_t(t.bn) : 0u;
    // which output pixel of a tile this thread's row is (the same for every tile)
    const int per_image = t.ph * t.pw;
    const int img = row / per_image;
    const int rem = row - img * per_image;
    const int ry = rem / t.pw, rx = rem - ry * t.pw;
    const bool row_in_box = img < t.box_n && ry < t.box_h && rx < t.box_w;
    uint8_t *staging = generic_base + (staging0 - smem_base);
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the output window may still be read by the previous kernel
#pragma unroll 1
    for (int ti = 0; ti < my_tiles; ++ti) {
        int cout0, ow0, oh0, n0;
        decode(int(blockIdx.x) + ti * int(gridDim.x), cout0, ow0, oh0, n0);
        const uint32_t a = uint32_t(ti) & 1u;
        float *bias = bias_s[a];
        for (int j = etid; j < t.bn; j += epi_threads) bias[j] = (p.bias && cout0 + j < g.Cout) ? p.bias[cout0 + j] : 0.0f;
        bool ok = mbar_wait(acc_full0 + 8u * a, (uint32_t(ti) >> 1) & 1u, p.error_flag);
        ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
        if (!ok && lane == 0) {
            atomicCAS(p.error_flag, 0, 60);
            if (warp == 2) gave_up(7, ti, 0, 0, 6);
        }
        tc_fence_after();
        // the bulk stores of the previous tile must have read the staging area before it is written again
        if (t.tma_store && etid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");      // bias complete, staging free
        const int valid = min(t.bn, g.Cout - cout0);
        const int n = n0 + img, oh = oh0 + ry, ow = ow0 + rx;
        const bool live = ok && row_in_box && n < g.N && oh < g.OH && ow < g.OW;
        const long pix_off = ((long(n) * g.OH + oh) * g.OW + ow) * p.out.pitch;
        if (ok) {
            const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + a * uint32_t(t.issuers * t.acc_stride);
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 16) {
                float v[16];
                acc_ld16(taddr + c, pair, v);              // (a warp-wide instruction: every lane takes part)
#pragma unroll 1
                for (int w = 1; w < t.issuers; ++w) {       // the other issuers' partial sums, always in this order
                    float u[16];
                    acc_ld16(taddr + uint32_t(w * t.acc_stride) + c, pair, u);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] += u[j];
                }
                if (!t.tma_store && (!live || c >= valid)) continue;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float z = act_apply(v[j] + bias[c + j], g.act);
                    v[j] = t.round_tf32 ? round_tf32(z) : z;
                }
                if (t.tma_store) {
                    // every row is staged, halo rows too: the stores below pick the row segments that are output
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        stage4(staging, row, c + j, make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]), kBf16);
                    continue;
                }
#pragma unroll
                for (int j = 0; j < 16; j += 8)
                    if (c + j < valid) store8_direct(p.out.ptr, kBf16, pix_off + cout0 + c + j, v + j, valid - (c + j));
            }
        }
        // hand the accumulator back to the MMA issuers: one arrival per epilogue warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8u * a) : "memory");
        if (t.tma_store) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");  // the tile is staged
            if (ok && etid == 0) {
                for (int c = 0; c < valid; c += t.slab) {
                    const uint32_t slab_base = staging0 + uint32_t(c / t.slab) * kATileBytes;
                    for (int i = 0; i < t.box_n && n0 + i < g.N; ++i)
                        for (int y = 0; y < t.box_h && oh0 + y < g.OH; ++y)
                            tma_store_4d(&tmap_c, slab_base + uint32_t((i * t.ph + y) * t.pw) * 128u, cout0 + c, ow0, oh0 + y, n0 + i);
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

}  // namespace

// ---- host side -------------------------------------------------------------------------------
namespace {

int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

// Cycles the TMA unit of an SM spends on a load of `rows` rows of 128 bytes (measured on B200: a layer
// bound by its loads takes about 1.15 cycles per row plus one cycle per 100 bytes, whatever the mode).
double tma_cycles(double rows, int row_bytes) { return rows * 1.15 + rows * row_bytes / 100.0; }

}  // namespace

// Decides whether a convolution that conv_tc_choose gave to the resident-CTA kernel should run as a patch
// convolution instead, and if so rewrites the plan (tile width, geometry, shared memory, grid).
void conv_tc_patch_consider(const ConvGeom &g, int sm_count, ConvTcPlan *plan) {
    ConvTcPlan &q = *plan;
    q.patch = 0;
    if (q.no_patch || !q.persistent || q.split_k != 1) return;
    if (g.sh != 1 || g.sw != 1 || g.kh * g.kw < 2 || g.groups != 1) return;
    const int taps = g.kh * g.kw;
    if (g.kw > 64 || g.kh > 64) return;
    // a window of one row never looks across image rows: images and rows become one axis
    const bool merged = g.kh == 1 && g.ph == 0;
    const int OHm = merged ? g.N * g.OH : g.OH, Nm = merged ? 1 : g.N;
    // output-channel tile: as wide as tensor memory allows (a patch is loaded once per output-channel tile)
    const int bn_step = q.bf16 ? 64 : 32;
    const int bn_cap = 256;
    const int n_tiles = ceil_div_i(g.Cout, bn_cap);
    const int bn = std::min(bn_cap, ceil_div_i(ceil_div_i(g.Cout, n_tiles), bn_step) * bn_step);
    const bool wide = q.x3 && bn <= 128;
    const int acc_cols = (wide ? 2 : 1) * ceil_div_i(bn, 32) * 32;
    if (2 * acc_cols > 512) return;
    const int planes = q.x3 ? 2 : 1;
    const int row = q.half_rows ? 64 : 128;              // bfloat16 layers of at most 32 input channels: 64-byte operand rows
    const int chunk = q.bf16 ? (q.half_rows ? 32 : 64) : 32;
    const int cchunks = ceil_div_i(g.Cin, chunk);
    const int b_stage = planes * bn * row;
    // weights that fit stay resident (the first layers of a network: a few dozen KiB)
    const bool b_resident = n_tiles == 1 && taps * cchunks <= 48 && long(taps) * cchunks * b_stage <= 72 * 1024;
    auto fixed_bytes = [](int as, int bs) { return 1024 + 8 * (3 * as + 2 * bs) + 160; };   // alignment slack, barriers, slot
    const double tensor_col = 2.1 * 1.15 * (q.x3 ? 3.0 : 1.0);
    // one thread issues an instruction about every 140 cycles; up to four threads take turns
    const double issue_one = (q.x3 ? (wide ? 8 : 12) : row / 32) * 140.0 + 60.0;

    // tile extent: output rows cut into `parts` even segments of box_w pixels, as many rows (and, where a whole
    // image fits, images) as 128 GEMM rows hold beside the halo columns; the cheapest candidate wins
    struct Cand { int box_w, box_h, box_n, pw, ph, a_rows, tiles_w, tiles_h, tiles_n, resident, a_stages, b_stages, issuers, b_depth, staging; double cost; };
    const int slab_channels = q.bf16 ? 64 : 32;
    const int staging_bytes = ceil_div_i(bn, slab_channels) * kATileBytes;
    Cand best = {};
    best.cost = 1e30;
    const int min_parts = ceil_div_i(g.OW, kTileM - g.kw + 1);
    for (int parts = min_parts; parts < min_parts + 8 && parts <= g.OW; ++parts) {
        Cand c = {};
        c.box_w = ceil_div_i(g.OW, parts);
        c.pw = (c.box_w + g.kw - 1 + 7) / 8 * 8;        // a multiple of 8: output row segments start on whole swizzle atoms
        c.box_h = std::min(OHm, (kTileM - c.box_w) / c.pw + 1);
        c.box_h = ceil_div_i(OHm, ceil_div_i(OHm, c.box_h));
        c.ph = c.box_h + g.kh - 1;
        c.box_n = 1;
        if (c.box_w == g.OW && c.box_h == OHm && Nm > 1) {
            c.box_n = std::min(Nm, (kTileM - ((c.box_h - 1) * c.pw + c.box_w)) / (c.ph * c.pw) + 1);
            c.box_n = ceil_div_i(Nm, ceil_div_i(Nm, c.box_n));
        }
        if (c.pw > 256 || c.ph > 256 || c.box_n > 256) continue;
        const int patch_rows = c.box_n * c.ph * c.pw;
        const int max_off = (g.kh - 1) * c.pw + g.kw - 1;
        c.a_rows = (std::max(patch_rows, kTileM + max_off) + 15) / 16 * 16;      // whole 1024-byte units also with 64-byte rows
        c.tiles_w = ceil_div_i(g.OW, c.box_w);
        c.tiles_h = ceil_div_i(OHm, c.box_h);
        c.tiles_n = ceil_div_i(Nm, c.box_n);
        const long m_tiles = long(c.tiles_w) * c.tiles_h * c.tiles_n;
        if (m_tiles * n_tiles > (1l << 24)) continue;
        const int a_stage = planes * c.a_rows * row;
        // finished tiles leave through one bulk tensor store per output row segment and 128-byte channel slab, staged in
        // shared memory -- unless a tile has so many short segments (small images) that plain stores are cheaper
        // (measured on B200: with the patch loads queued ahead of them in the same TMA unit these small stores are
        //  slower than 16-byte stores from registers for most layers, so they are a testing aid, off by default)
        c.staging = (q.patch_bulk_store && ceil_div_i(bn, slab_channels) * c.box_h * c.box_n <= 16) ? staging_bytes : 0;
        // issuing warps: as many as there are taps, up to four (or the cap of the testing aid); when the weights are not
        // resident every issuer has a ring of its own of at least two stages, so fewer issuers where memory is short
        const int w_max = std::max(1, std::min({kMaxIssuers, taps, q.max_issuers > 0 ? q.max_issuers : kMaxIssuers}));
        // one CTA per SM (all of its shared and tensor memory) or two smaller ones: whichever the model below prefers
        const int patch_rows_c = patch_rows;
        Cand pick = c;
        pick.cost = 1e30;
        for (int want = 2; want >= 1; --want) {       // (on a tie two CTAs: measured faster than one with twice the issuers)
            Cand d = c;
            const int as_min = (cchunks > 1 || m_tiles * n_tiles > long(sm_count) * want) ? 2 : 1;
            const int budget = (want == 2 ? 110 : 210) * 1024;
            for (int w = w_max; w >= 1 && !d.resident; --w) {
                // tensor memory: two sets (alternating tiles) of one accumulator per issuer, a power of two of columns
                int tmem = 32;
                while (tmem < 2 * w * acc_cols) tmem *= 2;
                if (tmem > (want == 2 ? 256 : 512)) continue;
                const int bs_min = b_resident ? taps * cchunks : (w == 1 ? 3 : 2 * w);
                if (as_min * a_stage + bs_min * b_stage + d.staging + fixed_bytes(as_min, bs_min) > budget) continue;
                d.resident = want;
                d.issuers = w;
                d.a_stages = as_min;
                d.b_depth = b_resident ? 1 : bs_min / w;
                d.b_stages = bs_min;
                while (d.a_stages < 3 &&
                       (d.a_stages + 1) * a_stage + d.b_stages * b_stage + d.staging + fixed_bytes(d.a_stages + 1, d.b_stages) <= budget)
                    ++d.a_stages;
                while (!b_resident && d.b_depth < 4 &&
                       d.a_stages * a_stage + (d.b_depth + 1) * w * b_stage + d.staging + fixed_bytes(d.a_stages, (d.b_depth + 1) * w) <= budget) {
                    ++d.b_depth;
                    d.b_stages = d.b_depth * w;
                }
            }
            if (!d.resident) continue;
            // per SM: the TMA unit serves the resident CTAs in turn, the tensor pipe too, the issuing threads work side by side
            const double chunk_cycles = std::max({tma_cycles(patch_rows_c, row) + (b_resident ? 0.0 : tma_cycles(double(taps) * bn * planes, row)),
                                                  taps * bn * tensor_col, taps * issue_one / d.issuers / d.resident});
            d.cost = double(m_tiles) * n_tiles * (cchunks * chunk_cycles + 400.0);
            if (d.cost < pick.cost) pick = d;
        }
        c = pick;
        if (!c.resident) continue;
        if (c.cost < best.cost) best = c;
    }
    if (best.cost >= 1e30) return;
    // Measured inside whole networks (Inception-v3, batch 64 and 256): layers whose weights stay resident gain (the
    // first convolutions of a network, 3 % of a forward in bfloat16), except single-pass TF32 layers with wide float32
    // outputs, which are bound by their stores; layers that stream their weights win when timed alone but lose a few
    // per cent in the network, so they only take this path when asked to (option patch=all).
    if (!q.patch_all && (!b_resident || (!q.bf16 && !q.x3 && g.Cout > 32))) return;
    // compare with what the plan has now (an activation tile per tap)
    const long old_tiles = (long(g.N) * g.OH * g.OW + kTileM - 1) / kTileM * q.n_tiles;
    const double old_step = std::max({tma_cycles(kTileM + double(q.bn) * planes, row), q.bn * tensor_col, (q.x3 ? 700.0 : 450.0) / 2.0});
    const double old_cost = double(old_tiles) * (double(taps) * q.cchunks * old_step + 400.0);
    if (best.cost > 0.92 * old_cost) return;
    const int box_w = best.box_w, box_h = best.box_h, box_n = best.box_n, pw = best.pw, ph = best.ph, a_rows = best.a_rows;
    const int tiles_w = best.tiles_w, tiles_h = best.tiles_h, tiles_n = best.tiles_n;
    const int resident = best.resident, a_stages = best.a_stages, b_stages = best.b_stages;
    q.patch_issuers = best.issuers;
    q.patch_b_depth = best.b_depth;
    q.patch_staging = best.staging;
    const long m_tiles = long(tiles_w) * tiles_h * tiles_n;
    const int a_stage = planes * a_rows * row;
    const int fixed = fixed_bytes(a_stages, b_stages);

    q.patch = 1;
    q.cchunks = cchunks;
    q.k_iters = taps * cchunks;
    q.bn = bn;
    q.n_tiles = n_tiles;
    q.cout_pad = n_tiles * bn;
    q.box_w = box_w; q.box_h = box_h; q.box_n = box_n;
    q.tiles_w = tiles_w; q.tiles_h = tiles_h; q.tiles_n = tiles_n;
    q.patch_pw = pw; q.patch_ph = ph; q.patch_a_rows = a_rows;
    q.patch_a_stages = a_stages; q.patch_b_stages = b_stages; q.patch_b_resident = b_resident ? 1 : 0;
    q.patch_merged = merged ? 1 : 0;
    q.im2col = 0;
    q.flat_1x1 = 0;
    q.stages = b_stages;
    q.persistent = 1;
    q.grid_ctas = int(std::min<long>(m_tiles * n_tiles, long(sm_count) * resident));
    q.smem_bytes = size_t(a_stages) * a_stage + size_t(b_stages) * b_stage + size_t(best.staging) + fixed;
    // a CTA that needs the SM to itself also takes more than half of its shared memory
    if (resident == 1) q.smem_bytes = std::max(q.smem_bytes, size_t(120 * 1024));
    q.workspace_bytes = 0;
    q.counter_bytes = 0;
}

cudaError_t conv_tc_patch_prepare() {
    const void *forms[] = {reinterpret_cast<const void *>(conv_tc_patch_kernel<0>), reinterpret_cast<const void *>(conv_tc_patch_kernel<1>),
                           reinterpret_cast<const void *>(conv_tc_patch_kernel<2>), reinterpret_cast<const void *>(conv_tc_patch_kernel<4>)};
    for (const void *form : forms) {
        cudaError_t err = cudaFuncSetAttribute(form, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);
        if (err != cudaSuccess) return err;
    }
    return cudaSuccess;
}

void launch_conv_tc_patch(const ConvTcParams &p, const ConvTcPlan &q, cudaStream_t stream) {
    PatchGeom t;
    const ConvGeom &g = p.g;
    const int row = q.half_rows ? 64 : 128;
    t.bn = q.bn; t.cchunks = q.cchunks; t.taps = g.kh * g.kw; t.kw = g.kw; t.chunk = q.bf16 ? (q.half_rows ? 32 : 64) : 32;
    t.pw = q.patch_pw; t.ph = q.patch_ph;
    t.box_w = q.box_w; t.box_h = q.box_h; t.box_n = q.box_n;
    t.tiles_w = q.tiles_w; t.tiles_h = q.tiles_h; t.n_tiles = q.n_tiles;
    t.total_tiles = q.tiles_w * q.tiles_h * q.tiles_n * q.n_tiles;
    t.a_rows = q.patch_a_rows; t.a_stages = q.patch_a_stages; t.b_stages = q.patch_b_stages;
    t.a_tx_bytes = q.patch_pw * q.patch_ph * q.box_n * row;
    t.b_resident = q.patch_b_resident;
    t.wide = (q.x3 && q.bn <= 128) ? 1 : 0;
    t.acc_stride = (t.wide ? 2 : 1) * ceil_div_i(q.bn, 32) * 32;
    int cols = 32;
    while (cols < 2 * q.patch_issuers * t.acc_stride) cols *= 2;
    t.tmem_cols = cols;
    t.round_tf32 = g.round_out;
    t.cout_pad = q.cout_pad;
    t.pad_w = g.pw; t.pad_h = g.ph;
    t.issuers = q.patch_issuers;
    t.b_depth = q.patch_b_depth;
    t.tma_store = (q.patch_staging > 0 && q.tma_store) ? 1 : 0;
    t.slab = q.bf16 ? 64 : 32;
    ConvTcParams pp = p;
    if (q.patch_merged) {               // images and rows as one axis (see conv_tc_patch_consider)
        pp.g.H = g.N * g.H; pp.g.OH = g.N * g.OH; pp.g.N = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(std::min(q.grid_ctas, t.total_tiles)));
    cfg.blockDim = dim3(kPatchThreads);
    cfg.dynamicSmemBytes = q.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int n_attr = 0;
    if (q.pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    const CUtensorMap &ma = *reinterpret_cast<const CUtensorMap *>(q.tmap_a), &mb = *reinterpret_cast<const CUtensorMap *>(q.tmap_b),
                      &mc = *reinterpret_cast<const CUtensorMap *>(q.tmap_c);
    if (std::getenv("IOS_DEBUG_PATCH"))
        std::fprintf(stderr, "patch conv: N %d H %d W %d Cin %d Cout %d k %dx%d pad %d,%d | bn %d n_tiles %d cchunks %d box %dx%dx%d patch %dx%d "
                     "a_rows %d a_stages %d b_stages %d resident_b %d tiles %d grid %u smem %zu tmem %d issuers %d depth %d tma_store %d x3 %d bf16 %d merged %d\n",
                     pp.g.N, pp.g.H, pp.g.W, g.Cin, g.Cout, g.kh, g.kw, g.ph, g.pw, t.bn, t.n_tiles, t.cchunks, t.box_w, t.box_h, t.box_n, t.pw, t.ph,
                     t.a_rows, t.a_stages, t.b_stages, t.b_resident, t.total_tiles, cfg.gridDim.x, q.smem_bytes, t.tmem_cols, t.issuers, t.b_depth, t.tma_store, q.x3, q.bf16,
                     q.patch_merged);
    if (q.x3) cudaLaunchKernelEx(&cfg, conv_tc_patch_kernel<1>, ma, mb, mc, pp, t);
    else if (q.bf16 && q.half_rows) cudaLaunchKernelEx(&cfg, conv_tc_patch_kernel<4>, ma, mb, mc, pp, t);
    else if (q.bf16) cudaLaunchKernelEx(&cfg, conv_tc_patch_kernel<2>, ma, mb, mc, pp, t);
    else cudaLaunchKernelEx(&cfg, conv_tc_patch_kernel<0>, ma, mb, mc, pp, t);
}

}  // namespace ios
