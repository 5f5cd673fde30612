// A pointwise (1x1) convolution entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a convolution: a
// plug-in that runs inside another framework's memory pool and is forbidden to allocate outside
// it, a real-time loop that may not take the allocator's locks, a process whose whole device
// memory budget has been handed out up front.  For them the split-K scratch of the tensor-core
// convolution -- partial accumulator tiles, one arrival counter per output tile and the
// time-out word -- lives in a fixed array inside the library image instead of an arena.
//
// Consequences the caller has to know:
//  * every GPU that loads the library carries the array (8 MiB + 20 KiB) until the process exits;
//  * problems whose scratch need exceeds it are refused with IOS_ERR_LIMIT, nothing is launched;
//  * all calls share the one array and it keeps whatever the last call left in it: the counters
//    and the time-out word are cleared (stream-ordered) at the start of every call, partial tiles
//    are always written before they are read; two calls that overlap on the GPU (different
//    streams, no dependency) race on it and give undefined results;
//  * the first call on a device looks up the array's device address and raises the kernel's
//    shared-memory limit; make that first call outside of any stream capture;
//  * the call returns once the work is enqueued.  Whether a bounded wait inside the kernel ran out
//    is only known afterwards: ios_static_scratch_status() synchronises the stream, reads the
//    time-out word (again without allocating) and reports IOS_ERR_TIMEOUT, in which case y is not
//    complete.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/ios_runtime.h"
#include "kernels.h"

namespace ios {
void record_error(const char *message);

namespace {

constexpr size_t kFlagBytes = 256;                      // time-out word
constexpr size_t kCounterBytes = 20 * 1024 - 256;       // one 4-byte arrival counter per output tile
constexpr size_t kPartialBytes = size_t(8) << 20;       // split-K partial tiles
constexpr size_t kScratchBytes = kFlagBytes + kCounterBytes + kPartialBytes;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
    bool ready = false;
    unsigned char *scratch = nullptr;   // device address of g_static_scratch on this device
    int sm_count = 0;
};
PerDevice g_devices[kMaxDevices];
std::mutex g_setup_mutex;

int fail(int status, const char *message) {
    record_error(message);
    return status;
}

// Once per device, with that device current.
int setup_device(int device, PerDevice **out) {
    if (device < 0 || device >= kMaxDevices) return fail(IOS_ERR_LIMIT, "device index beyond the supported 64");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    PerDevice &d = g_devices[device];
    if (!d.ready) {
        void *address = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&address, g_static_scratch);
        if (err != cudaSuccess) {
            static thread_local char text[160];
            std::snprintf(text, sizeof text, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(err));
            return fail(IOS_ERR_CUDA, text);
        }
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || major < 10)
            return fail(IOS_ERR_CUDA, "the current device is not sm_100: the kernels are built for B200 only");
        if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
            return fail(IOS_ERR_CUDA, "cudaDeviceGetAttribute(multiProcessorCount) failed");
        if (conv_tc_prepare() != cudaSuccess) return fail(IOS_ERR_CUDA, "raising the shared-memory limit of the kernel failed");
        d.scratch = static_cast<unsigned char *>(address);
        d.ready = true;
    }
    *out = &d;
    return IOS_OK;
}

}  // namespace
}  // namespace ios

using namespace ios;

extern "C" int ios_pointwise_conv_static_scratch(const float *x, const float *w, const float *bias, float *y,
                                                 int pixels, int cin, int cout, int act, int split_k, void *cuda_stream) {
    if (!x || !w || !y) return fail(IOS_ERR_ARGUMENT, "x, w and y must be device pointers, not NULL");
    if (pixels <= 0 || cin <= 0 || cout <= 0 || act < 0 || act > 3 || split_k < 0)
        return fail(IOS_ERR_ARGUMENT, "pixels, cin, cout must be positive, act in 0..3, split_k >= 0");
    if (cin % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
        return fail(IOS_ERR_ARGUMENT, "cin must be a multiple of 4 and x, w 16-byte aligned (TMA row pitch)");
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return fail(IOS_ERR_CUDA, "no current CUDA device");
    PerDevice *dev = nullptr;
    if (int status = setup_device(device, &dev)) return status;

    ConvTcParams p = {};
    p.in.ptr = const_cast<float *>(x);
    p.in.esize = p.out.esize = 4;
    p.in.N = 1; p.in.H = 1; p.in.W = pixels; p.in.C = cin; p.in.pitch = cin;
    p.out.ptr = y;
    p.out.N = 1; p.out.H = 1; p.out.W = pixels; p.out.C = cout; p.out.pitch = cout;
    ConvGeom &g = p.g;
    g.N = 1; g.Cin = cin; g.H = 1; g.W = pixels;
    g.Cout = cout; g.OH = 1; g.OW = pixels;
    g.kh = g.kw = g.sh = g.sw = 1;
    g.ph = g.pw = 0;
    g.groups = 1;
    g.act = act;
    g.pre_relu = 0;
    g.round_out = 0;

    ConvTcPlan plan = {};
    plan.no_persistent = 1;                             // this entry point exists for the kernel that uses the scratch
    conv_tc_choose(g, dev->sm_count, 1, /*three_pass=*/false, &plan);
    plan.cluster = 0;                                   // reduce through the (static) workspace, not a cluster
    conv_tc_set_split(&plan, split_k > 0 ? split_k : plan.split_k);
    plan.pdl = 0;
    const size_t tiles = size_t(plan.tiles_w) * plan.tiles_h * plan.tiles_n * plan.n_tiles;
    if (plan.workspace_bytes > kPartialBytes || tiles * sizeof(unsigned int) > kCounterBytes) {
        static thread_local char text[200];
        std::snprintf(text, sizeof text,
                      "this problem needs %zu bytes of split-K scratch and %zu tile counters; the static scratch holds "
                      "%zu bytes and %zu counters (lower split_k or use the arena-backed entry points)",
                      plan.workspace_bytes, tiles, kPartialBytes, kCounterBytes / sizeof(unsigned int));
        return fail(IOS_ERR_LIMIT, text);
    }
    p.weight_packed = w;
    p.bias = bias;
    p.error_flag = reinterpret_cast<int *>(dev->scratch);
    p.counters = reinterpret_cast<unsigned int *>(dev->scratch + kFlagBytes);
    p.workspace = reinterpret_cast<float *>(dev->scratch + kFlagBytes + kCounterBytes);
    p.timeline = nullptr;
    if (const char *err = conv_tc_encode_dense_weights(p, &plan)) return fail(IOS_ERR_CUDA, err);

    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    // the counters and the time-out word must start at zero; partial tiles are written before they are read
    if (cudaMemsetAsync(dev->scratch, 0, kFlagBytes + kCounterBytes, stream) != cudaSuccess)
        return fail(IOS_ERR_CUDA, "clearing the static scratch failed");
    launch_conv_tc(p, plan, stream);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        static thread_local char text[160];
        std::snprintf(text, sizeof text, "launching the convolution failed: %s", cudaGetErrorString(err));
        return fail(IOS_ERR_CUDA, text);
    }
    record_error("");
    return IOS_OK;
}

extern "C" int ios_static_scratch_status(void *cuda_stream) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return fail(IOS_ERR_CUDA, "no current CUDA device");
    if (device < 0 || device >= kMaxDevices) return fail(IOS_ERR_LIMIT, "device index beyond the supported 64");
    unsigned char *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (g_devices[device].ready) scratch = g_devices[device].scratch;
    }
    if (!scratch) {                       // nothing has run on this device yet
        record_error("");
        return IOS_OK;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t err = cudaStreamSynchronize(stream);
    int word = 0;
    if (err == cudaSuccess) err = cudaMemcpy(&word, scratch, sizeof word, cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) {
        static thread_local char text[160];
        std::snprintf(text, sizeof text, "reading the time-out word failed: %s", cudaGetErrorString(err));
        return fail(IOS_ERR_CUDA, text);
    }
    if (word != 0) {
        // leave the scratch ready for the next call: the word and the arrival counters start at zero
        cudaMemset(scratch, 0, kFlagBytes + kCounterBytes);
        static thread_local char text[160];
        std::snprintf(text, sizeof text, "a bounded wait inside the convolution kernel ran out (code %d): the output is incomplete", word);
        return fail(IOS_ERR_TIMEOUT, text);
    }
    record_error("");
    return IOS_OK;
}
