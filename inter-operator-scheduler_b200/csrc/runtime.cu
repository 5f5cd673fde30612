// Stage executor, latency measurement and the C-ABI of libios_runtime.so.
//
// Counterpart of Graph::forward, measure_latency, measure_stage_latency and the four extern "C"
// functions of the reference (src/ios/ios_runtime.cu:1297-1315, 1328-1455, 1478-1519), rebuilt
// around a launch list and CUDA graphs:
//  * group j of a stage is issued on stream j; stream 0 is the spine: a multi-group stage forks the
//    other streams off an event on stream 0 and joins them back before the next stage, so stage
//    boundaries cost event edges instead of the reference's cudaDeviceSynchronize (:1309-1312);
//  * a whole forward (or `number` repetitions of a candidate stage) is captured once into a CUDA
//    graph and replayed, which removes the per-kernel host launch cost that dominates batch 1;
//  * all device memory of a plan comes from one grow-only arena per process, so the thousands of
//    stage_latency calls of a schedule search allocate nothing after the first few.
// Errors never terminate the process: every entry point catches, records a message for
// ios_last_error() and returns a status.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/ios_runtime.h"
#include "graph.h"
#include "kernels.h"
#include "plan.h"

namespace ios {
namespace {

thread_local std::string g_last_error;
std::mutex g_mutex;              // the process-wide arena and option block are shared
Options g_options;
int g_device = 0;

struct CudaError : std::runtime_error {
    explicit CudaError(const std::string &what) : std::runtime_error(what) {}
};
struct TimeoutError : std::runtime_error {
    explicit TimeoutError(const std::string &what) : std::runtime_error(what) {}
};
struct ArgumentError : std::runtime_error {
    explicit ArgumentError(const std::string &what) : std::runtime_error(what) {}
};
struct MissingWeights : std::runtime_error {
    explicit MissingWeights(const std::string &what) : std::runtime_error(what) {}
};

#define CUDA_OK(expr)                                                                                   \
    do {                                                                                                \
        cudaError_t err__ = (expr);                                                                     \
        if (err__ != cudaSuccess)                                                                       \
            throw CudaError(std::string(#expr) + ": " + cudaGetErrorString(err__));                     \
    } while (0)

// ---- streams and events of one executor ---------------------------------------------------
// Group j of a stage runs on streams[j]; events are the fork / join edges.  The process-wide context of
// a device owns one set (used by the latency and inference entry points), every engine owns its own, so
// that engines run side by side from several host threads.
struct StreamSet {
    std::vector<cudaStream_t> streams;
    std::vector<cudaEvent_t> events;       // fork / join edges, reused by every plan
    cudaEvent_t t_start = nullptr, t_end = nullptr;

    void init_timers() {
        if (!t_start) CUDA_OK(cudaEventCreate(&t_start));
        if (!t_end) CUDA_OK(cudaEventCreate(&t_end));
    }
    void need_streams(int n) {
        while (int(streams.size()) < n) {
            cudaStream_t s;
            CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
            streams.push_back(s);
        }
    }
    cudaEvent_t event(size_t i) {
        while (events.size() <= i) {
            cudaEvent_t e;
            CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            events.push_back(e);
        }
        return events[i];
    }
    void release() {
        for (cudaStream_t s : streams) cudaStreamDestroy(s);
        for (cudaEvent_t e : events) cudaEventDestroy(e);
        if (t_start) cudaEventDestroy(t_start);
        if (t_end) cudaEventDestroy(t_end);
        streams.clear();
        events.clear();
        t_start = t_end = nullptr;
    }
};

// ---- device context: shared streams and the grow-only arena --------------------------------
struct DeviceContext : StreamSet {
    int device = -1;
    int sm_count = 148;
    char *arena = nullptr;
    size_t arena_capacity = 0;

    void init(int dev) {
        if (device == dev) return;
        int count = 0;
        cudaError_t err = cudaGetDeviceCount(&count);
        if (err != cudaSuccess || count == 0)
            throw CudaError("no CUDA device is available: this library has no CPU path (" +
                            std::string(err == cudaSuccess ? "device count is 0" : cudaGetErrorString(err)) + ")");
        if (dev < 0 || dev >= count) throw ArgumentError("device index out of range");
        CUDA_OK(cudaSetDevice(dev));
        cudaDeviceProp prop;
        CUDA_OK(cudaGetDeviceProperties(&prop, dev));
        if (prop.major < 10)
            throw CudaError(std::string("device '") + prop.name + "' is not sm_100: the kernels are built for B200 only");
        sm_count = prop.multiProcessorCount;
        CUDA_OK(conv_tc_prepare());
        init_timers();
        device = dev;
    }
    char *need_arena(size_t bytes) {
        if (bytes > arena_capacity) {
            if (arena) {
                CUDA_OK(cudaDeviceSynchronize());
                CUDA_OK(cudaFree(arena));
                arena = nullptr;
                arena_capacity = 0;
            }
            size_t want = bytes + bytes / 4;
            want = (want + (size_t(1) << 21) - 1) >> 21 << 21;
            cudaError_t err = cudaMalloc(&arena, want);
            if (err != cudaSuccess) {
                cudaGetLastError();
                want = (bytes + 4095) / 4096 * 4096;
                CUDA_OK(cudaMalloc(&arena, want));
            }
            arena_capacity = want;
            // padding lanes of the NHWC buffers are never written: keep them finite.  The memset runs on
            // the legacy default stream, which the (non-blocking) working streams do not wait for.
            CUDA_OK(cudaMemset(arena, 0, want));
            CUDA_OK(cudaDeviceSynchronize());
        }
        return arena;
    }
};

std::map<int, DeviceContext> g_contexts;   // one per device this process has used

// The device of the calling thread: what this thread last passed to ios_set_device, else the process default.
thread_local int t_device = -1;
int current_device() { return t_device >= 0 ? t_device : g_device; }

// Callers hold g_mutex.
DeviceContext &context(int device) {
    DeviceContext &ctx = g_contexts[device];
    ctx.init(device);
    CUDA_OK(cudaSetDevice(device));
    return ctx;
}
DeviceContext &context() { return context(current_device()); }

// ---- issuing a plan -------------------------------------------------------------------------
void launch_step(const Step &s, cudaStream_t stream) {
    switch (s.kind) {
        case StepKind::SumAct: launch_sum_act(s.sum, s.vec4, stream); break;
        case StepKind::Pool: launch_pool(s.pool, stream); break;
        case StepKind::ConvTc: launch_conv_tc(s.tc, s.tcplan, stream); break;
        case StepKind::ConvDirect: launch_conv_direct(s.direct, stream); break;
        case StepKind::ConvDepthwise: launch_conv_depthwise(s.direct, stream); break;
    }
}

// Issues one forward with data-flow edges instead of stage barriers: group j still runs on stream j
// in schedule order, but an operator only waits for the operators whose outputs it reads (an event
// edge when the producer ran on another stream).  Legal because no buffer of a plan is ever reused:
// read-after-write is the only hazard.  The schedule keeps deciding what is merged and what shares
// a stream; a short branch no longer idles until the longest group of its stage has finished.
void issue_forward_dataflow(StreamSet &ctx, const Plan &plan) {
    ctx.need_streams(plan.max_groups);
    cudaStream_t spine = ctx.streams[0];
    const Model &m = plan.model;
    const int n_ops = int(m.ops.size());
    std::vector<int> stream_of(n_ops, -1), last_step(n_ops, -1);
    for (size_t i = 0; i < plan.steps.size(); ++i) {
        stream_of[plan.steps[i].op] = plan.steps[i].group;
        last_step[plan.steps[i].op] = int(i);
    }
    // producers that launch something, looking through operators that are pure aliases
    std::vector<std::vector<int>> deps(n_ops);
    for (int op = 0; op < n_ops; ++op) {
        for (const Term &term : m.ops[op].inputs)
            for (const ValueRef &v : term) {
                if (last_step[v.node] >= 0) deps[op].push_back(v.node);
                else deps[op].insert(deps[op].end(), deps[v.node].begin(), deps[v.node].end());
            }
    }
    std::vector<char> needs_event(n_ops, 0);
    for (int op = 0; op < n_ops; ++op)
        if (stream_of[op] >= 0)
            for (int d : deps[op])
                if (stream_of[d] != stream_of[op]) needs_event[d] = 1;
    // alias operators (no launch) forward their dependencies to consumers; nothing else to do for them
    size_t ev = 0;
    cudaEvent_t begin = ctx.event(ev++);
    CUDA_OK(cudaEventRecord(begin, spine));
    std::vector<char> started(size_t(plan.max_groups), 0);
    started[0] = 1;
    std::vector<cudaEvent_t> done(size_t(n_ops), nullptr);
    int current = -1;
    for (size_t i = 0; i < plan.steps.size(); ++i) {
        const Step &step = plan.steps[i];
        cudaStream_t stream = ctx.streams[step.group];
        if (step.op != current) {
            current = step.op;
            if (!started[step.group]) {
                CUDA_OK(cudaStreamWaitEvent(stream, begin, 0));
                started[step.group] = 1;
            }
            for (int d : deps[current])
                if (stream_of[d] != step.group && done[d]) CUDA_OK(cudaStreamWaitEvent(stream, done[d], 0));
        }
        launch_step(step, stream);
        if (int(i) == last_step[current] && needs_event[current]) {
            done[current] = ctx.event(ev++);
            CUDA_OK(cudaEventRecord(done[current], stream));
        }
    }
    for (int g = 1; g < plan.max_groups; ++g)
        if (started[g]) {
            cudaEvent_t tail = ctx.event(ev++);
            CUDA_OK(cudaEventRecord(tail, ctx.streams[g]));
            CUDA_OK(cudaStreamWaitEvent(spine, tail, 0));
        }
    CUDA_OK(cudaGetLastError());
}

// Issues one forward on the context's streams.  stage_marks (optional) receives one timing event
// per stage, recorded on stream 0 after the stage's groups have joined.
void issue_forward(StreamSet &ctx, const Plan &plan, const std::vector<cudaEvent_t> *stage_marks) {
    if (!stage_marks && !plan.options.stage_barriers) {
        issue_forward_dataflow(ctx, plan);
        return;
    }
    ctx.need_streams(plan.max_groups);
    cudaStream_t spine = ctx.streams[0];
    size_t next = 0;
    size_t ev = 0;
    const auto &stages = plan.model.stages;
    for (size_t si = 0; si < stages.size(); ++si) {
        const int groups = int(stages[si].size());
        if (groups > 1) {
            cudaEvent_t fork = ctx.event(ev++);
            CUDA_OK(cudaEventRecord(fork, spine));
            for (int g = 1; g < groups; ++g) CUDA_OK(cudaStreamWaitEvent(ctx.streams[g], fork, 0));
        }
        // steps are stored stage by stage, group by group
        for (int g = 0; g < groups; ++g) {
            while (next < plan.steps.size() && plan.steps[next].stage == int(si) && plan.steps[next].group == g) {
                launch_step(plan.steps[next], ctx.streams[g]);
                ++next;
            }
        }
        for (int g = 1; g < groups; ++g) {
            cudaEvent_t done = ctx.event(ev++);
            CUDA_OK(cudaEventRecord(done, ctx.streams[g]));
            CUDA_OK(cudaStreamWaitEvent(spine, done, 0));
        }
        if (stage_marks) CUDA_OK(cudaEventRecord((*stage_marks)[si], spine));
    }
    CUDA_OK(cudaGetLastError());
}

struct GraphExec {
    cudaGraphExec_t exec = nullptr;
    bool programmatic = false;   // its kernel -> kernel edges were all made programmatic
    ~GraphExec() {
        if (exec) cudaGraphExecDestroy(exec);
    }
};

// Turns every full kernel -> kernel dependency of a captured graph into a programmatic one, so that the
// prologue of a kernel (barrier set-up, tensor-memory allocation, the first weight tiles) also overlaps the
// tail of predecessors that ran on OTHER streams -- the fork and join edges of a multi-group stage.  Stream
// capture only makes the edge to the predecessor on the same stream programmatic.  Every kernel of this
// library executes griddepcontrol.wait before it touches memory another kernel writes or reads.
void make_edges_programmatic(cudaGraph_t graph) {
    size_t n = 0;
    CUDA_OK(cudaGraphGetEdges_v2(graph, nullptr, nullptr, nullptr, &n));
    if (n == 0) return;
    std::vector<cudaGraphNode_t> from(n), to(n);
    std::vector<cudaGraphEdgeData> data(n);
    CUDA_OK(cudaGraphGetEdges_v2(graph, from.data(), to.data(), data.data(), &n));
    for (size_t i = 0; i < n; ++i) {
        if (data[i].type != cudaGraphDependencyTypeDefault) continue;
        cudaGraphNodeType tf, tt;
        CUDA_OK(cudaGraphNodeGetType(from[i], &tf));
        CUDA_OK(cudaGraphNodeGetType(to[i], &tt));
        if (tf != cudaGraphNodeTypeKernel || tt != cudaGraphNodeTypeKernel) continue;
        CUDA_OK(cudaGraphRemoveDependencies_v2(graph, &from[i], &to[i], &data[i], 1));
        cudaGraphEdgeData edge = {};
        edge.from_port = cudaGraphKernelNodePortProgrammatic;
        edge.to_port = 0;
        edge.type = cudaGraphDependencyTypeProgrammatic;
        CUDA_OK(cudaGraphAddDependencies_v2(graph, &from[i], &to[i], &edge, 1));
    }
}

template <class F>
void capture(StreamSet &ctx, GraphExec *out, F &&body, bool programmatic_edges = false) {
    cudaStream_t spine = ctx.streams[0];
    cudaGraph_t graph = nullptr;
    CUDA_OK(cudaStreamBeginCapture(spine, cudaStreamCaptureModeThreadLocal));
    try {
        body();
    } catch (...) {
        cudaStreamEndCapture(spine, &graph);
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        throw;
    }
    CUDA_OK(cudaStreamEndCapture(spine, &graph));
    cudaError_t err = cudaErrorUnknown;
    if (programmatic_edges) {
        // on a driver that refuses such a graph the captured edges are kept as they were
        cudaGraph_t upgraded = nullptr;
        if (cudaGraphClone(&upgraded, graph) == cudaSuccess) {
            try {
                make_edges_programmatic(upgraded);
                err = cudaGraphInstantiate(&out->exec, upgraded, 0);
            } catch (const CudaError &) {
                err = cudaErrorUnknown;
            }
            cudaGraphDestroy(upgraded);
            if (err != cudaSuccess) {
                cudaGetLastError();
                out->exec = nullptr;
            } else {
                out->programmatic = true;
            }
        }
    }
    if (err != cudaSuccess) err = cudaGraphInstantiate(&out->exec, graph, 0);
    cudaGraphDestroy(graph);
    CUDA_OK(err);
}

// ---- building a bound plan in the shared arena ---------------------------------------------
struct HostWeights {
    int count = 0;
    char **names = nullptr;
    float **filters = nullptr;
    float **biases = nullptr;
};

void check_error_flag(const Plan &plan, char *base) {
    if (plan.options.timeline) {
        long long stamps[16];
        CUDA_OK(cudaMemcpy(stamps, base + plan.error_flag_offset + 64, sizeof stamps, cudaMemcpyDeviceToHost));
        // (slots 10-12 mean "staged / fenced / stores issued" in the bulk-store epilogue and "partials received / loaded /
        //  first rows stored" in the cluster reduction; 8 and 13-15 are the cluster epilogue's preparation steps)
        std::fprintf(stderr, "conv_tc timeline (SM cycles since entry): setup %lld, first load issued %lld, first tile usable %lld, "
                     "last mma issued %lld, accumulator ready %lld, bias ready %lld, partial handed over %lld, staged|received %lld, "
                     "fenced|loaded %lld, stores issued|first rows stored %lld, epilogue done %lld, tmem freed|preparation begins %lld; "
                     "first chunk loaded|barriers seen %lld, finished|pushes prepared %lld, staged|rows prepared %lld\n",
                     stamps[1] - stamps[0], stamps[2] - stamps[0], stamps[3] - stamps[0], stamps[4] - stamps[0],
                     stamps[5] - stamps[0], stamps[9] - stamps[0], stamps[6] - stamps[0], stamps[10] - stamps[0],
                     stamps[11] - stamps[0], stamps[12] - stamps[0], stamps[7] - stamps[0], stamps[8] - stamps[0],
                     stamps[13] - stamps[0], stamps[14] - stamps[0], stamps[15] - stamps[0]);
    }
    int flag = 0;
    CUDA_OK(cudaMemcpy(&flag, base + plan.error_flag_offset, sizeof flag, cudaMemcpyDeviceToHost));
    if (flag != 0) {
        int where[16] = {0};
        CUDA_OK(cudaMemcpy(where, base + plan.error_flag_offset, sizeof where, cudaMemcpyDeviceToHost));
        std::string detail;
        static const char *roles[] = {"patch loads", "weight loads", "issuer 0", "issuer 1", "issuer 2", "issuer 3", "split", "epilogue"};
        for (int r = 0; r < 8; ++r)
            if (where[1 + r])
                detail += std::string("; ") + roles[r] + " gave up at tile " + std::to_string(where[1 + r] & 0xFFF) + " chunk " +
                          std::to_string((where[1 + r] >> 12) & 63) + " tap " + std::to_string((where[1 + r] >> 18) & 255) + " wait " +
                          std::to_string((where[1 + r] >> 26) & 31);
        CUDA_OK(cudaMemset(base + plan.error_flag_offset, 0, 64));
        // a CTA that gave up never reached its tile's arrival counter: start the next run from zero again
        if (plan.zero_bytes) CUDA_OK(cudaMemset(base + plan.zero_begin, 0, plan.zero_bytes));
        throw TimeoutError("a bounded wait inside the convolution kernel ran out (code " + std::to_string(flag) + ")" + detail);
    }
}

// Packs and uploads (or synthesises) the parameters of every convolution of a bound plan.
void load_parameters(const Plan &plan, char *base, const HostWeights *host, cudaStream_t stream) {
    std::vector<float> packed;
    uint32_t seed = 1;
    for (const ConvSlot &slot : plan.convs) {
        const Op &op = plan.model.ops[slot.op];
        float *w_dev = reinterpret_cast<float *>(base + slot.weight_offset);
        float *b_dev = reinterpret_cast<float *>(base + slot.bias_offset);
        const int fan_in = slot.geom.kh * slot.geom.kw * (slot.geom.Cin / slot.geom.groups);
        const bool bf16_weights = slot.impl == StepKind::ConvTc && slot.tcplan.bf16;
        if (!host) {
            // timing run: bounded pseudo-random parameters keep the activations finite
            launch_fill(w_dev, long(slot.weight_bytes / (bf16_weights ? 2 : 4)), seed++, std::sqrt(3.0f / float(fan_in)), stream,
                        bf16_weights ? 2 : 4);
            launch_fill(b_dev, slot.geom.Cout, seed++, 0.05f, stream);
            continue;
        }
        int found = -1;
        for (int i = 0; i < host->count; ++i)
            if (host->names[i] && op.name == host->names[i]) {
                found = i;
                break;
            }
        if (found < 0 || !host->filters[found] || !host->biases[found])
            throw MissingWeights("convolution '" + op.name + "' was given no weight or bias");
        packed.resize((slot.weight_bytes + 3) / 4);
        switch (slot.impl) {
            case StepKind::ConvTc: conv_tc_pack_weights(host->filters[found], slot.geom, slot.tcplan, packed.data()); break;
            case StepKind::ConvDepthwise: conv_depthwise_pack_weights(host->filters[found], slot.geom, packed.data()); break;
            default: conv_direct_pack_weights(host->filters[found], slot.geom, packed.data()); break;
        }
        CUDA_OK(cudaMemcpyAsync(w_dev, packed.data(), slot.weight_bytes, cudaMemcpyHostToDevice, stream));
        CUDA_OK(cudaStreamSynchronize(stream));   // `packed` is reused for the next convolution
        CUDA_OK(cudaMemcpyAsync(b_dev, host->biases[found], size_t(slot.geom.Cout) * sizeof(float), cudaMemcpyHostToDevice, stream));
    }
    CUDA_OK(cudaStreamSynchronize(stream));
}

// Lays the plan out, binds it to `base` (or to the shared arena when base is null).
char *bind_plan(DeviceContext &ctx, Plan *plan, char *base, StreamSet *streams = nullptr, const Options *options = nullptr) {
    plan->options = options ? *options : g_options;
    plan_layout(plan, ctx.sm_count);
    if (!base) base = ctx.need_arena(plan->arena_bytes);
    plan_bind(plan, base, ctx.sm_count);
    StreamSet &set = streams ? *streams : ctx;
    set.need_streams(plan->max_groups);
    CUDA_OK(cudaMemsetAsync(base + plan->error_flag_offset, 0, 256, set.streams[0]));
    if (plan->zero_bytes) CUDA_OK(cudaMemsetAsync(base + plan->zero_begin, 0, plan->zero_bytes, set.streams[0]));
    return base;
}

void fill_inputs(StreamSet &ctx, const Plan &plan, char *base) {
    uint32_t seed = 1000;
    for (size_t i = 0; i < plan.model.placeholders.size(); ++i) {
        const TensorRef &t = plan.tensors[plan.model.placeholders[i]];
        launch_fill(base + plan.input_offsets[i], t.pixels() * t.pitch, seed++, 1.0f, ctx.streams[0], t.esize);
    }
}

void fill_nan(float *dst, int count) {
    if (!dst) return;
    for (int i = 0; i < count; ++i) dst[i] = std::nanf("");
}

// ---- measurement ----------------------------------------------------------------------------
void measure_graph(const Model &model_in, int warmup, int number, int repeat, bool profile_stage, float *results,
                   float *stage_results) {
    if (!results) throw ArgumentError("results must not be NULL");
    if (number <= 0 || repeat <= 0 || warmup < 0) throw ArgumentError("warmup, number and repeat must be positive");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceContext &ctx = context();
    Plan plan;
    plan.model = model_in;
    char *base = bind_plan(ctx, &plan, nullptr);
    load_parameters(plan, base, nullptr, ctx.streams[0]);
    fill_inputs(ctx, plan, base);
    cudaStream_t spine = ctx.streams[0];
    const size_t num_stages = plan.model.stages.size();

    std::vector<cudaEvent_t> marks;
    GraphExec exec;
    const bool replay = plan.options.use_graph && !profile_stage;
    if (profile_stage) {
        if (!stage_results) throw ArgumentError("stage_results must not be NULL when stages are profiled");
        marks.resize(num_stages);
        for (auto &e : marks) CUDA_OK(cudaEventCreate(&e));
    }
    auto forward = [&]() {
        if (replay) CUDA_OK(cudaGraphLaunch(exec.exec, spine));
        else issue_forward(ctx, plan, profile_stage ? &marks : nullptr);
    };
    try {
        if (replay) capture(ctx, &exec, [&]() { issue_forward(ctx, plan, nullptr); }, plan.options.pdl_edges);
        for (int i = 0; i < warmup; ++i) forward();
        CUDA_OK(cudaDeviceSynchronize());
        check_error_flag(plan, base);
        for (int i = 0; i < repeat; ++i) {
            double total = 0.0;
            std::vector<double> per_stage(num_stages, 0.0);
            for (int t = 0; t < number; ++t) {
                CUDA_OK(cudaDeviceSynchronize());
                CUDA_OK(cudaEventRecord(ctx.t_start, spine));
                forward();
                CUDA_OK(cudaEventRecord(ctx.t_end, spine));
                CUDA_OK(cudaDeviceSynchronize());
                float ms = 0.f;
                CUDA_OK(cudaEventElapsedTime(&ms, ctx.t_start, ctx.t_end));
                total += ms;
                if (profile_stage)
                    for (size_t j = 0; j < num_stages; ++j) {
                        CUDA_OK(cudaEventElapsedTime(&ms, j == 0 ? ctx.t_start : marks[j - 1], marks[j]));
                        per_stage[j] += ms;
                    }
            }
            results[i] = float(total / number);
            if (profile_stage)
                for (size_t j = 0; j < num_stages; ++j) stage_results[size_t(i) * num_stages + j] = float(per_stage[j] / number);
        }
        check_error_flag(plan, base);
    } catch (...) {
        for (auto &e : marks) cudaEventDestroy(e);
        throw;
    }
    for (auto &e : marks) cudaEventDestroy(e);
}

// One candidate stage: `number` repetitions are captured into ONE graph, so a sample measures the
// stage as it will run inside a captured schedule (fork, kernels, join), not a host launch each.
void measure_stage(const Model &model_in, int warmup, int number, int repeat, float *results) {
    if (!results) throw ArgumentError("results must not be NULL");
    if (number <= 0 || repeat <= 0 || warmup < 0) throw ArgumentError("warmup, number and repeat must be positive");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceContext &ctx = context();
    Plan plan;
    plan.model = model_in;
    char *base = bind_plan(ctx, &plan, nullptr);
    load_parameters(plan, base, nullptr, ctx.streams[0]);
    fill_inputs(ctx, plan, base);
    cudaStream_t spine = ctx.streams[0];
    GraphExec exec;
    const bool replay = plan.options.use_graph;
    if (replay) capture(ctx, &exec, [&]() { for (int t = 0; t < number; ++t) issue_forward(ctx, plan, nullptr); }, plan.options.pdl_edges);
    auto sample = [&]() {
        if (replay) CUDA_OK(cudaGraphLaunch(exec.exec, spine));
        else for (int t = 0; t < number; ++t) issue_forward(ctx, plan, nullptr);
    };
    for (int i = 0; i < (warmup + number - 1) / number; ++i) sample();
    for (int i = 0; i < repeat; ++i) {
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaEventRecord(ctx.t_start, spine));
        sample();
        CUDA_OK(cudaEventRecord(ctx.t_end, spine));
        CUDA_OK(cudaDeviceSynchronize());
        float ms = 0.f;
        CUDA_OK(cudaEventElapsedTime(&ms, ctx.t_start, ctx.t_end));
        results[i] = ms / float(number);
    }
    check_error_flag(plan, base);
}

void require_single_group_output(const Model &model) {
    if (!model.output_is_single_group)
        throw GraphError("the last stage must have exactly one group: its last operator is the graph output");
}

void run_inference(const Model &model_in, const float *input, const HostWeights &weights, float *output) {
    if (!input || !output) throw ArgumentError("input and output must not be NULL");
    require_single_group_output(model_in);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceContext &ctx = context();
    Plan plan;
    plan.model = model_in;
    char *base = bind_plan(ctx, &plan, nullptr);
    cudaStream_t spine = ctx.streams[0];
    load_parameters(plan, base, &weights, spine);
    const Op &in_op = plan.model.ops[plan.model.placeholders[0]];
    const Op &out_op = plan.model.ops[plan.model.output];
    const size_t in_bytes = size_t(plan.model.batch) * in_op.C * in_op.H * in_op.W * sizeof(float);
    const size_t out_bytes = size_t(plan.model.batch) * out_op.C * out_op.H * out_op.W * sizeof(float);
    float *stage_in = reinterpret_cast<float *>(base + plan.staging_in_offset);
    float *stage_out = reinterpret_cast<float *>(base + plan.staging_out_offset);
    CUDA_OK(cudaMemcpyAsync(stage_in, input, in_bytes, cudaMemcpyHostToDevice, spine));
    launch_nchw_to_nhwc(stage_in, plan.tensors[plan.model.placeholders[0]], plan.input_round_tf32, spine);
    issue_forward(ctx, plan, nullptr);
    launch_nhwc_to_nchw(plan.tensors[plan.model.output], stage_out, spine);
    CUDA_OK(cudaMemcpyAsync(output, stage_out, out_bytes, cudaMemcpyDeviceToHost, spine));
    CUDA_OK(cudaDeviceSynchronize());
    check_error_flag(plan, base);
}

// ---- status plumbing -------------------------------------------------------------------------
template <class F>
int guarded(F &&body) {
    try {
        body();
        g_last_error.clear();
        return IOS_OK;
    } catch (const JsonError &e) {
        g_last_error = e.what();
        return IOS_ERR_JSON;
    } catch (const GraphError &e) {
        g_last_error = e.what();
        return std::strncmp(e.what(), "limit:", 6) == 0 ? IOS_ERR_LIMIT : IOS_ERR_GRAPH;
    } catch (const ArgumentError &e) {
        g_last_error = e.what();
        return IOS_ERR_ARGUMENT;
    } catch (const TimeoutError &e) {
        g_last_error = e.what();
        return IOS_ERR_TIMEOUT;
    } catch (const MissingWeights &e) {
        g_last_error = e.what();
        return IOS_ERR_MISSING;
    } catch (const CudaError &e) {
        g_last_error = e.what();
        cudaGetLastError();
        return IOS_ERR_CUDA;
    } catch (const std::exception &e) {
        g_last_error = e.what();
        return IOS_ERR_CUDA;
    }
}

}  // namespace

// Lets other translation units of the library report through ios_last_error().
void record_error(const char *message) { g_last_error = message ? message : ""; }

// ---- engine ----------------------------------------------------------------------------------
// A plan bound to memory, streams and events of its own: engines on the same or on different devices run
// side by side from several host threads; a call only takes the engine's own lock.
struct EngineImpl {
    Plan plan;
    int device = 0;
    char *base = nullptr;
    size_t bytes = 0;
    std::mutex mutex;
    StreamSet set;
    GraphExec exec;            // staging -> NHWC, forward, NHWC -> staging
    GraphExec exec_core;       // forward only (resident input)
    size_t in_bytes = 0, out_bytes = 0;
    // host-buffer pipeline: a second staging pair behind the plan's arena, copy streams and their events
    size_t stage_in_off[2] = {0, 0}, stage_out_off[2] = {0, 0};
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t in_ready[2] = {nullptr, nullptr}, in_free[2] = {nullptr, nullptr};
    cudaEvent_t out_ready[2] = {nullptr, nullptr}, out_free[2] = {nullptr, nullptr};
    int *flag_host = nullptr;  // pinned: the time-out word travels with the results, no extra round trip
    std::string graph_text;    // the scheduled graph this engine was built from (kept for ios_engine_save)
    int sm_count = 0;

    ~EngineImpl() {
        cudaSetDevice(device);
        set.release();
        if (copy_in) cudaStreamDestroy(copy_in);
        if (copy_out) cudaStreamDestroy(copy_out);
        for (int i = 0; i < 2; ++i)
            for (cudaEvent_t e : {in_ready[i], in_free[i], out_ready[i], out_free[i]})
                if (e) cudaEventDestroy(e);
        if (flag_host) cudaFreeHost(flag_host);
        if (base) cudaFree(base);
    }
};

}  // namespace ios

struct ios_engine {
    ios::EngineImpl impl;
};

using namespace ios;

// Lays a parsed model out on the current device, allocates and binds it, lets `load` fill in the
// parameters (on the engine's first stream) and captures the schedule.  Callers hold g_mutex.
template <class Load>
static ios_engine *engine_build(const Model &model, const char *graph_json, int batch_size, const Options &options, Load &&load) {
    require_single_group_output(model);
    DeviceContext &ctx = context();
    std::unique_ptr<ios_engine> holder(new ios_engine);
    EngineImpl &e = holder->impl;
    e.device = ctx.device;
    e.sm_count = ctx.sm_count;
    e.graph_text = graph_json;
    e.plan.model = model;
    e.plan.options = options;
    plan_layout(&e.plan, ctx.sm_count);
    const Op &in_op = e.plan.model.ops[e.plan.model.placeholders[0]];
    const Op &out_op = e.plan.model.ops[e.plan.model.output];
    e.in_bytes = size_t(batch_size) * in_op.C * in_op.H * in_op.W * sizeof(float);
    e.out_bytes = size_t(batch_size) * out_op.C * out_op.H * out_op.W * sizeof(float);
    // the plan's arena, then the second staging pair of the host-buffer pipeline
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    e.stage_in_off[1] = up(e.plan.arena_bytes);
    e.stage_out_off[1] = e.stage_in_off[1] + up(e.in_bytes);
    e.bytes = e.stage_out_off[1] + up(e.out_bytes);
    CUDA_OK(cudaMalloc(&e.base, e.bytes));
    CUDA_OK(cudaMemset(e.base, 0, e.bytes));
    CUDA_OK(cudaDeviceSynchronize());      // the working streams do not wait for the default stream
    e.set.init_timers();
    bind_plan(ctx, &e.plan, e.base, &e.set, &options);
    e.stage_in_off[0] = e.plan.staging_in_offset;
    e.stage_out_off[0] = e.plan.staging_out_offset;
    CUDA_OK(cudaStreamCreateWithFlags(&e.copy_in, cudaStreamNonBlocking));
    CUDA_OK(cudaStreamCreateWithFlags(&e.copy_out, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i)
        for (cudaEvent_t *ev : {&e.in_ready[i], &e.in_free[i], &e.out_ready[i], &e.out_free[i]})
            CUDA_OK(cudaEventCreateWithFlags(ev, cudaEventDisableTiming));
    CUDA_OK(cudaHostAlloc(reinterpret_cast<void **>(&e.flag_host), 64, cudaHostAllocDefault));
    e.flag_host[0] = 0;
    cudaStream_t spine = e.set.streams[0];
    load(e, spine);
    fill_inputs(e.set, e.plan, e.base);
    float *stage_in = reinterpret_cast<float *>(e.base + e.stage_in_off[0]);
    float *stage_out = reinterpret_cast<float *>(e.base + e.stage_out_off[0]);
    if (e.plan.options.use_graph) {
        capture(e.set, &e.exec, [&]() {
            launch_nchw_to_nhwc(stage_in, e.plan.tensors[e.plan.model.placeholders[0]], e.plan.input_round_tf32, spine);
            issue_forward(e.set, e.plan, nullptr);
            launch_nhwc_to_nchw(e.plan.tensors[e.plan.model.output], stage_out, spine);
        }, e.plan.options.pdl_edges);
        capture(e.set, &e.exec_core, [&]() { issue_forward(e.set, e.plan, nullptr); }, e.plan.options.pdl_edges);
    }
    CUDA_OK(cudaDeviceSynchronize());
    return holder.release();
}

// ---- engine artefact: scheduled graph + packed parameters + what the tiling was chosen for -------------
namespace {

constexpr char kArtefactMagic[8] = {'I', 'O', 'S', 'E', 'N', 'G', '2', '\0'};

struct FileWriter {
    std::FILE *fh;
    explicit FileWriter(const char *path) : fh(std::fopen(path, "wb")) {
        if (!fh) throw ArgumentError(std::string("cannot open '") + path + "' for writing");
    }
    ~FileWriter() { if (fh) std::fclose(fh); }
    void bytes(const void *data, size_t n) {
        if (n && std::fwrite(data, 1, n, fh) != n) throw ArgumentError("writing the engine artefact failed (disk full?)");
    }
    template <class T> void pod(const T &v) { bytes(&v, sizeof v); }
    void text(const std::string &v) { pod(uint64_t(v.size())); bytes(v.data(), v.size()); }
};

struct FileReader {
    std::FILE *fh;
    explicit FileReader(const char *path) : fh(std::fopen(path, "rb")) {
        if (!fh) throw ArgumentError(std::string("cannot open '") + path + "'");
    }
    ~FileReader() { if (fh) std::fclose(fh); }
    void bytes(void *data, size_t n) {
        if (n && std::fread(data, 1, n, fh) != n) throw ArgumentError("the engine artefact is truncated");
    }
    template <class T> T pod() { T v; bytes(&v, sizeof v); return v; }
    std::string text(size_t limit = size_t(1) << 30) {
        const uint64_t n = pod<uint64_t>();
        if (n > limit) throw ArgumentError("the engine artefact is damaged (a length field is out of range)");
        std::string v(size_t(n), '\0');
        bytes(&v[0], size_t(n));
        return v;
    }
};

// What a convolution's packed parameters depend on: if any of it differs at load time (another library
// version, another GPU, other options), the stored planes would be read with the wrong layout.
struct SlotSignature {
    int32_t impl, bn, cout_pad, cchunks, half_rows, x3, bf16, patch, cout, cin, kh, kw;
    uint64_t weight_bytes;
};

SlotSignature signature_of(const ConvSlot &slot) {
    SlotSignature sig = {};
    sig.impl = int(slot.impl);
    if (slot.impl == StepKind::ConvTc) {
        sig.bn = slot.tcplan.bn; sig.cout_pad = slot.tcplan.cout_pad; sig.cchunks = slot.tcplan.cchunks;
        sig.half_rows = slot.tcplan.half_rows; sig.x3 = slot.tcplan.x3; sig.bf16 = slot.tcplan.bf16; sig.patch = slot.tcplan.patch;
    }
    sig.cout = slot.geom.Cout; sig.cin = slot.geom.Cin; sig.kh = slot.geom.kh; sig.kw = slot.geom.kw;
    sig.weight_bytes = slot.weight_bytes;
    return sig;
}

}  // namespace

extern "C" {

const char *ios_last_error(void) { return g_last_error.c_str(); }

int ios_graph_latency(const char *graph_json, int batch_size, int warmup, int number, int repeat,
                      int profile_stage_latency, float *results, float *stage_results) {
    int status = guarded([&]() {
        Model model = model_from_graph(Json::parse(graph_json), batch_size);
        measure_graph(model, warmup, number, repeat, profile_stage_latency != 0, results, stage_results);
    });
    if (status != IOS_OK && repeat > 0) fill_nan(results, repeat);
    return status;
}

int ios_block_latency(const char *block_json, int batch_size, int warmup, int number, int repeat,
                      int profile_stage_latency, float *results, float *stage_results) {
    int status = guarded([&]() {
        Model model = model_from_block(Json::parse(block_json), batch_size);
        measure_graph(model, warmup, number, repeat, profile_stage_latency != 0, results, stage_results);
    });
    if (status != IOS_OK && repeat > 0) fill_nan(results, repeat);
    return status;
}

int ios_stage_latency(const char *stage_json, const char *input_json, int batch_size, int warmup, int number,
                      int repeat, int profile_stage_latency, float *results, float *stage_results) {
    (void)stage_results;   // the reference never writes it for a stage (src/ios/ios_runtime.cu:1329)
    int status = guarded([&]() {
        if (profile_stage_latency) throw ArgumentError("a single stage cannot be profiled per stage");
        Model model = model_from_stage(Json::parse(stage_json), Json::parse(input_json), batch_size);
        measure_stage(model, warmup, number, repeat, results);
    });
    if (status != IOS_OK && repeat > 0) fill_nan(results, repeat);
    return status;
}

int ios_graph_inference(const char *graph_json, int batch_size, const float *input, int num_convs, char **conv_names,
                        float **filter_data, float **bias_data, float *output) {
    return guarded([&]() {
        if (num_convs < 0 || (num_convs > 0 && (!conv_names || !filter_data || !bias_data)))
            throw ArgumentError("conv_names, filter_data and bias_data must hold num_convs entries");
        Model model = model_from_graph(Json::parse(graph_json), batch_size);
        HostWeights hw{num_convs, conv_names, filter_data, bias_data};
        run_inference(model, input, hw, output);
    });
}

void graph_latency(const char *graph_json, int batch_size, int warmup, int number, int repeat,
                   int profile_stage_latency, float *results, float *stage_results) {
    int status = ios_graph_latency(graph_json, batch_size, warmup, number, repeat, profile_stage_latency, results, stage_results);
    if (status != IOS_OK) std::fprintf(stderr, "ios_runtime: graph_latency failed: %s\n", g_last_error.c_str());
}
void block_latency(const char *block_json, int batch_size, int warmup, int number, int repeat,
                   int profile_stage_latency, float *results, float *stage_results) {
    int status = ios_block_latency(block_json, batch_size, warmup, number, repeat, profile_stage_latency, results, stage_results);
    if (status != IOS_OK) std::fprintf(stderr, "ios_runtime: block_latency failed: %s\n", g_last_error.c_str());
}
void stage_latency(const char *stage_json, const char *input_json, int batch_size, int warmup, int number, int repeat,
                   int profile_stage_latency, float *results, float *stage_results) {
    int status = ios_stage_latency(stage_json, input_json, batch_size, warmup, number, repeat, profile_stage_latency, results, stage_results);
    if (status != IOS_OK) std::fprintf(stderr, "ios_runtime: stage_latency failed: %s\n", g_last_error.c_str());
}
void graph_inference(const char *graph_json, int batch_size, float *input, int num_convs, char **conv_names,
                     float **filter_data, float **bias_data, float *output) {
    int status = ios_graph_inference(graph_json, batch_size, input, num_convs, conv_names, filter_data, bias_data, output);
    if (status != IOS_OK) std::fprintf(stderr, "ios_runtime: graph_inference failed: %s\n", g_last_error.c_str());
}

int ios_set_option(const char *key, const char *value) {
    return guarded([&]() {
        if (!key || !value) throw ArgumentError("key and value must not be NULL");
        std::lock_guard<std::mutex> lock(g_mutex);
        const std::string k = key, v = value;
        if (k == "precision" && (v == "tf32x3" || v == "tf32" || v == "fp32" || v == "bf16")) {
            g_options.bf16 = v == "bf16";
            g_options.tf32 = v == "tf32x3" || v == "tf32";
            g_options.three_pass = v == "tf32x3";
        } else if (k == "pdl" && (v == "0" || v == "1")) g_options.pdl = v == "1";
        else if (k == "executor" && (v == "graph" || v == "streams")) g_options.use_graph = v == "graph";
        else if (k == "conv" && (v == "auto" || v == "direct")) g_options.allow_tc = v == "auto";
        else if (k == "split_k") g_options.force_split_k = std::atoi(value);
        else if (k == "bn") g_options.force_bn = std::atoi(value);
        else if (k == "stages") g_options.force_stages = std::atoi(value);
        else if (k == "producers") g_options.producers = std::atoi(value);
        else if (k == "issuers") g_options.patch_issuers = std::atoi(value);
        else if (k == "patch_store" && (v == "bulk" || v == "direct")) g_options.patch_bulk_store = v == "bulk";
        else if (k == "bulk_store" && (v == "0" || v == "1")) g_options.no_bulk_store = v == "0";
        else if (k == "im2col" && (v == "0" || v == "1")) g_options.no_im2col = v == "0";
        else if (k == "persistent" && (v == "0" || v == "1")) g_options.no_persistent = v == "0";
        else if (k == "cluster_push" && (v == "0" || v == "1")) g_options.no_cluster_push = v == "0";
        else if (k == "dual_issue" && (v == "0" || v == "1")) g_options.no_dual_issue = v == "0";
        else if (k == "weight_prefetch" && (v == "0" || v == "1")) g_options.no_weight_prefetch = v == "0";
        else if (k == "patch" && (v == "0" || v == "1" || v == "all")) {
            g_options.no_patch = v == "0";
            g_options.patch_all = v == "all";
        }
        else if (k == "stem" && (v == "0" || v == "1")) g_options.no_stem_kernel = v == "0";
        else if (k == "half_rows" && (v == "0" || v == "1")) g_options.no_half_rows = v == "0";
        else if (k == "timeline") g_options.timeline = v == "1";
        else if (k == "stage_barriers" && (v == "0" || v == "1")) g_options.stage_barriers = v == "1";
        else if (k == "pdl_edges" && (v == "0" || v == "1")) g_options.pdl_edges = v == "1";
        else throw ArgumentError("unknown option " + k + "=" + v);
    });
}

int ios_get_option(const char *key, char *value, int capacity) {
    return guarded([&]() {
        if (!key || !value || capacity <= 0) throw ArgumentError("key and value must not be NULL");
        std::lock_guard<std::mutex> lock(g_mutex);
        const std::string k = key;
        std::string v;
        if (k == "precision") v = g_options.bf16 ? "bf16" : !g_options.tf32 ? "fp32" : g_options.three_pass ? "tf32x3" : "tf32";
        else if (k == "pdl") v = g_options.pdl ? "1" : "0";
        else if (k == "stage_barriers") v = g_options.stage_barriers ? "1" : "0";
        else if (k == "pdl_edges") v = g_options.pdl_edges ? "1" : "0";
        else if (k == "bulk_store") v = g_options.no_bulk_store ? "0" : "1";
        else if (k == "persistent") v = g_options.no_persistent ? "0" : "1";
        else if (k == "cluster_push") v = g_options.no_cluster_push ? "0" : "1";
        else if (k == "dual_issue") v = g_options.no_dual_issue ? "0" : "1";
        else if (k == "weight_prefetch") v = g_options.no_weight_prefetch ? "0" : "1";
        else if (k == "patch") v = g_options.no_patch ? "0" : g_options.patch_all ? "all" : "1";
        else if (k == "executor") v = g_options.use_graph ? "graph" : "streams";
        else if (k == "conv") v = g_options.allow_tc ? "auto" : "direct";
        else if (k == "split_k") v = std::to_string(g_options.force_split_k);
        else throw ArgumentError("unknown option " + k);
        std::snprintf(value, size_t(capacity), "%s", v.c_str());
    });
}

int ios_set_device(int device) {
    return guarded([&]() {
        std::lock_guard<std::mutex> lock(g_mutex);
        int count = 0;
        CUDA_OK(cudaGetDeviceCount(&count));
        if (device < 0 || device >= count) throw ArgumentError("device index out of range");
        g_device = device;      // the default of threads that never chose one
        t_device = device;      // what this thread uses from now on
    });
}

int ios_device_count(int *count) {
    return guarded([&]() {
        if (!count) throw ArgumentError("count must not be NULL");
        CUDA_OK(cudaGetDeviceCount(count));
    });
}

int ios_host_register(void *memory, size_t bytes) {
    return guarded([&]() {
        if (!memory || bytes == 0) throw ArgumentError("memory must not be NULL and bytes > 0");
        CUDA_OK(cudaHostRegister(memory, bytes, cudaHostRegisterPortable));
    });
}

int ios_host_unregister(void *memory) {
    return guarded([&]() {
        if (!memory) throw ArgumentError("memory must not be NULL");
        CUDA_OK(cudaHostUnregister(memory));
    });
}

int ios_engine_create(const char *graph_json, int batch_size, int num_convs, char **conv_names, float **filter_data,
                      float **bias_data, ios_engine **engine) {
    return guarded([&]() {
        if (!engine) throw ArgumentError("engine must not be NULL");
        *engine = nullptr;
        Model model = model_from_graph(Json::parse(graph_json), batch_size);
        std::lock_guard<std::mutex> lock(g_mutex);
        const Options options = g_options;
        *engine = engine_build(model, graph_json, batch_size, options, [&](EngineImpl &e, cudaStream_t spine) {
            if (filter_data && bias_data && conv_names) {
                HostWeights hw{num_convs, conv_names, filter_data, bias_data};
                load_parameters(e.plan, e.base, &hw, spine);
            } else {
                load_parameters(e.plan, e.base, nullptr, spine);
            }
        });
    });
}

int ios_engine_save(ios_engine *engine, const char *path) {
    return guarded([&]() {
        if (!engine || !path) throw ArgumentError("engine and path must not be NULL");
        EngineImpl &e = engine->impl;
        std::lock_guard<std::mutex> lock(e.mutex);
        CUDA_OK(cudaSetDevice(e.device));
        CUDA_OK(cudaStreamSynchronize(e.set.streams[0]));
        FileWriter out(path);
        out.bytes(kArtefactMagic, sizeof kArtefactMagic);
        out.pod(uint32_t(sizeof(Options)));
        out.pod(e.plan.options);
        out.pod(int32_t(e.sm_count));
        out.pod(int32_t(e.plan.model.batch));
        out.text(e.graph_text);
        out.pod(uint32_t(e.plan.convs.size()));
        std::vector<char> blob;
        for (const ConvSlot &slot : e.plan.convs) {
            out.text(e.plan.model.ops[size_t(slot.op)].name);
            out.pod(signature_of(slot));
            blob.resize(slot.weight_bytes);
            CUDA_OK(cudaMemcpy(blob.data(), e.base + slot.weight_offset, slot.weight_bytes, cudaMemcpyDeviceToHost));
            out.bytes(blob.data(), blob.size());
            blob.resize(size_t(slot.geom.Cout) * sizeof(float));
            CUDA_OK(cudaMemcpy(blob.data(), e.base + slot.bias_offset, blob.size(), cudaMemcpyDeviceToHost));
            out.bytes(blob.data(), blob.size());
        }
        out.bytes(kArtefactMagic, sizeof kArtefactMagic);      // end mark: a truncated file is recognised
    });
}

int ios_engine_load(const char *path, ios_engine **engine) {
    return guarded([&]() {
        if (!engine || !path) throw ArgumentError("path and engine must not be NULL");
        *engine = nullptr;
        FileReader in(path);
        char magic[8];
        in.bytes(magic, sizeof magic);
        if (std::memcmp(magic, kArtefactMagic, sizeof magic) != 0) throw ArgumentError("not an engine artefact of this library version");
        if (in.pod<uint32_t>() != sizeof(Options)) throw ArgumentError("the engine artefact was written with another option block");
        const Options options = in.pod<Options>();
        const int sm_count = in.pod<int32_t>();
        const int batch = in.pod<int32_t>();
        const std::string graph_text = in.text();
        Model model = model_from_graph(Json::parse(graph_text.c_str()), batch);
        std::lock_guard<std::mutex> lock(g_mutex);
        if (context().sm_count != sm_count)
            throw ArgumentError("the engine artefact was tiled for a GPU with " + std::to_string(sm_count) + " SMs, this one has " +
                                std::to_string(context().sm_count));
        *engine = engine_build(model, graph_text.c_str(), batch, options, [&](EngineImpl &e, cudaStream_t spine) {
            if (in.pod<uint32_t>() != e.plan.convs.size()) throw ArgumentError("the engine artefact holds another number of convolutions");
            std::vector<char> blob;
            for (const ConvSlot &slot : e.plan.convs) {
                const std::string name = in.text(4096);
                const SlotSignature stored = in.pod<SlotSignature>(), now = signature_of(slot);
                if (name != e.plan.model.ops[size_t(slot.op)].name || std::memcmp(&stored, &now, sizeof now) != 0)
                    throw ArgumentError("the engine artefact does not match the plan this library builds for convolution '" + name +
                                        "' (another library version or other options)");
                blob.resize(slot.weight_bytes);
                in.bytes(blob.data(), blob.size());
                CUDA_OK(cudaMemcpyAsync(e.base + slot.weight_offset, blob.data(), blob.size(), cudaMemcpyHostToDevice, spine));
                CUDA_OK(cudaStreamSynchronize(spine));          // `blob` is reused
                blob.resize(size_t(slot.geom.Cout) * sizeof(float));
                in.bytes(blob.data(), blob.size());
                CUDA_OK(cudaMemcpyAsync(e.base + slot.bias_offset, blob.data(), blob.size(), cudaMemcpyHostToDevice, spine));
                CUDA_OK(cudaStreamSynchronize(spine));
            }
            char tail[8];
            in.bytes(tail, sizeof tail);
            if (std::memcmp(tail, kArtefactMagic, sizeof tail) != 0) throw ArgumentError("the engine artefact is damaged (no end mark)");
        });
    });
}

int ios_engine_destroy(ios_engine *engine) {
    return guarded([&]() {
        if (!engine) return;
        {
            std::lock_guard<std::mutex> lock(engine->impl.mutex);
            cudaSetDevice(engine->impl.device);
            cudaDeviceSynchronize();
        }
        delete engine;
    });
}

static void engine_forward(EngineImpl &e, bool with_layout) {
    cudaStream_t spine = e.set.streams[0];
    float *stage_in = reinterpret_cast<float *>(e.base + e.stage_in_off[0]);
    float *stage_out = reinterpret_cast<float *>(e.base + e.stage_out_off[0]);
    if (e.plan.options.use_graph) {
        CUDA_OK(cudaGraphLaunch(with_layout ? e.exec.exec : e.exec_core.exec, spine));
        return;
    }
    if (with_layout)
        launch_nchw_to_nhwc(stage_in, e.plan.tensors[e.plan.model.placeholders[0]], e.plan.input_round_tf32, spine);
    issue_forward(e.set, e.plan, nullptr);
    if (with_layout) launch_nhwc_to_nchw(e.plan.tensors[e.plan.model.output], stage_out, spine);
}

// The time-out word rides behind the results: an asynchronous copy into pinned memory on the stream
// that was just used, read after the stream has been synchronised.
static void engine_fetch_flag(EngineImpl &e, cudaStream_t stream) {
    CUDA_OK(cudaMemcpyAsync(e.flag_host, e.base + e.plan.error_flag_offset, sizeof(int), cudaMemcpyDeviceToHost, stream));
}
static void engine_check_flag(EngineImpl &e) {
    if (e.flag_host[0] != 0 || e.plan.options.timeline) check_error_flag(e.plan, e.base);
}

int ios_engine_run(ios_engine *engine, const float *input, float *output) {
    return guarded([&]() {
        if (!engine || !input || !output) throw ArgumentError("engine, input and output must not be NULL");
        EngineImpl &e = engine->impl;
        std::lock_guard<std::mutex> lock(e.mutex);
        CUDA_OK(cudaSetDevice(e.device));
        cudaStream_t spine = e.set.streams[0];
        CUDA_OK(cudaMemcpyAsync(e.base + e.stage_in_off[0], input, e.in_bytes, cudaMemcpyHostToDevice, spine));
        engine_forward(e, true);
        CUDA_OK(cudaMemcpyAsync(output, e.base + e.stage_out_off[0], e.out_bytes, cudaMemcpyDeviceToHost, spine));
        engine_fetch_flag(e, spine);
        CUDA_OK(cudaStreamSynchronize(spine));
        engine_check_flag(e);
    });
}

int ios_engine_run_pipelined(ios_engine *engine, int count, const float *const *inputs, float *const *outputs) {
    return guarded([&]() {
        if (!engine || count < 0 || (count > 0 && (!inputs || !outputs)))
            throw ArgumentError("engine, inputs and outputs must not be NULL and count >= 0");
        for (int i = 0; i < count; ++i)
            if (!inputs[i] || !outputs[i]) throw ArgumentError("every input and output pointer must not be NULL");
        if (count == 0) return;
        EngineImpl &e = engine->impl;
        std::lock_guard<std::mutex> lock(e.mutex);
        CUDA_OK(cudaSetDevice(e.device));
        cudaStream_t spine = e.set.streams[0];
        const TensorRef &in_t = e.plan.tensors[e.plan.model.placeholders[0]];
        const TensorRef &out_t = e.plan.tensors[e.plan.model.output];
        // Batch i uses staging pair i % 2.  Three streams: uploads, the forward (layout kernels and the
        // captured schedule), downloads.  An upload may overwrite its staging buffer once the layout kernel
        // of batch i - 2 has read it; a layout kernel may overwrite the output staging once the download
        // of batch i - 2 has read it.  So the upload of batch i + 1 and the download of batch i - 1 run
        // beside the forward of batch i.
        CUDA_OK(cudaEventRecord(e.in_free[0], spine));      // everything issued earlier on the spine is ordered before
        CUDA_OK(cudaStreamWaitEvent(e.copy_in, e.in_free[0], 0));
        for (int i = 0; i < count; ++i) {
            const int b = i & 1;
            float *stage_in = reinterpret_cast<float *>(e.base + e.stage_in_off[b]);
            float *stage_out = reinterpret_cast<float *>(e.base + e.stage_out_off[b]);
            if (i >= 2) CUDA_OK(cudaStreamWaitEvent(e.copy_in, e.in_free[b], 0));
            CUDA_OK(cudaMemcpyAsync(stage_in, inputs[i], e.in_bytes, cudaMemcpyHostToDevice, e.copy_in));
            CUDA_OK(cudaEventRecord(e.in_ready[b], e.copy_in));
            CUDA_OK(cudaStreamWaitEvent(spine, e.in_ready[b], 0));
            launch_nchw_to_nhwc(stage_in, in_t, e.plan.input_round_tf32, spine);
            CUDA_OK(cudaEventRecord(e.in_free[b], spine));
            if (e.plan.options.use_graph) CUDA_OK(cudaGraphLaunch(e.exec_core.exec, spine));
            else issue_forward(e.set, e.plan, nullptr);
            if (i >= 2) CUDA_OK(cudaStreamWaitEvent(spine, e.out_free[b], 0));
            launch_nhwc_to_nchw(out_t, stage_out, spine);
            CUDA_OK(cudaEventRecord(e.out_ready[b], spine));
            CUDA_OK(cudaStreamWaitEvent(e.copy_out, e.out_ready[b], 0));
            CUDA_OK(cudaMemcpyAsync(outputs[i], stage_out, e.out_bytes, cudaMemcpyDeviceToHost, e.copy_out));
            CUDA_OK(cudaEventRecord(e.out_free[b], e.copy_out));
        }
        engine_fetch_flag(e, e.copy_out);
        CUDA_OK(cudaStreamSynchronize(e.copy_out));
        CUDA_OK(cudaStreamSynchronize(spine));
        engine_check_flag(e);
    });
}

int ios_engine_set_input(ios_engine *engine, const float *input) {
    return guarded([&]() {
        if (!engine || !input) throw ArgumentError("engine and input must not be NULL");
        EngineImpl &e = engine->impl;
        std::lock_guard<std::mutex> lock(e.mutex);
        CUDA_OK(cudaSetDevice(e.device));
        cudaStream_t spine = e.set.streams[0];
        float *stage_in = reinterpret_cast<float *>(e.base + e.stage_in_off[0]);
        CUDA_OK(cudaMemcpyAsync(stage_in, input, e.in_bytes, cudaMemcpyHostToDevice, spine));
        launch_nchw_to_nhwc(stage_in, e.plan.tensors[e.plan.model.placeholders[0]], e.plan.input_round_tf32, spine);
        CUDA_OK(cudaStreamSynchronize(spine));
    });
}

int ios_engine_get_output(ios_engine *engine, float *output) {
    return guarded([&]() {
        if (!engine || !output) throw ArgumentError("engine and output must not be NULL");
        EngineImpl &e = engine->impl;
        std::lock_guard<std::mutex> lock(e.mutex);
        CUDA_OK(cudaSetDevice(e.device));
        cudaStream_t spine = e.set.streams[0];
        float *stage_out = reinterpret_cast<float *>(e.base + e.stage_out_off[0]);
        launch_nhwc_to_nchw(e.plan.tensors[e.plan.model.output], stage_out, spine);
        CUDA_OK(cudaMemcpyAsync(output, stage_out, e.out_bytes, cudaMemcpyDeviceToHost, spine));
        engine_fetch_flag(e, spine);
        CUDA_OK(cudaStreamSynchronize(spine));
        engine_check_flag(e);
    });
}

int ios_engine_time(ios_engine *engine, int iters, float *ms_per_iter) {
    return guarded([&]() {
        if (!engine || !ms_per_iter || iters <= 0) throw ArgumentError("engine, ms_per_iter must not be NULL and iters > 0");
        EngineImpl &e = engine->impl;
        std::lock_guard<std::mutex> lock(e.mutex);
        CUDA_OK(cudaSetDevice(e.device));
        cudaStream_t spine = e.set.streams[0];
        CUDA_OK(cudaStreamSynchronize(spine));
        CUDA_OK(cudaEventRecord(e.set.t_start, spine));
        for (int i = 0; i < iters; ++i) engine_forward(e, false);
        CUDA_OK(cudaEventRecord(e.set.t_end, spine));
        engine_fetch_flag(e, spine);
        CUDA_OK(cudaStreamSynchronize(spine));
        float ms = 0.f;
        CUDA_OK(cudaEventElapsedTime(&ms, e.set.t_start, e.set.t_end));
        *ms_per_iter = ms / float(iters);
        engine_check_flag(e);
    });
}

int ios_engine_profile(ios_engine *engine, int iters, int capacity, int *count, float *step_ms, int *step_kind,
                       double *step_work) {
    return guarded([&]() {
        if (!engine || !count || !step_ms || !step_kind || !step_work || iters <= 0)
            throw ArgumentError("engine and the output arrays must not be NULL and iters > 0");
        EngineImpl &e = engine->impl;
        std::lock_guard<std::mutex> lock(e.mutex);
        CUDA_OK(cudaSetDevice(e.device));
        StreamSet &ctx = e.set;
        cudaStream_t spine = ctx.streams[0];
        const int n = int(e.plan.steps.size());
        *count = n;
        if (capacity < n) throw ArgumentError("capacity is smaller than the number of launches");
        // All launches of one kind are captured, one after another on a single stream, into a graph
        // of their own; the graph's device time divided by its launch count is what every launch
        // of that kind is credited with.  (No host launch cost, no timing nodes between kernels.)
        for (int i = 0; i < n; ++i) step_ms[i] = 0.f;
        for (int kind = 0; kind < 5; ++kind) {
            std::vector<int> members;
            for (int i = 0; i < n; ++i)
                if (int(e.plan.steps[i].kind) == kind) members.push_back(i);
            if (members.empty()) continue;
            auto issue = [&]() { for (int i : members) launch_step(e.plan.steps[i], spine); };
            GraphExec serial;
            const bool replay = e.plan.options.use_graph;
            if (replay) capture(ctx, &serial, issue);
            float total = 0.f;
            for (int it = 0; it < iters + 1; ++it) {       // the first pass is a warm-up
                CUDA_OK(cudaStreamSynchronize(spine));
                CUDA_OK(cudaEventRecord(ctx.t_start, spine));
                if (replay) CUDA_OK(cudaGraphLaunch(serial.exec, spine));
                else issue();
                CUDA_OK(cudaEventRecord(ctx.t_end, spine));
                CUDA_OK(cudaStreamSynchronize(spine));
                float ms = 0.f;
                CUDA_OK(cudaEventElapsedTime(&ms, ctx.t_start, ctx.t_end));
                if (it > 0) total += ms;
            }
            for (int i : members) step_ms[i] = total / float(iters) / float(members.size());
        }
        for (int i = 0; i < n; ++i) {
            const Step &s = e.plan.steps[i];
            step_kind[i] = int(s.kind);
            switch (s.kind) {
                case StepKind::SumAct:
                    step_work[i] = double(s.sum.k + 1) * double(s.sum.pixels) * s.sum.C * double(s.sum.esize);
                    break;
                case StepKind::Pool:
                    step_work[i] = (double(s.pool.in.pixels()) + double(s.pool.out.pixels())) * s.pool.in.C * double(s.pool.in.esize);
                    break;
                case StepKind::ConvDepthwise: {
                    const ConvGeom &g = s.direct.g;
                    step_work[i] = (double(g.N) * g.H * g.W * g.Cin + double(g.N) * g.OH * g.OW * g.Cout) * double(s.direct.in.esize) +
                                   double(g.kh) * g.kw * g.Cout * 4.0;
                    break;
                }
                default: {
                    const ConvGeom &g = s.kind == StepKind::ConvTc ? s.tc.g : s.direct.g;
                    step_work[i] = 2.0 * g.N * g.OH * g.OW * double(g.Cout) * g.kh * g.kw * (g.Cin / g.groups);
                }
            }
        }
        check_error_flag(e.plan, e.base);
    });
}

int ios_plan_describe(const char *graph_json, int batch_size, int sm_count, char *text, int capacity) {
    return guarded([&]() {
        if (!graph_json || !text || capacity <= 0 || batch_size <= 0) throw ArgumentError("graph_json and text must not be NULL, batch_size > 0");
        Plan plan;
        plan.model = model_from_graph(Json::parse(graph_json), batch_size);
        {
            std::lock_guard<std::mutex> lock(g_mutex);
            plan.options = g_options;
        }
        plan_layout(&plan, sm_count > 0 ? sm_count : 148);        // sizes and tilings only: no device is touched
        std::string out = "{\"arena_bytes\": " + std::to_string(plan.arena_bytes) + ", \"launches\": " +
                          std::to_string(plan.launches_per_forward) + ", \"convolutions\": [";
        bool first = true;
        for (const Step &s : plan.steps) {
            if (s.kind != StepKind::ConvTc && s.kind != StepKind::ConvDirect && s.kind != StepKind::ConvDepthwise) continue;
            const ConvGeom &g = s.kind == StepKind::ConvTc ? s.tc.g : s.direct.g;
            char line[640];
            if (s.kind == StepKind::ConvTc) {
                const ConvTcPlan &q = s.tcplan;
                std::snprintf(line, sizeof line,
                              "{\"op\": \"%s\", \"kind\": \"tensor\", \"cin\": %d, \"cout\": %d, \"kh\": %d, \"kw\": %d, \"oh\": %d, \"ow\": %d, "
                              "\"bn\": %d, \"n_tiles\": %d, \"k_iters\": %d, \"split_k\": %d, \"cluster\": %d, \"push\": %d, \"recv_off\": %d, "
                              "\"stages\": %d, \"smem_bytes\": %zu, \"workspace_bytes\": %zu, \"persistent\": %d, \"patch\": %d, \"grid_ctas\": %d, "
                              "\"x3\": %d, \"bf16\": %d, \"half_rows\": %d}",
                              plan.model.ops[s.op].name.c_str(), g.Cin, g.Cout, g.kh, g.kw, g.OH, g.OW, q.bn, q.n_tiles, q.k_iters, q.split_k,
                              q.cluster, q.push, q.recv_off, q.stages, q.smem_bytes, q.workspace_bytes, q.persistent, q.patch, q.grid_ctas,
                              q.x3, q.bf16, q.half_rows);
            } else {
                std::snprintf(line, sizeof line, "{\"op\": \"%s\", \"kind\": \"%s\", \"cin\": %d, \"cout\": %d, \"kh\": %d, \"kw\": %d}",
                              plan.model.ops[s.op].name.c_str(), s.kind == StepKind::ConvDirect ? "cuda_core" : "depthwise", g.Cin, g.Cout,
                              g.kh, g.kw);
            }
            out += (first ? "" : ", ") + std::string(line);
            first = false;
        }
        out += "]}";
        if (int(out.size()) + 1 > capacity) throw ArgumentError("capacity is too small for the description (" + std::to_string(out.size() + 1) + " bytes)");
        std::memcpy(text, out.c_str(), out.size() + 1);
    });
}

int ios_engine_describe(ios_engine *engine, char *text, int capacity) {
    return guarded([&]() {
        if (!engine || !text || capacity <= 0) throw ArgumentError("engine and text must not be NULL");
        const EngineImpl &e = engine->impl;
        const Plan &p = e.plan;
        int n_tc = 0, n_direct = 0, n_dw = 0, n_sum = 0, n_pool = 0, n_split = 0, n_persistent = 0, n_half = 0, n_few = 0,
            n_direct_store = 0, n_patch = 0, n_push = 0;
        for (const Step &s : p.steps) {
            switch (s.kind) {
                case StepKind::ConvTc:
                    ++n_tc;
                    if (s.tcplan.split_k > 1) ++n_split;
                    if (s.tcplan.split_k > 1 && s.tcplan.cluster && s.tcplan.push) ++n_push;
                    if (s.tcplan.persistent) ++n_persistent;
                    if (s.tcplan.patch) ++n_patch;
                    if (s.tcplan.half_rows) ++n_half;
                    if (!s.tcplan.tma_store) ++n_direct_store;
                    break;
                case StepKind::ConvDirect:
                    ++n_direct;
                    if (conv_few_channels_supported(s.direct.in, s.direct.out, s.direct.g)) ++n_few;
                    break;
                case StepKind::ConvDepthwise: ++n_dw; break;
                case StepKind::SumAct: ++n_sum; break;
                case StepKind::Pool: ++n_pool; break;
            }
        }
        size_t weight_bytes = 0;
        for (const ConvSlot &c : p.convs) weight_bytes += c.weight_bytes + c.geom.Cout * sizeof(float);
        const Op &out = p.model.ops[p.model.output];
        const Op &in = p.model.ops[p.model.placeholders[0]];
        std::snprintf(text, size_t(capacity),
                      "{\"launches\": %d, \"conv_tc\": %d, \"conv_tc_split_k\": %d, \"conv_tc_cluster_push\": %d, \"conv_tc_persistent\": %d, "
                      "\"conv_tc_half_rows\": %d, \"conv_tc_patch\": %d, \"conv_tc_direct_store\": %d, \"conv_direct\": %d, \"conv_few_channels\": %d, "
                      "\"conv_depthwise\": %d, "
                      "\"sum_act\": %d, \"pool\": %d, \"stages\": %zu, \"arena_bytes\": %zu, \"workspace_bytes\": %zu, "
                      "\"weight_bytes\": %zu, \"conv_flops\": %.0f, \"output_shape\": [%d, %d, %d, %d], \"input_shape\": [%d, %d, %d, %d], \"executor\": \"%s\", "
                      "\"stage_barriers\": %d, \"pdl_edges\": %d, \"pdl_edges_applied\": %d, \"device\": %d, \"precision\": \"%s\"}",
                      p.launches_per_forward, n_tc, n_split, n_push, n_persistent, n_half, n_patch, n_direct_store, n_direct, n_few, n_dw, n_sum,
                      n_pool, p.model.stages.size(), e.bytes,
                      p.workspace_bytes, weight_bytes, p.model.conv_flops(), p.model.batch, out.C, out.H, out.W,
                      p.model.batch, in.C, in.H, in.W,
                      p.options.use_graph ? "graph" : "streams", p.options.stage_barriers ? 1 : 0, p.options.pdl_edges ? 1 : 0,
                      e.exec_core.programmatic ? 1 : 0, e.device,
                      p.options.bf16 ? "bf16" : !p.options.tf32 ? "fp32" : p.options.three_pass ? "tf32x3" : "tf32");
    });
}

int ios_conv2d(const float *x, const float *w, const float *bias, float *y, int n, int cin, int h, int wdt, int cout,
               int kh, int kw, int sh, int sw, int ph, int pw, int groups, int act, int impl) {
    return guarded([&]() {
        if (!x || !w || !y) throw ArgumentError("x, w and y must not be NULL");
        if (n <= 0 || cin <= 0 || h <= 0 || wdt <= 0 || cout <= 0 || groups <= 0 || act < 0 || act > 3 || impl < 0 || impl > 4)
            throw ArgumentError("bad convolution arguments");
        // a one-operator graph drives exactly the code path a scheduled convolution takes
        static const char *acts[] = {"identity", "relu", "sigmoid", "tanh"};
        char json[1024];
        std::snprintf(json, sizeof json,
                      "{\"name\":\"conv2d\",\"input\":{\"type\":\"placeholder\",\"name\":\"x\",\"hint_name\":\"x\",\"output_shape\":[%d,%d,%d]},"
                      "\"blocks\":[{\"enter_name\":\"x\",\"enter_node\":{},\"inner_nodes\":[],\"exit_node\":{\"type\":\"conv\",\"name\":\"y\","
                      "\"hint_name\":\"y\",\"inputs\":[[[\"x\",0,%d]]],\"out_channels\":%d,\"kernel\":[%d,%d],\"stride\":[%d,%d],"
                      "\"padding\":[%d,%d],\"groups\":%d,\"act\":\"%s\",\"output_shape\":null},\"stages\":[[[\"y\"]]]}]}",
                      cin, h, wdt, cin, cout, kh, kw, sh, sw, ph, pw, groups, acts[act]);
        Model model = model_from_graph(Json::parse(json), n);
        std::vector<float> zero_bias;
        if (!bias) zero_bias.assign(size_t(cout), 0.0f);
        char name[] = "y";
        char *names[1] = {name};
        float *filters[1] = {const_cast<float *>(w)};
        float *biases[1] = {bias ? const_cast<float *>(bias) : zero_bias.data()};
        HostWeights hw{1, names, filters, biases};
        Options saved;
        {
            std::lock_guard<std::mutex> lock(g_mutex);
            saved = g_options;
            if (impl == 1) g_options.allow_tc = false;
            if (impl == 2) { g_options.allow_tc = true; if (!g_options.bf16) g_options.tf32 = true; }
            if (impl == 3) { g_options.allow_tc = true; g_options.tf32 = true; g_options.three_pass = false; g_options.bf16 = false; }
            if (impl == 4) { g_options.allow_tc = true; g_options.bf16 = true; g_options.tf32 = false; }
        }
        try {
            run_inference(model, x, hw, y);
        } catch (...) {
            std::lock_guard<std::mutex> lock(g_mutex);
            g_options = saved;
            throw;
        }
        std::lock_guard<std::mutex> lock(g_mutex);
        g_options = saved;
    });
}

}  // extern "C"
