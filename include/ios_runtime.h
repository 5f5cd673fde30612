/*
 * C-ABI of libios_runtime.so, the B200-native execution engine for IOS schedules.
 *
 * The first four symbols are exactly what the reference's ctypes front-end binds
 * (python/ios/contrib/ios_runtime.py:18-23 loads the library, :33, :63, :101, :124 call them) and
 * keep the reference's signatures (src/ios/ios_runtime.cu:1480-1502).  They return nothing; on an
 * error they fill their float outputs with NaN and record a message readable through
 * ios_last_error().  Every other entry point returns an int status (0 = IOS_OK).
 *
 * All pointers are owned by the caller and only have to stay valid for the duration of the call.
 * Tensors at this boundary are float32, NCHW, batch-major, C-contiguous; convolution weights are
 * OIHW (Cout, Cin/groups, kh, kw) and biases (Cout).  JSON arguments follow the wire format of
 * python/ios/ir.py (Graph.export_config, Block.export_config, Node.export_config).
 */
#ifndef IOS_RUNTIME_H_
#define IOS_RUNTIME_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IOS_API __attribute__((visibility("default")))

enum {
    IOS_OK = 0,
    IOS_ERR_JSON = 1,       /* malformed JSON text */
    IOS_ERR_GRAPH = 2,      /* well-formed JSON that is not a valid graph / block / stage */
    IOS_ERR_ARGUMENT = 3,   /* bad argument (NULL pointer, non-positive count, unknown option) */
    IOS_ERR_CUDA = 4,       /* a CUDA runtime or driver call failed */
    IOS_ERR_TIMEOUT = 5,    /* a bounded device-side wait ran out */
    IOS_ERR_LIMIT = 6,      /* a stated size limit was exceeded */
    IOS_ERR_MISSING = 7     /* a convolution was given no weights */
};

/* ---- drop-in symbols (reference src/ios/ios_runtime.cu:1480, :1486, :1492, :1500) ---------- */

/* Time a whole graph: results[repeat] (ms, each the mean of `number` forwards) and, when
 * profile_stage_latency != 0, stage_results[repeat * num_stages] row-major. */
IOS_API void graph_latency(const char *graph_json, int batch_size, int warmup, int number, int repeat,
                           int profile_stage_latency, float *results, float *stage_results);
/* Same for one block; its enter node becomes the input. */
IOS_API void block_latency(const char *block_json, int batch_size, int warmup, int number, int repeat,
                           int profile_stage_latency, float *results, float *stage_results);
/* Time one candidate stage: stage_json = [[node config, ...], ...] (groups x operators),
 * input_json = {producer name: [C, H, W]}.  results[repeat]; stage_results is not written. */
IOS_API void stage_latency(const char *stage_json, const char *input_json, int batch_size, int warmup,
                           int number, int repeat, int profile_stage_latency, float *results,
                           float *stage_results);
/* Run a graph once on host data: uploads input and weights, executes the schedule, downloads the
 * exit node of the last block into output[batch, C, H, W]. */
IOS_API void graph_inference(const char *graph_json, int batch_size, float *input, int num_convs,
                             char **conv_names, float **filter_data, float **bias_data, float *output);

/* ---- status-returning twins of the four symbols above (same arguments) --------------------- */
IOS_API int ios_graph_latency(const char *graph_json, int batch_size, int warmup, int number, int repeat,
                              int profile_stage_latency, float *results, float *stage_results);
IOS_API int ios_block_latency(const char *block_json, int batch_size, int warmup, int number, int repeat,
                              int profile_stage_latency, float *results, float *stage_results);
IOS_API int ios_stage_latency(const char *stage_json, const char *input_json, int batch_size, int warmup,
                              int number, int repeat, int profile_stage_latency, float *results,
                              float *stage_results);
IOS_API int ios_graph_inference(const char *graph_json, int batch_size, const float *input, int num_convs,
                                char **conv_names, float **filter_data, float **bias_data, float *output);

/* Message of the calling thread's most recent failure ("" if none).  Replaces the reference's
 * FatalError -> exit(1) (include/utils/utils.h:8-14): the library never terminates the process. */
IOS_API const char *ios_last_error(void);

/* ---- run-time options (replace the reference's compile-time switches, config.cmake:8-17) ----
 * key "precision": "tf32x3" (default; fp32 storage, every product formed from three TF32 tensor-core
 *                  products of value/residual operand pairs, fp32 accumulate: fp32-grade results),
 *                  "tf32" (one TF32 product per multiply: fastest, about 3e-4 relative error per layer),
 *                  "bf16" (activations and weights stored as bfloat16, bf16 tensor-core products, fp32
 *                  accumulate: half the memory traffic and twice the tensor rate, about 1e-2 relative error),
 *                  "fp32" (CUDA-core fp32 products, the slow exact path)
 * key "executor":  "graph" (default; a schedule is captured once into a CUDA graph),
 *                  "streams" (group j of every stage is launched on stream j, events between stages)
 * key "conv":      "auto" (default), "direct" (never use the tensor-core kernel)
 * key "pdl":       "1" (default; consecutive convolution kernels use programmatic dependent launch), "0"
 * key "stage_barriers": "1" (default; every stage joins all its groups, as the reference does), "0" (a group
 *                  waits only for the groups that produced its inputs)
 * key "pdl_edges": "0"/"1"; in a captured schedule every kernel -> kernel dependency, also between groups
 *                  on different streams, becomes a programmatic one: a kernel's set-up overlaps the tail of
 *                  all its predecessors, not only of the one on its own stream
 * Testing aids (each switches one mechanism of the tensor-core convolution off or pins one choice):
 * "im2col" "1"/"0" (pixel tiles over the flattened pixel axis by im2col-mode loads / boxes of the image),
 * "stem" "1"/"0" (a convolution over at most 4 input channels runs on CUDA cores / on the tensor cores like the rest),
 * "half_rows" "1"/"0" (bfloat16 layers of at most 32 input channels use 64-byte / 128-byte operand rows),
 * "patch" "1"/"0"/"all" (stride-1 windows over many tiles whose packed weights fit in shared memory load one input patch per
 * tile and read every tap from it / never / also layers that stream their weights), "patch_store" "direct"/"bulk"
 * (finished patch tiles leave from registers / through one bulk tensor store per row segment), "issuers" (cap on the
 * warps that issue tcgen05.mma in the patch convolution),
 * "cluster_push" "1"/"0" (the CTAs of a split-K cluster push their partial tiles into each other's shared memory / exchange
 * them through a workspace in L2; same bits), "dual_issue" "1"/"0" (three-pass products issued by two threads into
 * accumulators of their own / by one thread), "weight_prefetch" "1"/"0" (a tensor-core convolution asks the packed
 * weights of the next one into L2 while it runs / does not),
 * "persistent" "1"/"0" (grids of several waves run as resident CTAs that walk the tiles / one CTA per tile),
 * "bulk_store" "1"/"0" (results leave through a bulk tensor store / straight from registers),
 * "split_k", "bn", "stages", "producers" (a positive number overrides the K split, the output-channel tile
 * width, the depth of the shared-memory pipeline, the lanes that issue TMA loads; "0" = automatic), "timeline" "1"/"0" (phase stamps of one CTA).
 * Options apply to plans built afterwards on the calling process. */
IOS_API int ios_set_option(const char *key, const char *value);
IOS_API int ios_get_option(const char *key, char *value, int capacity);

/* Select the CUDA device used by subsequent calls of the calling thread; it also becomes the default
 * of threads that never chose one (reference: device 0 only, src/ios/profile.cu:40-46).  An engine stays
 * on the device it was created on and has streams of its own: engines on one or several devices can be
 * driven from several host threads at once, each call taking only its engine's lock. */
IOS_API int ios_set_device(int device);
IOS_API int ios_device_count(int *count);

/* Page-lock / release caller-owned host memory (cudaHostRegister, portable across devices) so that the
 * copies of ios_engine_run / ios_engine_run_pipelined from and to it are asynchronous.  Used by the batch
 * sharder for the shared-memory arrays its worker processes map.  No reference counterpart. */
IOS_API int ios_host_register(void *memory, size_t bytes);
IOS_API int ios_host_unregister(void *memory);

/* ---- engine: build once, run many (replaces the per-call map()/unmap() of the reference,
 *      src/ios/ios_runtime.cu:1273-1285, 1318-1327, for serving and for benchmarking) ---------- */
typedef struct ios_engine ios_engine;

/* Build a resident plan for (graph, batch size): parses, plans memory, packs and uploads the
 * weights (filter_data / bias_data may be NULL as a whole: synthetic weights are generated). */
IOS_API int ios_engine_create(const char *graph_json, int batch_size, int num_convs, char **conv_names,
                              float **filter_data, float **bias_data, ios_engine **engine);
IOS_API int ios_engine_destroy(ios_engine *engine);
/* Engine artefact: the scheduled graph, the options it was built under, and every convolution's parameters
 * already packed for the kernel and tiling that run it, in one file.  ios_engine_load rebuilds the engine
 * from it on the current device without the float32 weights, without packing and without a schedule
 * search -- what a serving process wants at start-up.  The tiling is re-derived and compared with the
 * stored one: an artefact written by another library version, under other options or for a GPU with another
 * SM count is refused (IOS_ERR_ARGUMENT), never misread.  Replaces the reference's conv2alg.txt side file
 * (src/ios/ios_runtime.cu:91-125), which only remembers cuDNN algorithm numbers, and its per-call weight
 * upload (:1252-1272). */
IOS_API int ios_engine_save(ios_engine *engine, const char *path);
IOS_API int ios_engine_load(const char *path, ios_engine **engine);
/* Host in -> host out.  input[batch, C, H, W], output[batch, Cexit, Hexit, Wexit]. */
IOS_API int ios_engine_run(ios_engine *engine, const float *input, float *output);
/* Host in -> host out for `count` batches in a row, copies overlapped with compute: while batch i runs,
 * batch i + 1 is uploaded and the result of batch i - 1 downloaded (two staging buffers each way, three
 * streams).  inputs[i] / outputs[i] are laid out as for ios_engine_run; the copies only overlap when the
 * buffers are page-locked (cudaHostAlloc / cudaHostRegister), pageable memory works but serialises.
 * Returns after the last result has arrived.  (The reference copies, runs and copies back strictly in
 * turn, src/ios/ios_runtime.cu:1500-1517.) */
IOS_API int ios_engine_run_pipelined(ios_engine *engine, int count, const float *const *inputs,
                                     float *const *outputs);
/* Execute `iters` forwards on the resident input; *ms_per_iter receives the CUDA-event time. */
IOS_API int ios_engine_time(ios_engine *engine, int iters, float *ms_per_iter);
/* Describe the plan: writes a JSON text (kernel launches per forward, arena bytes, workspace bytes,
 * algorithmic FLOPs, output shape) into text[capacity]. */
IOS_API int ios_engine_describe(ios_engine *engine, char *text, int capacity);
/* The plan of a scheduled graph without a device: arena size, launches, and for every convolution the kernel
 * and tiling the current options choose for a GPU of `sm_count` SMs (0: 148) -- JSON into `text`.  Nothing is
 * allocated or launched; a machine without a GPU can call it. */
IOS_API int ios_plan_describe(const char *graph_json, int batch_size, int sm_count, char *text, int capacity);
/* Device time of the launches of one forward by kind: all launches of a kind run one after another
 * on a single stream (captured into one CUDA graph of their own), and every launch is credited with
 * its kind's mean, averaged over `iters` passes.  step_kind: 0 sum/copy, 1 pool,
 * 2 tensor-core conv, 3 CUDA-core conv, 4 depthwise conv.  step_work: algorithmic FLOPs (2*MAC) for
 * kinds 2 and 3, algorithmic bytes (inputs read once + output written once) for kinds 0, 1, 4.
 * Replaces the CUPTI sampling thread of the reference (src/ios/profile.cu:49-143). */
IOS_API int ios_engine_profile(ios_engine *engine, int iters, int capacity, int *count, float *step_ms,
                               int *step_kind, double *step_work);
/* Upload the input once (for ios_engine_time) / read back the last output. */
IOS_API int ios_engine_set_input(ios_engine *engine, const float *input);
IOS_API int ios_engine_get_output(ios_engine *engine, float *output);

/* ---- single-operator entry points used by the parity tests (no reference counterpart: the
 *      reference reaches its operators only through a graph; ConvOP::forward is
 *      src/ios/ios_runtime.cu:309-332, PoolOP::forward :563-566) ------------------------------ */
/* y[n, cout, oh, ow] = act(conv(x[n, cin, h, w], w[cout, cin/groups, kh, kw]) + bias).
 * act: 0 identity, 1 relu, 2 sigmoid, 3 tanh.  impl: 0 auto, 1 direct (CUDA cores), 2 tensor cores with the
 * current precision option, 3 tensor cores single-pass TF32, 4 tensor cores bfloat16. */
IOS_API int ios_conv2d(const float *x, const float *w, const float *bias, float *y, int n, int cin, int h,
                       int wdt, int cout, int kh, int kw, int sh, int sw, int ph, int pw, int groups,
                       int act, int impl);

/* ---- the schedule search (replaces ending_iterator / dop / get_stage_list of the reference,
 *      python/ios/optimizer.py:450-606, which run in Python) ------------------------------------------
 * One handle per part of a block.  Operators are numbered 0..n-1 in topological order; succ_lo/succ_hi hold,
 * per operator, the bit set of its direct successors inside the part (bits 0-63 / 64-127); merge_key is -1
 * for an operator that is no convolution, else (class << 1) | plain, where convolutions of one class read the
 * same value at the same resolution with equal stride and activation and plain means groups == 1 and a single
 * input value; chains (chain_offsets[num_chains + 1] into chain_nodes) are a chain decomposition of the part.
 * ios_dp_enumerate lists every candidate stage the search will ask a latency for, in the order of the first
 * request; ios_dp_stage returns one (kind 0 = merged convolution, 1 = parallel groups; group_offsets has
 * num_groups + 1 entries into nodes; both arrays need room for n + 1 / n ints); after ios_dp_set_latency for
 * every stage, ios_dp_solve evaluates cost(s) = min over endings (cost(s - e) + latency(e)) and ios_dp_chosen
 * returns the chosen stage indices, first stage first. */
typedef struct ios_dp ios_dp;
IOS_API int ios_dp_create(int n, const unsigned long long *succ_lo, const unsigned long long *succ_hi,
                          const int *merge_key, int num_chains, const int *chain_offsets, const int *chain_nodes,
                          int use_merge, int use_parallel, int max_group_size, int max_num_groups, ios_dp **out);
IOS_API int ios_dp_enumerate(ios_dp *search, int *num_stages);
IOS_API int ios_dp_stage(ios_dp *search, int index, int *kind, int *num_groups, int *group_offsets, int *nodes);
IOS_API int ios_dp_set_latency(ios_dp *search, int index, double latency);
IOS_API int ios_dp_solve(ios_dp *search, int *num_chosen, double *best_cost, long long *num_states,
                         long long *num_transitions);
IOS_API int ios_dp_chosen(ios_dp *search, int *stage_indices);
IOS_API int ios_dp_destroy(ios_dp *search);

/* ---- allocation-free entry point (it has no counterpart in the reference) --------------------
 * y[pixels][cout] = act(x[pixels][cin] * w[cout][cin]^T + bias): a 1x1 convolution over NHWC data
 * (pixels = N*H*W), single-pass TF32 products with fp32 accumulation, for callers that are not
 * allowed to allocate device memory when they need it (a plug-in confined to its host's memory
 * pool, a latency-critical loop that must stay off the allocator, a process whose device memory
 * is fully budgeted).  All four pointers are DEVICE pointers the caller owns; w is the plain OIHW
 * array of a 1x1 convolution, bias may be NULL.  The kernel's split-K scratch (partial tiles,
 * arrival counters, time-out word) is a fixed 8 MiB + 20 KiB array inside the library image, held
 * by every GPU that loads the library until the process exits; the call performs no cudaMalloc /
 * cudaFree.  Requirements: cin % 4 == 0, x and w 16-byte aligned.  split_k: 0 = automatic,
 * otherwise the number of CTAs sharing one output tile.  A problem whose scratch need exceeds the
 * array returns IOS_ERR_LIMIT and launches nothing.  The work is enqueued on cuda_stream (a
 * cudaStream_t, NULL = default stream) and NOT synchronised.  Every call shares the one array,
 * which keeps the previous call's contents (the words that must be zero are cleared in stream
 * order at the start of each call): calls that overlap on the GPU race.  The first call on a
 * device resolves the array's device address; make it before any stream capture begins.
 * Results leave through bulk tensor stores when y is 16-byte aligned and cout % 4 == 0, through plain
 * stores from registers otherwise: same values, any alignment of y and any cout are accepted. */
IOS_API int ios_pointwise_conv_static_scratch(const float *x, const float *w, const float *bias, float *y,
                                              int pixels, int cin, int cout, int act, int split_k,
                                              void *cuda_stream);

/* Companion of the call above (it, too, has no counterpart in the reference): waits for cuda_stream,
 * then reads the time-out word of the static scratch -- without allocating -- and returns
 * IOS_ERR_TIMEOUT if a bounded wait inside the kernel ran out since the last check (the output of that
 * call is then incomplete; the word and the counters are cleared), IOS_OK otherwise. */
IOS_API int ios_static_scratch_status(void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif  /* IOS_RUNTIME_H_ */
