"""
Benchmark of the hot path: executing a scheduled CNN on B200 through libios_runtime.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model inception_v3|squeezenet|randwire_small|sample_block] [--batch B]
                    [--schedule dp|sequential|greedy]

One step = one forward of the model over one batch of synthetic input (seeded N(0,1) input,
He-normal seeded weights, the distribution the workload is defined on).  The default workload is
Inception-v3, batch 1 per GPU, under the schedule found by ``ios.optimize`` (the DP search) on the
GPU it runs on.  Batch 1 does not shard, so N > 1 runs N independent replicas (one process per
GPU, no collective on the data path) and reports the aggregate images/s; ``ms_per_step`` is the
batch-1 latency.

What is timed:
* ``value`` / ``ms_per_step``: device time of K forwards with input and weights resident in HBM,
  CUDA events on the launching stream around each step, an L2 flush (a 256 MiB write) between
  steps, max over ranks;
* ``e2e``: the same K steps through the host-buffer entry point (``ios_engine_run``): pinned host
  input -> H2D -> forward -> D2H -> pinned host output, wall clock around the blocking call;
* ``roofline``: per-launch device times of the convolution kernel measured live
  (``ios_engine_profile``), algorithmic FLOPs = 2 * MACs of the original convolutions;
* ``cpu_baseline``: the CPU oracle (a torch float32 restatement of the reference's CPU executor) on
  the host cores, a bounded number of forwards of the same workload.

``--impl reference`` times the reference's own runtime (its cuDNN executor, built unmodified from
its sources into oracle/_ref/) on the same workload through its own ``graph_latency`` protocol; if
that library cannot be loaded, the CPU oracle is timed instead.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _sub in ('inter-operator-scheduler_b200', 'oracle'):
    sys.path.insert(0, os.path.join(ROOT, _sub))

import numpy as np  # noqa: E402

METRIC = 'images/sec on Inception-v3 under the DP schedule (ms_per_step = batch-1 end-to-end latency ms)'
L2_FLUSH_BYTES = 256 << 20


def log(*args):
    print(*args, file=sys.stderr, flush=True)


def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as fh:
            peaks = json.load(fh)
        return peaks, 'measured'
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0}, 'fallback'


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--id={self.device_index}', f'--query-gpu={self.QUERY}',
                                          '--format=csv,noheader,nounits', '-lms', '50'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._drain, daemon=True)
            self.thread.start()
            deadline = time.time() + 5.0          # the timed region starts once the sampler is really running
            while not self.lines and time.time() < deadline:
                time.sleep(0.01)
        except OSError:
            self.proc = None
        return self

    def _drain(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in self.lines:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith('active'):
                    reasons.add(name)
        if not sm:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        return {'sm_mhz': statistics.median(sm), 'sm_max_mhz': max(mx), 'reasons': sorted(reasons), 'samples': len(sm)}


def kernel_sources_sha16():
    """Identifies the build: a hash over the CUDA sources of the convolution kernels."""
    import hashlib
    digest = hashlib.sha256()
    for name in ('conv_tc.cu', 'conv_tc_patch.cu', 'tc_device.h', 'conv_direct.cu', 'kernels.h', 'plan.cu'):
        with open(os.path.join(ROOT, 'inter-operator-scheduler_b200', 'csrc', name), 'rb') as fh:
            digest.update(fh.read())
    return digest.hexdigest()[:16]


def build_graph(model):
    import ios
    if model == 'sample_block':
        ios.reset_name()
        v = ios.placeholder(output_shape=(375, 15, 15))
        block = ios.Block(enter_node=v.node)
        v1 = ios.conv2d(block, inputs=[[v]], out_channels=375, kernel=(3, 3), stride=(1, 1), padding=(1, 1))
        v2 = ios.conv2d(block, inputs=[[v]], out_channels=750, kernel=(3, 3), stride=(1, 1), padding=(1, 1))
        v3 = ios.conv2d(block, inputs=[[v]], out_channels=375, kernel=(3, 3), stride=(1, 1), padding=(1, 1))
        v1 = ios.conv2d(block, inputs=[[v1]], out_channels=750, kernel=(3, 3), stride=(1, 1), padding=(1, 1))
        ios.identity(block, inputs=[[v1], [v2], [v3]], is_exit=True)
        graph = ios.Graph(name='demo', input=v.node, blocks=[block])
    else:
        graph = getattr(ios.models, model)()
    return graph


def seeded_weights(graph, seed=0):
    import ios_oracle as oracle
    config = graph.export_config()
    weights = oracle.he_normal_weights(config, seed)
    for conv in graph.convs():
        conv.weight, conv.bias = weights[conv.name]
    return weights


def schedule_graph(graph, schedule, batch, cost_model=None, warmup=2, number=6, repeat=3):
    """Returns the graph to execute and the seconds the schedule search took."""
    import ios
    t0 = time.time()
    if schedule == 'sequential':
        graph.sequential_schedule()
        return graph, 0.0
    if schedule == 'greedy':
        graph.greedy_schedule()
        return graph, 0.0
    opt = ios.optimize(graph, batch_size=batch, cost_model=cost_model, opt_type='dp_parallel_merge',
                       compute_weight=True, max_part_size=50, warmup=warmup, number=number, repeat=repeat)
    return opt, time.time() - t0


# ------------------------------------------------------------------------------------------------
# distributed plumbing (one process per GPU; only a barrier and a max-reduce of the timing)
# ------------------------------------------------------------------------------------------------
class Ranks:
    def __init__(self, gpus):
        self.world = int(os.environ.get('WORLD_SIZE', '1'))
        self.rank = int(os.environ.get('RANK', '0'))
        self.local = int(os.environ.get('LOCAL_RANK', '0'))
        self.dist = None
        if self.world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(self.local)
            dist.init_process_group('nccl', device_id=torch.device('cuda', self.local))
            self.dist = dist
        elif gpus > 1:
            log(f'--gpus {gpus} was given without torchrun: running a single replica on GPU 0')

    def barrier(self):
        import torch
        if self.dist:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, value):
        if not self.dist:
            return value
        import torch
        t = torch.tensor([value], dtype=torch.float64, device='cuda')
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, value):
        if not self.dist:
            return value
        import torch
        t = torch.tensor([value], dtype=torch.float64, device='cuda')
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def finish(self):
        if self.dist:
            self.dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import ios
    import ios_oracle as oracle
    from ios.contrib import ios_runtime as rt

    ranks = Ranks(args.gpus)
    device = ranks.local
    torch.cuda.set_device(device)
    rt.set_device(device)
    rt.set_option('executor', args.executor)
    if args.precision:
        rt.set_option('precision', args.precision)
    peaks, peak_kind = measured_peaks()

    graph = build_graph(args.model)
    weights = seeded_weights(graph, 0)
    base_config = graph.export_config()
    cost_model = ios.cost_model.IOSCostModel() if args.schedule == 'dp' else None
    exec_graph, search_s = schedule_graph(graph, args.schedule, args.batch, cost_model=cost_model)
    schedule_note = args.schedule
    additivity = None
    if args.schedule == 'dp':
        # what the search minimised: the sum of the latencies of the chosen stages, each measured alone
        # (answered from the cost model's memo); reported beside the latency of the whole schedule
        try:
            isolated = 0.0
            for block in exec_graph.blocks:
                nodes = {n.name: n for n in block.inner_nodes + [block.exit_node]}
                for stage in block.stages:
                    isolated += float(np.mean(cost_model.get_stage_latency(
                        [[nodes[name] for name in group] for group in stage], args.batch, 2, 6, 3)))
            additivity = {'sum_of_isolated_stage_ms': round(isolated, 4), 'stages_measured_by_search': cost_model.measured}
        except Exception as exc:      # (reporting only)
            additivity = {'error': repr(exc)}
    if args.schedule == 'dp':
        # the search adds up stage latencies measured one by one; the whole schedules are timed too and the
        # heuristic one is kept if it is faster (both numbers are reported)
        graph.greedy_schedule()          # (the search returned a new graph; the original is free to carry this one)
        exec_graph, whole = rt.pick_faster([exec_graph, graph], args.batch, warmup=3, number=10, repeat=5)
        schedule_note = (f'dp ({whole[0]:.4f} ms whole) vs greedy ({whole[1]:.4f} ms whole): '
                         f'{"dp" if whole[0] <= whole[1] else "greedy"} kept')
        if additivity and 'sum_of_isolated_stage_ms' in additivity:
            additivity['dp_whole_ms'] = round(whole[0], 4)
            additivity['greedy_whole_ms'] = round(whole[1], 4)
            additivity['whole_minus_sum_over_sum'] = round((whole[0] - additivity['sum_of_isolated_stage_ms']) /
                                                            additivity['sum_of_isolated_stage_ms'], 4)
    log(f'[rank {ranks.rank}] schedule "{schedule_note}": {sum(len(b.stages) for b in exec_graph.blocks)} stages, '
        f'search took {search_s:.1f} s')

    engine = rt.Engine(exec_graph, args.batch)
    info = engine.describe()
    x = oracle.normal_input(base_config, args.batch, 0)
    host_in = torch.from_numpy(x).pin_memory()
    host_out = torch.empty(engine.output_shape, dtype=torch.float32).pin_memory()
    engine.set_input(x)
    flush = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.float32, device='cuda')

    def flush_l2():
        flush.zero_()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------------------
    for _ in range(args.warmup):
        flush_l2()
        engine.time(1)
    ranks.barrier()
    with ClockSampler(device) as sampler:
        step_ms = []
        t_wall = time.perf_counter()
        for _ in range(args.steps):
            flush_l2()
            step_ms.append(engine.time(1))
        device_ms = sum(step_ms)
        ranks.barrier()
        wall_s = time.perf_counter() - t_wall
        warm_ms = engine.time(max(10, args.steps))          # back-to-back replays, weights stay in L2
        # ---- end to end through the host-buffer entry point -------------------------------------
        for _ in range(args.warmup):
            engine.run(host_in.data_ptr(), host_out.data_ptr())
        ranks.barrier()
        e2e_steps = []
        for _ in range(args.steps):
            flush_l2()
            t0 = time.perf_counter()
            engine.run(host_in.data_ptr(), host_out.data_ptr())
            e2e_steps.append(time.perf_counter() - t0)
        e2e_s = sum(e2e_steps)
        ranks.barrier()
        # the same K steps through the pipelined host-buffer entry point: upload of step i + 1 and download
        # of step i - 1 beside the forward of step i (throughput, not latency; reported beside e2e)
        engine.run_pipelined([host_in.data_ptr()] * args.warmup, [host_out.data_ptr()] * args.warmup)
        ranks.barrier()
        t0 = time.perf_counter()
        engine.run_pipelined([host_in.data_ptr()] * args.steps, [host_out.data_ptr()] * args.steps)
        pipelined_s = time.perf_counter() - t0
        ranks.barrier()
        sharded = None
        if args.sharded_sweep and args.model == 'inception_v3' and args.batch == 1:
            sharded = sharded_sweep(graph, base_config, weights, ranks, peaks, peak_kind, args)
    clocks = sampler.summary()
    pipelined_ms = ranks.max_over_ranks(1e3 * pipelined_s / args.steps)
    ms_per_step = ranks.max_over_ranks(device_ms / args.steps)
    e2e_ms = ranks.max_over_ranks(1e3 * e2e_s / args.steps)
    images = args.batch * ranks.world
    value = images / (ms_per_step * 1e-3)
    e2e_value = images / (e2e_ms * 1e-3)

    # the end-to-end result must be the function the oracle computes
    y = host_out.numpy().copy()

    # ---- roofline of the dominant kernel ----------------------------------------------------
    steps = engine.profile(5)
    by_kind = {}
    for kind, ms, work in steps:
        slot = by_kind.setdefault(kind, {'launches': 0, 'ms': 0.0, 'work': 0.0})
        slot['launches'] += 1
        slot['ms'] += ms
        slot['work'] += work
    total_ms = sum(v['ms'] for v in by_kind.values())
    conv = by_kind.get('conv_tc', {'launches': 0, 'ms': 0.0, 'work': 0.0})
    precision = rt.get_option('precision')
    if precision == 'bf16':
        tensor_peak = peaks['bf16_tflops']
        peak_note = f'{peak_kind} bf16 burst (cuBLAS bf16 GEMM)'
    else:
        tensor_peak = peaks['bf16_tflops'] / 2.0
        peak_note = f'{peak_kind} bf16 burst / 2 (dense TF32 is half the bf16 rate; not measured separately)'
    tf32_peak = tensor_peak
    achieved = conv['work'] / (conv['ms'] * 1e-3) / 1e12 if conv['ms'] > 0 else 0.0
    roofline = {
        'bound': 'tensor', 'kernel': 'conv_tc_kernel', 'achieved': round(achieved, 3), 'peak': tf32_peak,
        'unit': 'TFLOP/s', 'frac': round(achieved / tf32_peak, 5),
        'peak_source': peak_note,
        'traffic': None,
        'launches_per_step': conv['launches'], 'avg_launch_us': round(1e3 * conv['ms'] / max(1, conv['launches']), 3),
        'flops_per_step': conv['work'],
        'share_of_device_time': round(conv['ms'] / total_ms, 4) if total_ms else None,
        # work is bytes for the bandwidth kernels and multiply-add flops for the CUDA-core convolution
        'other_kernels': {k: {'launches': v['launches'], 'ms': round(v['ms'], 4),
                              ('GFLOP/s' if k == 'conv_direct' else 'GB/s'):
                                  round(v['work'] / (v['ms'] * 1e-3) / 1e9, 1) if v['ms'] > 0 else None}
                          for k, v in by_kind.items() if k != 'conv_tc'},
    }
    # DRAM bytes of the convolution launches of one forward: an ncu capture cannot run inside the bench, so the
    # figure is looked up in the table committed beside the profile summaries, by workload, and only used when
    # the kernel sources are still the ones it was captured with
    table = os.path.join(ROOT, 'profiles', 'conv_tc_traffic.json')
    if os.path.exists(table):
        with open(table) as fh:
            entries = json.load(fh)
        key = f'{args.model}/batch{args.batch}/{precision}'
        entry = entries.get(key)
        if entry:
            roofline['traffic'] = entry['dram_bytes_per_forward'] if entry.get('sources_sha16') == kernel_sources_sha16() else None
            roofline['traffic_source'] = (f"ncu dram__bytes_read+write over the convolution launches of one forward, "
                                          f"{entry.get('schedule')} schedule, kernel sources {entry.get('sources_sha16')} "
                                          f"(profiles/conv_tc_traffic.json; this build: {kernel_sources_sha16()})")

    line = {
        'metric': METRIC, 'value': round(value, 2), 'unit': 'images/s', 'n_gpus': ranks.world, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': round(ms_per_step, 5), 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'data': 'synthetic',
        'dtype': {'tf32x3': 'tf32 (fp32 storage, three TF32 products per multiply, fp32 accumulate)',
                  'tf32': 'tf32 (fp32 storage, fp32 accumulate)', 'bf16': 'bf16 (fp32 accumulate)',
                  'fp32': 'fp32 (CUDA cores)'}[precision],
        'config': {'workload': f'{args.model} batch {args.batch} per GPU, schedule {args.schedule} '
                               f'({info["stages"]} stages, {info["launches"]} launches)',
                   'global_batch': images, 'input': list(x.shape[1:]), 'parallelism':
                       'single GPU' if ranks.world == 1 else
                       (f'{ranks.world} independent replicas (batch 1 does not shard)' if args.batch == 1 else
                        f'global batch {images} sharded evenly, {args.batch} images per GPU, no collective on the data path'),
                   'l2': 'flushed between steps by a 256 MiB write', 'schedule_search_s': round(search_s, 1),
                   'schedule_choice': schedule_note},
        'e2e': {'value': round(e2e_value, 2), 'unit': 'images/s', 'ms_per_step': round(e2e_ms, 5),
                'h2d_bytes_per_step': int(x.nbytes), 'd2h_bytes_per_step': int(y.nbytes)},
        'gpu_launches': info['launches'] * args.steps + (info['launches'] + 2) * args.steps * 2 +
                        info['launches'] * max(10, args.steps),
        'schedule_additivity': additivity,
        'warm_l2_ms_per_step': round(warm_ms, 5),
        'ms_per_step_spread': {'median': round(statistics.median(step_ms), 5), 'p10': round(float(np.percentile(step_ms, 10)), 5),
                               'p90': round(float(np.percentile(step_ms, 90)), 5), 'note': 'rank 0, device time per step'},
        'e2e_ms_per_step_spread': {'median': round(1e3 * statistics.median(e2e_steps), 5),
                                   'p10': round(1e3 * float(np.percentile(e2e_steps, 10)), 5),
                                   'p90': round(1e3 * float(np.percentile(e2e_steps, 90)), 5)},
        'e2e_pipelined': {'value': round(images / (pipelined_ms * 1e-3), 2), 'unit': 'images/s',
                          'ms_per_step': round(pipelined_ms, 5),
                          'note': 'same host buffers and copies, K steps through ios_engine_run_pipelined '
                                  '(copies overlap compute)'},
        'wall_s_timed_region': round(wall_s, 3),
        'clocks': clocks, 'roofline': roofline,
    }

    if sharded is not None:
        line['sharded_sweep'] = sharded
    if ranks.world == 1 and args.sweep and args.model == 'inception_v3' and args.batch == 1:
        line['throughput_sweep'] = throughput_sweep(graph, base_config, weights, peaks, peak_kind)

    if ranks.rank == 0:
        ref = oracle.run_config(base_config, weights, x)
        line['parity_max_rel_err'] = float(f'{oracle.max_rel_err(y, ref):.3e}')
        if ranks.world == 1 and not args.no_cpu_baseline:
            line['cpu_baseline'] = cpu_baseline(base_config, weights, x, args.batch)
        print(json.dumps(line), flush=True)
    engine.close()
    ranks.finish()


def conv_flops_per_image(graph):
    return 2.0 * sum(c.output_shape[0] * c.output_shape[1] * c.output_shape[2] * c.kernel[0] * c.kernel[1] *
                     (c.input_shape[0] // c.groups) for c in graph.convs())


def tensor_peak(peaks, precision):
    return peaks['bf16_tflops'] if precision == 'bf16' else peaks['bf16_tflops'] / 2.0


PARITY_BOUND = {'tf32x3': 1e-3, 'tf32': 6e-3, 'bf16': 2e-2}     # tf32: the known growth over 47 layers, see the tests


def checked_images(engine_out, config, weights, x, count=2):
    """Max relative error of the first ``count`` images of a batch against the CPU oracle (every image is independent)."""
    import ios_oracle as oracle
    ref = oracle.run_config(config, weights, x[:count])
    return float(f'{oracle.max_rel_err(engine_out[:count], ref):.3e}')


def throughput_sweep(graph, config, weights, peaks, peak_kind):
    """
    Images/s of the same network at batch 16 / 64 / 256 on one GPU (greedy schedule, seeded weights,
    device-resident, CUDA events over back-to-back replays; the activations alone exceed L2 from batch
    16 on) for three-pass TF32, single-pass TF32 and bfloat16, each with its fraction of the measured
    tensor peak.  The batch-16 run of every precision is checked against the CPU oracle.
    """
    import ios_oracle as oracle
    from ios.contrib import ios_runtime as rt
    saved = rt.get_option('precision')
    flops_per_image = conv_flops_per_image(graph)
    greedy = graph
    greedy.greedy_schedule()
    out, parity = [], {}
    for precision in ('tf32x3', 'tf32', 'bf16'):
        rt.set_option('precision', precision)
        peak = tensor_peak(peaks, precision)
        for batch in (16, 64, 256):
            engine = rt.Engine(greedy, batch)
            if batch == 16:
                x = oracle.normal_input(config, batch, 1)
                parity[precision] = checked_images(engine.run(x), config, weights, x)
                if parity[precision] > PARITY_BOUND[precision]:
                    raise RuntimeError(f'throughput sweep: {precision} batch 16 is off by {parity[precision]}')
            engine.time(2)
            ms = engine.time(5)
            engine.close()
            tflops = flops_per_image * batch / (ms * 1e-3) / 1e12
            out.append({'precision': precision, 'batch': batch, 'ms': round(ms, 3), 'images_per_s': round(batch / ms * 1e3, 1),
                        'conv_tflops': round(tflops, 1), 'frac_of_tensor_peak': round(tflops / peak, 4)})
    rt.set_option('precision', saved)
    return {'schedule': 'greedy', 'peak_source': f'{peak_kind} bf16 burst (bf16) or half of it (tf32)',
            'parity_max_rel_err_batch16': parity, 'points': out}


def sharded_sweep(graph, config, weights, ranks, peaks, peak_kind, args):
    """
    The batch-sharded configuration: a global batch of 256 (and 64) images split evenly over the ranks,
    one engine per GPU on its shard, no collective on the data path.  Every rank searches the schedule for
    ITS shard's batch size and precision on its own GPU (ios.optimize, dp_parallel_merge, measured stage
    latencies) and keeps the greedy schedule instead if that is faster when timed whole.  Reported per
    point: device-resident images/s (CUDA events over K back-to-back forwards, max over ranks), end-to-end
    images/s (K steps through ios_engine_run_pipelined from / to page-locked host buffers, wall clock, max
    over ranks) and the convolution TFLOP/s as a fraction of N x the measured tensor peak.
    """
    import torch
    import ios
    import ios_oracle as oracle
    from ios.contrib import ios_runtime as rt
    saved = rt.get_option('precision')
    flops_per_image = conv_flops_per_image(graph)
    points = []
    steps = max(args.steps, 10)
    for precision in ('bf16', 'tf32x3'):
        rt.set_option('precision', precision)
        for global_batch in (256, 64):
            if global_batch % ranks.world:
                continue
            shard = global_batch // ranks.world
            t0 = time.time()
            dp = ios.optimize(graph, batch_size=shard, opt_type='dp_parallel_merge', compute_weight=True, max_part_size=50,
                              warmup=1, number=2, repeat=1)
            search_s = time.time() - t0
            graph.greedy_schedule()
            chosen, whole = rt.pick_faster([dp, graph], shard, warmup=1, number=3, repeat=2)
            engine = rt.Engine(chosen, shard)
            x = oracle.normal_input(config, shard, 100 + ranks.rank)
            host_in = torch.from_numpy(x).pin_memory()
            host_out = torch.empty(engine.output_shape, dtype=torch.float32).pin_memory()
            parity = checked_images(engine.run(host_in.data_ptr(), host_out.numpy()), config, weights, x)
            if parity > PARITY_BOUND[precision]:
                raise RuntimeError(f'sharded sweep: {precision} shard batch {shard} is off by {parity}')
            engine.set_input(x)
            engine.time(3)
            ranks.barrier()
            device_ms = ranks.max_over_ranks(engine.time(steps))
            engine.run_pipelined([host_in.data_ptr()] * 3, [host_out.data_ptr()] * 3)
            ranks.barrier()
            t0 = time.perf_counter()
            engine.run_pipelined([host_in.data_ptr()] * steps, [host_out.data_ptr()] * steps)
            e2e_ms = ranks.max_over_ranks(1e3 * (time.perf_counter() - t0) / steps)
            t0 = time.perf_counter()
            for _ in range(steps):
                engine.run(host_in.data_ptr(), host_out.data_ptr())
            serial_ms = ranks.max_over_ranks(1e3 * (time.perf_counter() - t0) / steps)
            ranks.barrier()
            info = engine.describe()
            engine.close()
            tflops = flops_per_image * global_batch / (device_ms * 1e-3) / 1e12
            points.append({
                'precision': precision, 'global_batch': global_batch, 'shard_batch': shard,
                'schedule': 'dp' if whole[0] <= whole[1] else 'greedy', 'stages': info['stages'],
                'whole_ms_dp_vs_greedy': [round(v, 4) for v in whole], 'schedule_search_s': round(search_s, 1),
                'device_ms_per_step': round(device_ms, 4), 'images_per_s': round(global_batch / device_ms * 1e3, 1),
                'e2e_ms_per_step': round(e2e_ms, 4), 'e2e_images_per_s': round(global_batch / e2e_ms * 1e3, 1),
                'e2e_unpipelined_images_per_s': round(global_batch / serial_ms * 1e3, 1),
                'h2d_bytes_per_step_per_gpu': int(x.nbytes), 'd2h_bytes_per_step_per_gpu': int(host_out.numel() * 4),
                'conv_tflops': round(tflops, 1),
                'frac_of_tensor_peak': round(tflops / (ranks.world * tensor_peak(peaks, precision)), 4),
                'parity_max_rel_err': parity})
            del host_in, host_out
    rt.set_option('precision', saved)
    return {'note': 'global batch split evenly over the ranks, no collective on the data path; schedule searched per rank '
                    'for the shard batch; steps per point: %d' % steps,
            'peak_source': f'{peak_kind} bf16 burst (bf16) or half of it (tf32x3), times the number of GPUs',
            'points': points}


def cpu_baseline(config, weights, x, batch, budget_s=15.0):
    """The CPU oracle on the host cores: as many forwards of the same workload as fit the budget."""
    import torch
    import ios_oracle as oracle
    cores = torch.get_num_threads()
    oracle.run_config(config, weights, x)
    t0 = time.perf_counter()
    n = 0
    while n < 3 or (time.perf_counter() - t0 < budget_s and n < 200):
        oracle.run_config(config, weights, x)
        n += 1
    per = (time.perf_counter() - t0) / n
    return {'value': round(batch / per, 2), 'unit': 'images/s', 'ms_per_step': round(per * 1e3, 3), 'cores': cores,
            'kind': 'port', 'sample': f'{n} forwards of the same graph and input on the host cores (torch CPU float32 '
                                      f'restatement of the reference executor ios.torch_utils.Net)'}


# ------------------------------------------------------------------------------------------------
class ReferenceRuntime:
    """The reference's own libios_runtime.so (cuDNN), driven with this package's JSON."""

    def __init__(self):
        self.lib = ctypes.cdll.LoadLibrary(os.path.join(ROOT, 'oracle', '_ref', 'libios_runtime_ref.so'))

    def graph_latency(self, graph, batch, warmup, number, repeat):
        text = json.dumps(graph.export_config()).encode()
        n_stages = sum(len(b.stages) for b in graph.blocks)
        res = (ctypes.c_float * repeat)()
        stage = (ctypes.c_float * (repeat * n_stages))()
        self.lib.graph_latency(ctypes.c_char_p(text), batch, warmup, number, repeat, 0, res, stage)
        return [float(v) for v in res]

    def stage_latency(self, stage, batch, warmup, number, repeat):
        from ios.contrib.ios_runtime import stage_config
        stage_text, input_text = stage_config(stage)
        res = (ctypes.c_float * repeat)()
        unused = (ctypes.c_float * repeat)()
        self.lib.stage_latency(ctypes.c_char_p(stage_text.encode()), ctypes.c_char_p(input_text.encode()), batch,
                               warmup, number, repeat, 0, res, unused)
        return [float(v) for v in res]


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    import ios
    import ios_oracle as oracle
    graph = build_graph(args.model)
    weights = seeded_weights(graph, 0)
    config = graph.export_config()
    x = oracle.normal_input(config, args.batch, 0)
    line = {'impl': 'reference', 'metric': METRIC, 'unit': 'images/s', 'n_gpus': 1, 'steps': args.steps,
            'warmup': args.warmup, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
            'data': 'synthetic'}
    try:
        ref = ReferenceRuntime()
    except OSError as err:
        ref = None
        log(f'reference runtime not loadable ({err}); timing the CPU oracle instead')
    if ref is not None:
        class RefCost(ios.cost_model.CostModel):
            def get_stage_latency(self, stage, batch_size, warmup, number, repeat, profile_stage=False):
                return ref.stage_latency(stage, batch_size, warmup, number, repeat)

        exec_graph, search_s = schedule_graph(graph, args.schedule, args.batch, cost_model=RefCost(), number=4, repeat=2)
        samples = ref.graph_latency(exec_graph, args.batch, args.warmup, 1, args.steps)
        ms = float(np.mean(samples))
        value = args.batch / (ms * 1e-3)
        line.update({
            'value': round(value, 2), 'ms_per_step': round(ms, 5), 'dtype': 'fp32 (cuDNN default math)',
            'config': {'workload': f'{args.model} batch {args.batch}, schedule {args.schedule} found by the same DP '
                                   f'search on the reference runtime\'s own stage_latency '
                                   f'({sum(len(b.stages) for b in exec_graph.blocks)} stages)',
                       'global_batch': args.batch, 'parallelism': 'single GPU', 'schedule_search_s': round(search_s, 1),
                       'l2': 'not flushed (the reference times back-to-back forwards inside graph_latency)'},
            'cpu_baseline': {'value': round(value, 2), 'unit': 'images/s', 'kind': 'reference', 'cores': 0,
                             'sample': 'the reference runtime executes on the GPU through cuDNN (it has no CPU '
                                       'executor in C++); graph_latency(warmup, number=1, repeat=steps) on device 0'},
            'e2e': {'value': round(value, 2), 'unit': 'images/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        })
    else:
        graph.sequential_schedule()
        base = cpu_baseline(config, weights, x, args.batch, budget_s=20.0)
        line.update({'value': base['value'], 'ms_per_step': base['ms_per_step'], 'dtype': 'fp32',
                     'config': {'workload': f'{args.model} batch {args.batch} on the host cores', 'global_batch': args.batch},
                     'cpu_baseline': base,
                     'e2e': {'value': base['value'], 'unit': 'images/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}})
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--model', default='inception_v3')
    ap.add_argument('--batch', type=int, default=1, help='images per GPU per step')
    ap.add_argument('--schedule', default='dp', choices=['dp', 'sequential', 'greedy'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-sweep', dest='sweep', action='store_false',
                    help='skip the batch 16/64/256 throughput sweep that the default single-GPU run appends')
    ap.add_argument('--no-sharded-sweep', dest='sharded_sweep', action='store_false',
                    help='skip the batch-sharded configuration (global batch 256 and 64 split over the ranks)')
    ap.add_argument('--executor', default='graph', choices=['graph', 'streams'],
                    help='streams: plain launches instead of a CUDA graph (used for kernel-level profiling)')
    ap.add_argument('--precision', default=None, help='runtime precision option (default: the library default)')
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
