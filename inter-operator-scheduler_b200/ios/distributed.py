"""
Multi-GPU use of the runtime on one 8 x B200 box: batch sharding and the stage-profiling farm.

The reference is single-GPU (device 0 only, ``src/ios/profile.cu:40-46``).  Its path shards over
independent units, so nothing here exchanges data between GPUs while a network runs:

* ``shard_slices`` / ``ShardedInference``: a batch of 16 or more images is split evenly across the
  GPUs; every GPU holds a full weight replica and an engine built for its shard's batch size; the
  host scatters input slices and gathers output slices.  No collective is involved.
* ``StageFarm`` / ``FarmCostModel``: the DP search of ``ios.optimize`` spends its time measuring
  candidate stages (thousands of independent ``stage_latency`` calls,
  ``python/ios/optimizer.py:297-340``).  The farm first enumerates every candidate the search will
  ask for, measures them in parallel on all GPUs, then lets the search run on the memo.  The memo
  can be saved and loaded, so an interrupted search resumes.

Both are built on ``GpuWorkerPool``: one worker PROCESS per GPU (the runtime keeps one context per
device, and a process per GPU keeps launches of different GPUs from serialising on one host
thread).  Failures are handled on the host: a worker that dies or exceeds the task time limit is
dropped and its task is re-queued on another worker; device-side faults are never provoked.
"""
import json
import multiprocessing as mp
import multiprocessing.connection
import os
import time
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

MIN_SHARD_BATCH = 16     # below this a batch stays on one GPU


def shard_slices(batch: int, parts: int) -> List[Tuple[int, int]]:
    """Split ``range(batch)`` into ``parts`` contiguous slices whose sizes differ by at most one."""
    if parts <= 0:
        raise ValueError('parts must be positive')
    base, extra = divmod(batch, parts)
    out, begin = [], 0
    for i in range(parts):
        end = begin + base + (1 if i < extra else 0)
        out.append((begin, end))
        begin = end
    return out


def plan_shards(batch: int, gpus: int) -> List[Tuple[int, int]]:
    """Slices actually used: one GPU below ``MIN_SHARD_BATCH``, never an empty shard."""
    if batch < MIN_SHARD_BATCH or gpus <= 1:
        return [(0, batch)]
    return [s for s in shard_slices(batch, min(gpus, batch)) if s[1] > s[0]]


# ------------------------------------------------------------------------------------------------
# worker pool
# ------------------------------------------------------------------------------------------------
class RuntimeBackend:
    """What a worker process runs on its GPU: the real runtime, bound to one device."""

    def __init__(self, device: int):
        from ios.contrib import ios_runtime
        self.rt = ios_runtime
        self.device = device
        ios_runtime.set_device(device)
        self.engines = {}

    def stage_latency(self, stage_json, input_json, batch, warmup, number, repeat):
        import ctypes
        lib = self.rt._library()
        results = (ctypes.c_float * repeat)()
        unused = (ctypes.c_float * repeat)()
        self.rt._check(lib.ios_stage_latency(stage_json.encode(), input_json.encode(), batch, warmup, number, repeat, 0,
                                             results, unused))
        return [float(v) for v in results]

    def engine_create(self, key, graph_json, batch, weights):
        import ios
        graph = ios.Graph.from_config(json.loads(graph_json))
        for conv in graph.convs():
            conv.weight, conv.bias = weights[conv.name]
        self.engines[key] = self.rt.Engine(graph, batch)
        return self.engines[key].output_shape

    def engine_run(self, key, x):
        return self.engines[key].run(x)

    def engine_attach(self, key, in_name, out_name, in_shape, out_shape, begin, end):
        """
        Map the parent's shared input / output arrays, page-lock this shard's part of them, and remember
        the addresses: ``engine_run_shared`` then moves no data between processes at all.
        """
        from multiprocessing import shared_memory
        shm_in = shared_memory.SharedMemory(name=in_name)
        shm_out = shared_memory.SharedMemory(name=out_name)
        x = np.ndarray(in_shape, dtype=np.float32, buffer=shm_in.buf)[begin:end]
        y = np.ndarray(out_shape, dtype=np.float32, buffer=shm_out.buf)[begin:end]
        pinned = [self.rt.host_register(x), self.rt.host_register(y)]
        self.shared = getattr(self, 'shared', {})
        self.shared[key] = (shm_in, shm_out, x, y, pinned)
        return all(pinned)

    def engine_run_shared(self, key, repeats=1):
        _, _, x, y, _ = self.shared[key]
        engine = self.engines[key]
        if repeats == 1:
            engine.run(x.ctypes.data, y.ctypes.data)
        else:
            engine.run_pipelined([x.ctypes.data] * repeats, [y.ctypes.data] * repeats)
        return True

    def engine_detach(self, key):
        shm_in, shm_out, x, y, pinned = self.shared.pop(key)
        for array, ok in zip((x, y), pinned):
            if ok:
                self.rt.host_unregister(array)
        del x, y
        shm_in.close()
        shm_out.close()
        return True

    def engine_time(self, key, iters):
        return self.engines[key].time(iters)

    def set_option(self, key, value):
        self.rt.set_option(key, value)
        return True


def _worker_main(conn, device, backend_factory):
    try:
        backend = backend_factory(device)
        conn.send(('ready', device))
    except Exception as err:                      # noqa: BLE001 - reported to the parent
        conn.send(('failed', repr(err)))
        return
    while True:
        try:
            message = conn.recv()
        except EOFError:
            return
        if message is None:
            return
        task_id, method, args = message
        try:
            conn.send((task_id, 'ok', getattr(backend, method)(*args)))
        except Exception as err:                  # noqa: BLE001 - reported to the parent
            conn.send((task_id, 'error', repr(err)))


class WorkerLost(RuntimeError):
    pass


class GpuWorkerPool:
    """
    One worker process per device.  ``map`` hands tasks to idle workers, re-queues the task of a
    worker that died or ran past ``task_timeout`` seconds (the worker is dropped), and raises once
    no worker is left or a task has failed ``max_attempts`` times.
    """

    def __init__(self, devices: Sequence[int], backend_factory: Callable = RuntimeBackend, task_timeout: float = 120.0,
                 max_attempts: int = 3, start_timeout: float = 300.0):
        self.ctx = mp.get_context('spawn')
        self.task_timeout = task_timeout
        self.max_attempts = max_attempts
        self.workers = {}
        self.lost = []
        self._next_id = 0
        for device in devices:
            parent, child = self.ctx.Pipe()
            proc = self.ctx.Process(target=_worker_main, args=(child, device, backend_factory), daemon=True)
            proc.start()
            child.close()
            self.workers[device] = (proc, parent)
        deadline = time.time() + start_timeout
        for device in list(self.workers):
            proc, conn = self.workers[device]
            if not conn.poll(max(0.0, deadline - time.time())):
                self._drop(device, 'did not start in time')
                continue
            try:
                status, detail = conn.recv()
            except EOFError:
                status, detail = 'failed', 'exited during start-up'
            if status != 'ready':
                self._drop(device, detail)
        if not self.workers:
            raise WorkerLost(f'no worker could be started: {self.lost}')

    @property
    def devices(self):
        return sorted(self.workers)

    def _drop(self, device, why):
        proc, conn = self.workers.pop(device)
        self.lost.append((device, why))
        try:
            conn.close()
        finally:
            if proc.is_alive():
                proc.terminate()
            proc.join(timeout=5)

    def new_task_id(self):
        """Every request carries an id of its own; a reply with another id is a leftover and is discarded."""
        self._next_id += 1
        return self._next_id

    def send(self, device, method, args):
        """Post one request to a worker; returns its task id (collect the reply with ``receive``)."""
        if device not in self.workers:
            raise WorkerLost(f'worker {device} is gone')
        task_id = self.new_task_id()
        try:
            self.workers[device][1].send((task_id, method, args))
        except (BrokenPipeError, OSError):
            self._drop(device, f'{method}: worker exited')
            raise WorkerLost(f'worker {device} exited before {method}')
        return task_id

    def receive(self, device, task_id, method='task', timeout=None):
        """The reply to ``task_id``: ``(status, value)``.  A worker that stays silent or exits is dropped."""
        if device not in self.workers:
            raise WorkerLost(f'worker {device} is gone')
        _, conn = self.workers[device]
        deadline = time.time() + (self.task_timeout if timeout is None else timeout)
        while True:
            if not conn.poll(max(0.0, deadline - time.time())):
                self._drop(device, f'{method} timed out')
                raise WorkerLost(f'worker {device} timed out in {method}')
            try:
                reply_id, status, value = conn.recv()
            except (EOFError, OSError):
                self._drop(device, f'{method}: worker exited')
                raise WorkerLost(f'worker {device} exited in {method}')
            if reply_id == task_id:
                return status, value

    def call(self, device, method, *args, timeout=None):
        """Run one task on a specific worker (used for per-device state such as engines)."""
        task_id = self.send(device, method, args)
        status, value = self.receive(device, task_id, method, timeout)
        if status != 'ok':
            raise RuntimeError(f'worker {device}: {value}')
        return value

    def broadcast(self, method, *args):
        return {device: self.call(device, method, *args) for device in self.devices}

    def map(self, method: str, arg_list: Sequence[tuple], on_result: Optional[Callable] = None) -> list:
        """Run ``method(*args)`` for every args tuple on whichever worker is free; results in task order."""
        results: List = [None] * len(arg_list)
        attempts = [0] * len(arg_list)
        queue = list(range(len(arg_list)))[::-1]
        busy: Dict[int, Tuple[int, float, int]] = {}     # device -> (task index, start time, task id)
        self.last_devices = [None] * len(arg_list)       # which device produced each result
        done = 0
        while done < len(arg_list):
            if not self.workers:
                raise WorkerLost(f'every worker was lost: {self.lost}')
            for device in self.devices:
                if device not in busy and queue:
                    index = queue.pop()
                    attempts[index] += 1
                    task_id = self.new_task_id()
                    try:
                        self.workers[device][1].send((task_id, method, arg_list[index]))
                    except (BrokenPipeError, OSError):
                        self._drop(device, f'exited before task {index}')
                        self._requeue(index, attempts, queue)
                        continue
                    busy[device] = (index, time.time(), task_id)
            conns = {self.workers[d][1]: d for d in busy}
            ready = mp.connection.wait(list(conns), timeout=1.0)
            for conn in ready:
                device = conns[conn]
                index, _, task_id = busy[device]
                try:
                    reply_id, status, value = conn.recv()
                except (EOFError, OSError):
                    busy.pop(device)
                    self._drop(device, f'exited while running task {index}')
                    self._requeue(index, attempts, queue)
                    continue
                if reply_id != task_id:
                    continue                                 # a leftover of an earlier, abandoned request
                busy.pop(device)
                if status != 'ok':
                    self._drain(busy)
                    raise RuntimeError(f'task {index} failed on worker {device}: {value}')
                results[index] = value
                self.last_devices[index] = device
                done += 1
                if on_result:
                    on_result(index, value)
            now = time.time()
            for device, (index, started, _) in list(busy.items()):
                if now - started > self.task_timeout:
                    busy.pop(device)
                    self._drop(device, f'task {index} timed out')
                    self._requeue(index, attempts, queue)
        return results

    def _drain(self, busy):
        """Before an error leaves ``map``: collect (or give up on) every reply that is still outstanding."""
        for device, (index, _, task_id) in list(busy.items()):
            try:
                self.receive(device, task_id, f'task {index}')
            except WorkerLost:
                pass
        busy.clear()

    def _requeue(self, index, attempts, queue):
        if attempts[index] >= self.max_attempts:
            raise WorkerLost(f'task {index} failed on {attempts[index]} workers')
        queue.append(index)

    def close(self):
        for device in list(self.workers):
            proc, conn = self.workers.pop(device)
            try:
                conn.send(None)
                conn.close()
            except (BrokenPipeError, OSError):
                pass
            proc.join(timeout=5)
            if proc.is_alive():
                proc.terminate()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


# ------------------------------------------------------------------------------------------------
# stage-profiling farm
# ------------------------------------------------------------------------------------------------
class _Recorder:
    """Cost model that only records what the search asks for."""
    _prefetching = True

    def __init__(self):
        self.requests: Dict[Tuple[str, str, int], None] = {}

    def get_stage_latency(self, stage, batch_size, warmup, number, repeat, profile_stage=False):
        from ios.contrib.ios_runtime import stage_config
        stage_json, input_json = stage_config(stage)
        self.requests.setdefault((stage_json, input_json, int(batch_size)), None)
        return [0.0] * repeat


class FarmCostModel:
    """
    Cost model for ``ios.optimize`` backed by a worker pool.  ``optimize`` calls
    ``prefetch_stages`` once; it replays the search's enumeration with a recording cost model (the
    set of candidate stages does not depend on the latencies), measures all candidates in parallel,
    and the real search then reads the memo.  All GPUs of one box are the same part at the same
    clocks; ``calibrate=True`` still measures one common stage on every worker first and multiplies
    each worker's later numbers by (median over workers) / (its own time for that stage); the
    factors are kept in ``self.scale``.
    """

    def __init__(self, pool: GpuWorkerPool, memo_path: Optional[str] = None, calibrate: bool = False):
        self.pool = pool
        self.memo: Dict[str, List[float]] = {}
        self.memo_path = memo_path
        self.calibrate = calibrate
        self.scale: Dict[int, float] = {}
        self.measured = 0
        if memo_path and os.path.exists(memo_path):
            self.load(memo_path)

    @staticmethod
    def _key(stage_json, input_json, batch, warmup, number, repeat):
        return json.dumps([stage_json, input_json, batch, warmup, number, repeat])

    def save(self, path):
        with open(path, 'w') as fh:
            json.dump(self.memo, fh)

    def load(self, path):
        with open(path) as fh:
            self.memo.update(json.load(fh))

    def _canonical(self, stage_json, input_json, batch, warmup, number, repeat):
        from ios.contrib.ios_runtime import canonical_stage_key
        return self._key(canonical_stage_key(stage_json, input_json), '', int(batch), warmup, number, repeat)

    def _measure(self, tasks):
        """
        Measure ``tasks`` -- tuples (stage json, input json, batch, warmup, number, repeat) -- in parallel on the pool,
        structurally equal ones only once, and store them in the memo.  With ``calibrate`` one common stage is first
        measured on every worker and each worker's numbers are multiplied by median / its own time for that stage.
        """
        todo, first = [], {}
        for task in tasks:
            key = self._canonical(*task)
            if key not in self.memo and key not in first:
                first[key] = len(todo)
                todo.append(task)
        if not todo:
            return
        if self.calibrate and not self.scale:
            times = self.pool.broadcast('stage_latency', *todo[0])
            ref = float(np.median([np.mean(t) for t in times.values()]))
            self.scale = {d: ref / float(np.mean(t)) for d, t in times.items()}
        values = self.pool.map('stage_latency', todo)
        for key, index in first.items():
            factor = self.scale.get(self.pool.last_devices[index], 1.0)
            self.memo[key] = [float(v) * factor for v in values[index]]
        self.measured += len(todo)
        if self.memo_path:
            self.save(self.memo_path)

    def prefetch_stages(self, graph, params):
        """The Python search asks for stages one by one: replay its enumeration first and measure everything at once."""
        from ios.optimizer import optimize
        recorder = _Recorder()
        optimize(graph, batch_size=params['batch_size'], cost_model=recorder, opt_type=params['opt_type'],
                 warmup=params['warmup'], number=params['number'], repeat=params['repeat'],
                 max_num_groups=params['max_num_groups'], max_part_size=params['max_part_size'],
                 max_group_size=params['max_group_size'], compute_weight=False)
        w, n, r = params['warmup'], params['number'], params['repeat']
        self._measure([(s, i, b, w, n, r) for (s, i, b) in recorder.requests])

    def get_stage_latency(self, stage, batch_size, warmup, number, repeat, profile_stage=False):
        return self.get_stage_latencies([stage], batch_size, warmup, number, repeat)[0]

    def get_stage_latencies(self, stages, batch_size, warmup, number, repeat):
        """Many candidate stages at once (what the native search asks for)."""
        from ios.contrib.ios_runtime import stage_config
        tasks = [(*stage_config(stage), int(batch_size), warmup, number, repeat) for stage in stages]
        self._measure(tasks)
        return [list(self.memo[self._canonical(*task)]) for task in tasks]

    def get_block_latency(self, block, batch_size, warmup, number, repeat, profile_stage=False):
        raise NotImplementedError('the DP search only asks for stage latencies')

    get_graph_latency = get_block_latency


# ------------------------------------------------------------------------------------------------
# batch sharding
# ------------------------------------------------------------------------------------------------
class ShardedInference:
    """
    Run a graph on a batch split across the pool's GPUs.  ``graph_for_batch(b)`` returns the graph
    (with weights and a schedule) to use for a shard of ``b`` images -- IOS schedules are
    specialised to the batch size -- and defaults to the given graph for every size.

    Input and output live in two shared-memory arrays (``self.input``, ``self.output``) that every
    worker maps and page-locks for its own slice, so a run moves no tensor between processes: the
    parent writes the batch into ``self.input`` (or passes it to ``run``, which copies it there),
    each worker uploads its slice straight from the shared pages and downloads into them.
    """

    def __init__(self, pool: GpuWorkerPool, graph, batch: int, graph_for_batch: Optional[Callable] = None):
        from multiprocessing import shared_memory
        self.pool = pool
        self.batch = batch
        self.slices = plan_shards(batch, len(pool.devices))
        self.devices = pool.devices[:len(self.slices)]
        self.output_shape = None
        self.key = f'shard-{id(self)}'
        in_shape = (batch, *graph.input.output_shape)
        for device, (begin, end) in zip(self.devices, self.slices):
            shard_graph = graph_for_batch(end - begin) if graph_for_batch else graph
            weights = {conv.name: (conv.weight, conv.bias) for conv in shard_graph.convs()}
            shape = pool.call(device, 'engine_create', self.key, json.dumps(shard_graph.export_config()), end - begin,
                              weights, timeout=600)
            self.output_shape = (batch, *shape[1:])
        self._shm_in = shared_memory.SharedMemory(create=True, size=max(4, int(np.prod(in_shape)) * 4))
        self._shm_out = shared_memory.SharedMemory(create=True, size=max(4, int(np.prod(self.output_shape)) * 4))
        self.input = np.ndarray(in_shape, dtype=np.float32, buffer=self._shm_in.buf)
        self.output = np.ndarray(self.output_shape, dtype=np.float32, buffer=self._shm_out.buf)
        self.pinned = True
        for device, (begin, end) in zip(self.devices, self.slices):
            ok = pool.call(device, 'engine_attach', self.key, self._shm_in.name, self._shm_out.name, in_shape,
                           self.output_shape, begin, end)
            self.pinned = self.pinned and bool(ok)

    def run(self, x: Optional[np.ndarray] = None, repeats: int = 1) -> np.ndarray:
        """
        One pass over the batch (``repeats`` > 1: the same batch that many times through the pipelined
        entry point, for timing).  ``x`` = None runs on what is already in ``self.input``.  Every shard is
        issued before any reply is collected; all replies are collected (or their workers dropped) before
        an error is raised, so a failed run never leaves a stale reply for the next one.
        """
        if x is not None:
            if x.shape[0] != self.batch:
                raise ValueError(f'expected a batch of {self.batch}, got {x.shape[0]}')
            np.copyto(self.input, x, casting='same_kind')
        pending, failure = [], None
        for device in self.devices:
            try:
                pending.append((device, self.pool.send(device, 'engine_run_shared', (self.key, repeats))))
            except WorkerLost as err:
                failure = failure or err
        for device, task_id in pending:
            try:
                status, value = self.pool.receive(device, task_id, 'engine_run_shared')
                if status != 'ok':
                    failure = failure or RuntimeError(f'worker {device}: {value}')
            except WorkerLost as err:
                failure = failure or err
        if failure is not None:
            raise failure
        return self.output.copy()

    def close(self):
        for device in self.devices:
            if device in self.pool.workers:
                try:
                    self.pool.call(device, 'engine_detach', self.key)
                except (WorkerLost, RuntimeError):
                    pass
        self.input = self.output = None
        for shm in (self._shm_in, self._shm_out):
            try:
                shm.close()
                shm.unlink()
            except (FileNotFoundError, BufferError):
                pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def gather_to_rank0(local: np.ndarray, batch: int, group=None) -> Optional[np.ndarray]:
    """
    For one-process-per-GPU jobs (torchrun): every rank passes the output of its shard
    (``shard_slices(batch, world)[rank]``); rank 0 receives the whole batch, the others ``None``.
    Host-side gather over the process group (gloo or nccl) AFTER the last kernel: nothing on the
    inference path waits on another GPU.
    """
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    pieces = [None] * world if rank == 0 else None
    dist.gather_object(np.ascontiguousarray(local), pieces, dst=0, group=group)
    if rank != 0:
        return None
    slices = shard_slices(batch, world)
    out = np.empty((batch, *local.shape[1:]), dtype=local.dtype)
    for piece, (begin, end) in zip(pieces, slices):
        out[begin:end] = piece
    return out
