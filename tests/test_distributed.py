"""
Host-side logic of the multi-GPU paths, on CPU: shard planning, the worker pool with injected
host failures (a worker that exits, one that never answers, one that cannot start), the
stage-profiling farm against a deterministic fake backend, and a world-size-2 gloo gather.
No GPU is touched and no device fault is provoked.
"""
import json
import os
import socket

import numpy as np
import pytest
import torch.multiprocessing as tmp

import ios
from ios import distributed as D
from fake_backends import (AlwaysDies, DiesOnDeviceOne, FailsToStart, FakeBackend, HangsOnDeviceOne, fake_latency)
from helpers import sample_block


def test_shard_slices_cover_the_batch_evenly():
    for batch in (1, 15, 16, 17, 64, 250, 256):
        for parts in (1, 2, 4, 8):
            slices = D.shard_slices(batch, parts)
            assert slices[0][0] == 0 and slices[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(slices, slices[1:]))
            sizes = [e - b for b, e in slices]
            assert max(sizes) - min(sizes) <= 1
    assert D.plan_shards(8, 8) == [(0, 8)]                       # below 16 images: one GPU
    assert D.plan_shards(16, 8) == [(2 * i, 2 * i + 2) for i in range(8)]
    assert len(D.plan_shards(256, 4)) == 4
    with pytest.raises(ValueError):
        D.shard_slices(4, 0)


def test_pool_maps_tasks_in_order():
    with D.GpuWorkerPool([0, 1, 2], FakeBackend) as pool:
        out = pool.map('echo', [(i,) for i in range(20)])
        assert [v for _, v in out] == list(range(20))
        assert {d for d, _ in out} <= {0, 1, 2}
        assert pool.call(2, 'echo', 'x') == (2, 'x')


def test_pool_requeues_the_task_of_a_worker_that_exits():
    with D.GpuWorkerPool([0, 1], DiesOnDeviceOne) as pool:
        out = pool.map('echo', [(i,) for i in range(8)])
        assert [v for _, v in out] == list(range(8))
        assert all(d == 0 for d, _ in out)
        assert pool.devices == [0] and pool.lost[0][0] == 1


def test_pool_drops_a_worker_that_never_answers():
    with D.GpuWorkerPool([0, 1], HangsOnDeviceOne, task_timeout=1.5) as pool:
        out = pool.map('echo', [(i,) for i in range(4)])
        assert [v for _, v in out] == list(range(4))
        assert pool.devices == [0]


def test_pool_reports_total_loss():
    with D.GpuWorkerPool([0, 1], AlwaysDies) as pool:
        with pytest.raises(D.WorkerLost):
            pool.map('echo', [(1,), (2,), (3,)])
    with pytest.raises(D.WorkerLost):
        D.GpuWorkerPool([0], FailsToStart)


class _DirectFake(ios.cost_model.CostModel):
    def get_stage_latency(self, stage, batch_size, warmup, number, repeat, profile_stage=False):
        from ios.contrib.ios_runtime import stage_config
        s, i = stage_config(stage)
        return [fake_latency(s, i, int(batch_size))] * repeat


def test_farm_gives_the_same_schedule_as_direct_measurement(tmp_path):
    graph = ios.models.squeezenet()
    direct = ios.optimize(graph, batch_size=1, cost_model=_DirectFake(), opt_type='dp_parallel_merge')
    memo = str(tmp_path / 'memo.json')
    with D.GpuWorkerPool([0, 1, 2, 3], FakeBackend) as pool:
        farm = D.FarmCostModel(pool, memo_path=memo)
        farmed = ios.optimize(graph, batch_size=1, cost_model=farm, opt_type='dp_parallel_merge')
        assert farm.measured > 100
        assert json.dumps(farmed.export_config()) == json.dumps(direct.export_config())
        # a second search resumes from the saved memo and measures nothing
        again = D.FarmCostModel(pool, memo_path=memo)
        ios.optimize(graph, batch_size=1, cost_model=again, opt_type='dp_parallel_merge')
        assert again.measured == 0


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _gloo_rank(rank, world, port, batch, out_dir):
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    begin, end = D.shard_slices(batch, world)[rank]
    full = np.arange(batch * 3, dtype=np.float32).reshape(batch, 3)
    local = full[begin:end] * 2.0                       # each rank's "inference" on its shard
    gathered = D.gather_to_rank0(local, batch)
    if rank == 0:
        np.save(os.path.join(out_dir, 'gathered.npy'), gathered)
    else:
        assert gathered is None
    dist.destroy_process_group()


def test_gloo_world_size_2_gather(tmp_path):
    batch = 17
    tmp.spawn(_gloo_rank, args=(2, _free_port(), batch, str(tmp_path)), nprocs=2, join=True)
    got = np.load(str(tmp_path / 'gathered.npy'))
    assert np.array_equal(got, np.arange(batch * 3, dtype=np.float32).reshape(batch, 3) * 2.0)


def _sharded_case(batch=18):
    graph = sample_block()
    graph.sequential_schedule()
    x = np.random.default_rng(0).standard_normal((batch, 375, 15, 15)).astype(np.float32)
    return graph, x, x.sum(axis=(2, 3), keepdims=True)


def test_sharded_inference_through_shared_memory():
    from fake_backends import FakeEngineBackend
    graph, x, expect = _sharded_case()
    with D.GpuWorkerPool([0, 1, 2], FakeEngineBackend) as pool:
        with D.ShardedInference(pool, graph, x.shape[0]) as sharded:
            assert [e - b for b, e in sharded.slices] == [6, 6, 6] and not sharded.pinned
            assert np.allclose(sharded.run(x), expect, rtol=1e-5)
            sharded.input[...] = 2.0 * x                      # written in place: no copy through run()
            assert np.allclose(sharded.run(), 2.0 * expect, rtol=1e-5)
            with pytest.raises(ValueError):
                sharded.run(x[:5])


def test_a_failed_shard_does_not_poison_the_next_run():
    """Shard 0 raises once: the error surfaces, every other reply is collected, and the next run is right."""
    from fake_backends import FakeEngineFailsOnceOnDeviceZero
    graph, x, expect = _sharded_case()
    with D.GpuWorkerPool([0, 1], FakeEngineFailsOnceOnDeviceZero) as pool:
        with D.ShardedInference(pool, graph, x.shape[0]) as sharded:
            with pytest.raises(RuntimeError, match='injected'):
                sharded.run(x)
            assert np.allclose(sharded.run(3.0 * x), 3.0 * expect, rtol=1e-4, atol=1e-3)
            assert pool.call(1, 'echo', 'still in step') == (1, 'still in step')


def test_stale_replies_are_discarded_by_task_id():
    with D.GpuWorkerPool([0], FakeBackend) as pool:
        abandoned = pool.send(0, 'echo', ('old',))            # a request whose reply nobody collects
        assert pool.call(0, 'echo', 'new') == (0, 'new')       # the leftover reply is skipped, not returned
        assert abandoned != pool.new_task_id()


def test_farm_calibration_is_applied_to_the_measurements():
    from fake_backends import SlowOnDeviceOne
    graph = sample_block()
    with D.GpuWorkerPool([0, 1, 2], SlowOnDeviceOne) as pool:
        farm = D.FarmCostModel(pool, calibrate=True)
        ios.optimize(graph, batch_size=1, cost_model=farm, opt_type='dp_parallel_merge')
        assert abs(farm.scale[1] - 0.5) < 1e-9 and abs(farm.scale[0] - 1.0) < 1e-9
        from fake_backends import fake_latency_of_structure
        for key, value in farm.memo.items():
            canonical, _, batch = json.loads(key)[:3]
            assert abs(value[0] - fake_latency_of_structure(canonical, batch)) < 1e-9
