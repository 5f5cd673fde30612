"""
The multi-GPU helpers against a real device: worker processes bound to GPUs run shards of a batch
and farmed stage measurements through the C-ABI.  With one GPU present the pool has one worker.
"""
import json

import numpy as np
import pytest

import ios
import ios_oracle as oracle
from ios import distributed as D
from ios.contrib import ios_runtime as rt
from helpers import TOL_TF32, sample_block, seeded

pytestmark = pytest.mark.gpu


def _devices(limit=2):
    return list(range(min(limit, rt.device_count())))


def test_sharded_inference_matches_oracle():
    graph = ios.models.squeezenet()
    graph.sequential_schedule()
    config, weights = seeded(graph, 0)
    batch = 18
    x = oracle.normal_input(config, batch, 3)
    ref = oracle.run_config(config, weights, x)
    with D.GpuWorkerPool(_devices()) as pool:
        with D.ShardedInference(pool, graph, batch) as sharded:
            assert sum(e - b for b, e in sharded.slices) == batch and len(sharded.slices) == len(pool.devices)
            assert sharded.pinned                   # every worker page-locked its slice of the shared arrays
            y = sharded.run(x)
            assert y.shape == ref.shape
            assert oracle.max_rel_err(y, ref) <= TOL_TF32
            sharded.input[...] = x[::-1]            # written in place; three pipelined passes over the same batch
            y = sharded.run(repeats=3)
            assert oracle.max_rel_err(y, ref[::-1]) <= TOL_TF32


def test_stage_farm_drives_the_search():
    graph = sample_block()
    config, weights = seeded(graph, 0)
    with D.GpuWorkerPool(_devices()) as pool:
        farm = D.FarmCostModel(pool)
        opt = ios.optimize(graph, batch_size=1, cost_model=farm, opt_type='dp_parallel_merge', compute_weight=True,
                           number=2, repeat=2)
        assert farm.measured >= 20 and all(np.isfinite(v).all() and min(v) > 0 for v in farm.memo.values())
    names = sorted(n for stage in opt.blocks[0].stages for group in stage for n in group)
    assert len(names) >= 2
    x = oracle.normal_input(config, 1, 0)
    y = rt.graph_inference(opt, 1, x)
    assert oracle.max_rel_err(y, oracle.run_config(config, weights, x)) <= TOL_TF32
