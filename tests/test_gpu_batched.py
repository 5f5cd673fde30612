"""
GPU parity at the batch sizes of the throughput configurations: Inception-v3 at batch 16 / 64 / 256
through the engine (the call a serving process makes), against the CPU oracle on the same seeded
He-normal weights and inputs.  At these sizes other kernels take over than at batch 1 -- resident
CTAs that walk the tiles, the CUDA-core kernel for the 3-channel stem, 64-byte operand rows in
bfloat16 -- and the tests assert from the engine's description that they really ran.

Tolerances (max|y - ref| / max|ref|): 1e-3 for three-pass TF32, 2e-2 for bfloat16.
"""
import numpy as np
import pytest

import ios
import ios_oracle as oracle
from ios.contrib import ios_runtime as rt
from helpers import TOL_BF16, TOL_TF32, oracle_in_chunks, seeded

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def default_options():
    for key, value in (('precision', 'tf32x3'), ('pdl', '1'), ('executor', 'graph'), ('conv', 'auto'), ('split_k', '0'),
                       ('im2col', '1'), ('persistent', '1'), ('stem', '1'), ('bulk_store', '1'), ('stage_barriers', '1'),
                       ('pdl_edges', '0')):
        rt.set_option(key, value)
    yield
    rt.set_option('precision', 'tf32x3')


@pytest.fixture(scope='module')
def inception():
    graph = ios.models.inception_v3()
    config, weights = seeded(graph, 0)
    refs = {}

    def reference(batch):
        if batch not in refs:
            x = oracle.normal_input(config, batch, 0)
            refs[batch] = (x, oracle_in_chunks(config, weights, x))
        return refs[batch]

    return graph, config, weights, reference


def _run(graph, batch, x, precision):
    rt.set_option('precision', precision)
    engine = rt.Engine(graph, batch)
    try:
        return engine.run(x), engine.describe()
    finally:
        engine.close()


@pytest.mark.parametrize('batch,precision,tol', [
    (16, 'tf32x3', TOL_TF32), (16, 'bf16', TOL_BF16), (64, 'tf32x3', TOL_TF32), (64, 'bf16', TOL_BF16),
    (256, 'bf16', TOL_BF16)])
def test_inception_v3_batched_greedy_schedule(inception, batch, precision, tol):
    graph, config, weights, reference = inception
    graph.greedy_schedule()
    x, ref = reference(batch)
    y, info = _run(graph, batch, x, precision)
    err = oracle.max_rel_err(y, ref)
    assert err <= tol, f'batch {batch} {precision}: {err:.3e}'
    assert info['conv_tc_persistent'] > 0, info            # resident CTAs walking the tiles
    assert info['conv_few_channels'] > 0, info             # the 3-channel stem on CUDA cores
    if precision == 'bf16':
        assert info['conv_tc_half_rows'] > 0, info         # 32-channel layers with 64-byte operand rows
    assert info['precision'] == precision


@pytest.mark.parametrize('precision,tol', [('tf32x3', TOL_TF32), ('bf16', TOL_BF16)])
def test_inception_v3_batch_16_measured_dp_schedule(inception, precision, tol):
    """A schedule found by the DP search on latencies measured at this batch size and precision."""
    graph, config, weights, reference = inception
    rt.set_option('precision', precision)
    opt = ios.optimize(graph, batch_size=16, opt_type='dp_parallel_merge', compute_weight=True, max_part_size=50,
                       warmup=1, number=2, repeat=1)
    x, ref = reference(16)
    y, info = _run(opt, 16, x, precision)
    err = oracle.max_rel_err(y, ref)
    assert err <= tol, f'{precision}: {err:.3e}'
    assert info['conv_tc_persistent'] > 0 and info['stages'] < 119


def test_single_pass_tf32_batch_16_stays_within_its_known_growth(inception):
    graph, config, weights, reference = inception
    graph.greedy_schedule()
    x, ref = reference(16)
    y, info = _run(graph, 16, x, 'tf32')
    assert oracle.max_rel_err(y, ref) <= 6e-3
