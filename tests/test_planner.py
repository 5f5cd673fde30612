"""
The planner's choices, checked without a GPU: `ios_plan_describe` lays a scheduled graph out for a 148-SM device
and reports every convolution's kernel and tiling.  These are the invariants a launch depends on (shared memory within
what a CTA may have, a receive area that fits behind the pipeline, a workspace where one is needed, clusters of at most
eight CTAs ...), over the model zoo, three batch sizes and the three tensor-core precisions.
"""
import math

import pytest

import ios
from ios.contrib import ios_runtime as rt

SMEM_LIMIT = 225 * 1024          # dynamic shared memory the convolution kernels may ask for
OPTIONS = (('precision', 'tf32x3'), ('cluster_push', '1'), ('dual_issue', '1'), ('persistent', '1'), ('patch', '1'),
           ('split_k', '0'), ('bn', '0'), ('stages', '0'))


@pytest.fixture(autouse=True)
def default_options():
    for key, value in OPTIONS:
        rt.set_option(key, value)
    yield
    for key, value in OPTIONS:
        rt.set_option(key, value)


def _graph(model):
    graph = getattr(ios.models, model)()
    graph.greedy_schedule()
    return graph


def _check_convolution(c, precision, sms=148):
    if c['kind'] != 'tensor':
        return
    assert c['bn'] % (64 if precision == 'bf16' else 32) == 0 and 32 <= c['bn'] <= 256, c
    assert c['n_tiles'] * c['bn'] >= c['cout'], c
    assert c['stages'] >= 2 or c['patch'], c
    assert 1 <= c['split_k'] <= max(1, c['k_iters']), c
    assert c['smem_bytes'] <= SMEM_LIMIT, c
    if c['patch']:
        return
    if c['persistent']:
        assert c['split_k'] == 1, c
        assert c['grid_ctas'] in (sms, 2 * sms), c
    if c['split_k'] > 1:
        assert c['cluster'] == (1 if c['split_k'] <= 8 else 0), c
        tiles = c['grid_ctas'] // c['split_k']
        if c['push']:
            assert c['cluster'] == 1 and c['workspace_bytes'] == 0, c
            assert c['recv_off'] % 16 == 0 and c['stages'] >= 2, c
            receive = c['split_k'] * math.ceil(128 / c['split_k']) * c['bn'] * 4
            assert c['recv_off'] + receive + 1024 == c['smem_bytes'], c
        else:
            assert c['workspace_bytes'] >= tiles * c['split_k'] * c['bn'] * 128 * 4, c
    else:
        assert not c['push'] and c['workspace_bytes'] == 0, c
    # tensor-memory columns (power of two, at most 512): accumulator ranges of the issuing threads
    clustered = c['split_k'] > 1 and c['cluster']
    ranges = 1
    if not c['persistent']:
        if c['x3'] and c['bn'] <= 128:
            ranges = 3 if 3 * c['bn'] <= (512 if clustered else 256) else 2
        elif not c['x3'] and 2 * c['bn'] <= (512 if clustered else 256):
            ranges = 2
    assert ranges * c['bn'] <= 512, c


@pytest.mark.parametrize('precision', ['tf32x3', 'tf32', 'bf16'])
@pytest.mark.parametrize('batch', [1, 16, 256])
@pytest.mark.parametrize('model', ['inception_v3', 'squeezenet', 'randwire_small', 'resnet18'])
def test_every_planned_convolution_can_be_launched(model, batch, precision):
    rt.set_option('precision', precision)
    plan = rt.plan_describe(_graph(model), batch)
    assert plan['arena_bytes'] > 0 and plan['launches'] >= len(plan['convolutions']) > 0
    for c in plan['convolutions']:
        _check_convolution(c, precision)


def test_batch_one_defaults_of_inception_v3():
    graph = ios.models.inception_v3()
    graph.sequential_schedule()
    plan = rt.plan_describe(graph, 1)
    convs = plan['convolutions']
    assert plan['launches'] == 108 and len(convs) == 94
    pushed = [c for c in convs if c['push']]
    assert len(pushed) >= 80 and all(c['x3'] for c in convs)          # the split-K layers exchange through shared memory
    rt.set_option('cluster_push', '0')
    fallback = rt.plan_describe(graph, 1)['convolutions']
    assert not any(c['push'] for c in fallback)
    assert all(c['workspace_bytes'] > 0 for c in fallback if c['split_k'] > 1)
    # the exchange form does not change tile widths or splits
    assert [(c['bn'], c['split_k']) for c in fallback] == [(c['bn'], c['split_k']) for c in convs]


def test_other_device_sizes_and_bad_arguments():
    graph = _graph('squeezenet')
    small = rt.plan_describe(graph, 8, sm_count=64)
    large = rt.plan_describe(graph, 8, sm_count=148)
    assert len(small['convolutions']) == len(large['convolutions'])
    for c in small['convolutions']:
        _check_convolution(c, 'tf32x3', 64)
    for c in large['convolutions']:
        _check_convolution(c, 'tf32x3', 148)
    with pytest.raises(RuntimeError):
        rt.plan_describe(graph, 0)
