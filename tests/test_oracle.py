"""
The CPU oracle against the golden vectors produced by the reference's own package
(tests/golden/make_golden.py), and its two back-ends against each other.  No GPU.
"""
import json
import os

import numpy as np
import pytest

import ios
import ios_oracle as oracle
from helpers import GOLDEN_DIR, load_ref_schedule, sample_block, seeded, sha

# the oracle and the reference executor both run torch's CPU float32 kernels, possibly with a
# different thread count and summation order
ORACLE_TOL = 2e-5


def _model(name):
    if name == 'sample_block':
        return sample_block()
    return getattr(ios.models, name)()


@pytest.mark.parametrize('case,model,law,wseed,xseed,batch', [
    ('sample_block', 'sample_block', 'he', 0, 0, 1),
    ('inception_v3', 'inception_v3', 'he', 0, 0, 1),
    ('inception_v3_uniform_b2', 'inception_v3', 'uniform', 1, 1, 2),
    ('squeezenet', 'squeezenet', 'he', 0, 0, 1),
    ('randwire_small', 'randwire_small', 'he', 0, 0, 1),
    ('resnet18', 'resnet18', 'he', 0, 0, 1),            # residual adds are element nodes
    ('resnet34', 'resnet34', 'he', 0, 0, 1),
    ('nasnet_large', 'nasnet_large', 'he', 0, 0, 1),    # one block of 370 schedule units, ReLU-separable convolutions
])
def test_oracle_matches_reference_outputs(golden, case, model, law, wseed, xseed, batch):
    graph = _model(model)
    graph.sequential_schedule()
    config, weights = seeded(graph, wseed, law)
    assert sha(config) == golden.meta(case)['config_sha256'], 'the exported graph differs from the reference export'
    x = oracle.normal_input(config, batch, xseed)
    y = oracle.run_config(config, weights, x)
    golden.expect(case, y, ORACLE_TOL)


def test_oracle_all_operator_types(golden):
    with open(os.path.join(GOLDEN_DIR, 'all_ops.json')) as fh:
        config = json.load(fh)
    weights = oracle.uniform_weights(config, 3)
    x = oracle.normal_input(config, 3, 4)
    y_torch = oracle.run_config(config, weights, x)
    golden.expect('all_ops_b3', y_torch, ORACLE_TOL)
    y_numpy = oracle.run_config_numpy(config, weights, x)
    golden.expect('all_ops_b3', y_numpy, ORACLE_TOL)
    y_double = oracle.run_config(config, weights, x, double=True)
    assert oracle.max_rel_err(y_numpy, y_double) < 1e-12


@pytest.mark.parametrize('name', ['1', '16', '32', '64', '128', 'k80', 'v100'])
def test_oracle_runs_reference_schedules(golden, name):
    config = load_ref_schedule(name)
    graph = ios.Graph.from_config(config)
    config = graph.export_config()
    weights = oracle.he_normal_weights(config, 0)
    y = oracle.run_config(config, weights, oracle.normal_input(config, 1, 0))
    golden.expect('ref_schedule_' + name, y, ORACLE_TOL)


@pytest.mark.parametrize('shape', [
    # n, cin, h, w, cout, kh, kw, sh, sw, ph, pw, groups
    (2, 5, 9, 7, 6, 3, 3, 1, 1, 1, 1, 1),
    (1, 8, 11, 11, 12, 1, 7, 1, 1, 0, 3, 1),
    (1, 6, 12, 10, 6, 3, 3, 2, 2, 1, 1, 6),
    (3, 4, 8, 8, 10, 5, 5, 2, 1, 2, 2, 2),
])
def test_numpy_conv_equals_torch_conv(shape):
    import torch
    n, cin, h, w, cout, kh, kw, sh, sw, ph, pw, groups = shape
    rng = np.random.default_rng(5)
    x = rng.standard_normal((n, cin, h, w))
    wt = rng.standard_normal((cout, cin // groups, kh, kw))
    b = rng.standard_normal(cout)
    ref = torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(wt), torch.from_numpy(b), (sh, sw),
                                     (ph, pw), 1, groups).numpy()
    got = oracle.conv2d_numpy(x, wt, b, (sh, sw), (ph, pw), groups)
    assert got.shape == ref.shape
    assert np.max(np.abs(got - ref)) < 1e-10


def test_numpy_pools_equal_torch_pools():
    import torch
    x = np.random.default_rng(6).standard_normal((2, 3, 9, 8))
    t = torch.from_numpy(x)
    F = torch.nn.functional
    assert np.allclose(oracle.pool2d_numpy(x, 'max', (3, 3), (2, 2), (1, 1)), F.max_pool2d(t, 3, 2, 1).numpy())
    assert np.allclose(oracle.pool2d_numpy(x, 'avg', (3, 3), (1, 1), (1, 1)),
                       F.avg_pool2d(t, 3, 1, 1, count_include_pad=True).numpy())
    assert np.allclose(oracle.pool2d_numpy(x, 'global_avg', None, None, None), x.mean(axis=(2, 3), keepdims=True))
