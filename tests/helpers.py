"""Shared helpers of the test-suite: golden fixtures, seeded graphs, weight transfer."""
import gzip
import hashlib
import json
import os

import numpy as np

import ios
import ios_oracle as oracle

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')

# tolerances of the parity contract: max|y - ref| / max|ref|
TOL_TF32 = 1e-3     # TF32 products, fp32 accumulate
TOL_FP32 = 2e-5     # CUDA-core fp32 path against an fp32/fp64 oracle
TOL_BF16 = 2e-2     # bfloat16 storage and products, fp32 accumulate


class Golden:
    def __init__(self):
        self.arrays = np.load(os.path.join(GOLDEN_DIR, 'golden.npz'))
        with open(os.path.join(GOLDEN_DIR, 'manifest.json')) as fh:
            self.manifest = json.load(fh)

    def vector(self, case):
        return self.arrays[case]

    def meta(self, case):
        return self.manifest[case]

    def expect(self, case, y, tol):
        """Compare a full output with the stored (possibly sub-sampled) reference vector."""
        meta = self.manifest[case]
        assert list(y.shape) == meta['output_shape'], (y.shape, meta['output_shape'])
        got = np.asarray(y, dtype=np.float32).reshape(-1)[::meta.get('subsample', 1)]
        err = oracle.max_rel_err(got, self.arrays[case])
        assert err <= tol, f'{case}: max relative error {err:.3e} exceeds {tol:.1e}'
        return err


def load_golden():
    return Golden()


def sha(config):
    return hashlib.sha256(json.dumps(config).encode()).hexdigest()


def load_ref_schedule(name):
    with gzip.open(os.path.join(GOLDEN_DIR, 'ref_schedules', name + '.json.gz'), 'rb') as fh:
        return json.loads(fh.read().decode())


def set_weights(graph, weights):
    """Assign ``{conv name: (weight, bias)}`` to the Conv nodes of a graph (inside Sequential too)."""
    for conv in graph.convs():
        conv.weight, conv.bias = weights[conv.name]


def weights_of(graph):
    return {conv.name: (conv.weight, conv.bias) for conv in graph.convs()}


def sample_block():
    """The README sample block: four 3x3 convolutions and a concat (reference examples/sample.py)."""
    ios.reset_name()
    v = ios.placeholder(output_shape=(375, 15, 15))
    block = ios.Block(enter_node=v.node)
    v1 = ios.conv2d(block, inputs=[[v]], out_channels=375, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
    v2 = ios.conv2d(block, inputs=[[v]], out_channels=750, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
    v3 = ios.conv2d(block, inputs=[[v]], out_channels=375, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
    v1 = ios.conv2d(block, inputs=[[v1]], out_channels=750, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
    ios.identity(block, inputs=[[v1], [v2], [v3]], is_exit=True)
    graph = ios.Graph(name="demo", input=v.node, blocks=[block])
    graph.init_weights()
    return graph


def seeded(graph, wseed=0, law='he'):
    """Give the graph the oracle's seeded weights; returns (config, weights)."""
    config = graph.export_config()
    weights = (oracle.he_normal_weights if law == 'he' else oracle.uniform_weights)(config, wseed)
    set_weights(graph, weights)
    return config, weights


def has_gpu():
    try:
        return ios.ios_runtime.device_count() > 0
    except Exception:
        return False


def oracle_in_chunks(config, weights, x, chunk=16):
    """The oracle over a large batch, a few images at a time (every operator is per image): bounded host memory."""
    parts = [oracle.run_config(config, weights, x[i:i + chunk]) for i in range(0, x.shape[0], chunk)]
    return np.concatenate(parts, axis=0)
