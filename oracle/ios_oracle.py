"""
CPU oracle for the IOS execution path.  TEST INFRASTRUCTURE ONLY: nothing in the product imports
this file; only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may.

It restates, on the host, what the reference computes when it executes a graph:

* the graph walk and the input algebra -- every operator's input is the concatenation over terms of
  the sum (product for an ``element`` operator with ``op_type == 'mul'``) over values of channel
  slices of earlier outputs -- follow the reference's own CPU executor, ``ios.torch_utils.Net.forward``
  (reference ``python/ios/torch_utils.py:79-125``), which is also what its CUDA runtime does in
  ``Input/Term/Value::forward`` (``src/ios/ios_runtime.cu:652-812``);
* convolution = cross-correlation, dilation 1, zero padding, groups, bias, then the activation
  (``src/ios/ios_runtime.cu:207-332``, ``torch_utils.py:9-27``); output extent ``1 + (in - k + 2p) // s``;
* pooling: max ignores the padding; avg divides by the full window, padding included
  (``CUDNN_POOLING_AVERAGE_COUNT_INCLUDE_PADDING``, ``src/ios/ios_runtime.cu:542-550``; torch's
  ``AvgPool2d`` default); global pooling is a window equal to the input (``:1051-1057``).

Two implementations are kept: ``run_config`` uses torch's CPU float32/float64 convolutions (fast
enough for the full networks) and ``run_config_numpy`` uses explicit NumPy loops (small cases only)
so that the torch path is itself cross-checked.  Parity pin: tests/golden/ holds outputs produced
by the reference's own package (``ios.torch_utils.Net``) on the same seeded weights and inputs;
tests/test_oracle.py checks this oracle against them.

The graphs are taken in the JSON wire format (``Graph.export_config()``), so the oracle does not
depend on the package under test.
"""
import math
from typing import Dict, Iterable, Tuple

import numpy as np

Weights = Dict[str, Tuple[np.ndarray, np.ndarray]]


# --------------------------------------------------------------------------------------------
# seeded synthetic data
# --------------------------------------------------------------------------------------------
def iter_conv_configs(config) -> Iterable[dict]:
    """Convolution node configs of a graph config in graph order (inside ``sequential`` nodes too)."""
    def walk(nodes):
        for node in nodes:
            if node['type'] == 'conv':
                yield node
            elif node['type'] == 'sequential':
                yield from walk(node['nodes'])
    for block in config['blocks']:
        yield from walk(block['inner_nodes'])
        yield from walk([block['exit_node']])


def _shapes(config):
    """name -> (C, H, W) of every node, re-inferred from the config (output_shape may be null)."""
    shapes = {config['input']['name']: tuple(config['input']['output_shape'])}

    def input_shape(node):
        terms = node['inputs']
        c = sum(terms_[0][2] - terms_[0][1] for terms_ in terms)
        _, h, w = shapes[terms[0][0][0]]
        return c, h, w

    def visit(node):
        kind = node['type']
        if kind == 'sequential':
            for sub in node['nodes']:
                visit(sub)
            shapes[node['name']] = shapes[node['nodes'][-1]['name']]
            return
        c, h, w = input_shape(node)
        if kind == 'conv':
            k, s, p = node['kernel'], node['stride'], node['padding']
            shapes[node['name']] = (node['out_channels'], 1 + (h - k[0] + 2 * p[0]) // s[0],
                                    1 + (w - k[1] + 2 * p[1]) // s[1])
        elif kind == 'pool':
            if 'global' in node['pool_type']:
                k, s, p = (h, w), (1, 1), (0, 0)
            else:
                k, s, p = node['kernel'], node['stride'], node['padding']
            shapes[node['name']] = (c, 1 + (h - k[0] + 2 * p[0]) // s[0], 1 + (w - k[1] + 2 * p[1]) // s[1])
        else:
            shapes[node['name']] = (c, h, w)
        shapes.setdefault('__in__' + node['name'], (c, h, w))

    for block in config['blocks']:
        for node in block['inner_nodes']:
            visit(node)
        visit(block['exit_node'])
    return shapes


def conv_weight_shapes(config) -> Dict[str, Tuple[int, int, int, int]]:
    shapes = _shapes(config)
    out = {}
    for node in iter_conv_configs(config):
        cin = shapes['__in__' + node['name']][0]
        out[node['name']] = (node['out_channels'], cin // node['groups'], node['kernel'][0], node['kernel'][1])
    return out


def he_normal_weights(config, seed: int) -> Weights:
    """He-normal weights N(0, 2/fan_in), fan_in = kh*kw*Cin/groups, zero bias; one generator, graph order."""
    rng = np.random.default_rng(seed)
    weights = {}
    for name, shape in conv_weight_shapes(config).items():
        fan_in = shape[1] * shape[2] * shape[3]
        w = (rng.standard_normal(shape) * math.sqrt(2.0 / fan_in)).astype(np.float32)
        weights[name] = (w, np.zeros(shape[0], dtype=np.float32))
    return weights


def uniform_weights(config, seed: int) -> Weights:
    """The reference's own initialisation law (U(-b, b), b = 1/sqrt(fan_in), bias too; ``ir.py:360-363``), seeded."""
    rng = np.random.default_rng(seed)
    weights = {}
    for name, shape in conv_weight_shapes(config).items():
        bound = 1.0 / math.sqrt(shape[1] * shape[2] * shape[3])
        w = rng.uniform(-bound, bound, size=shape).astype(np.float32)
        b = rng.uniform(-bound, bound, size=shape[0]).astype(np.float32)
        weights[name] = (w, b)
    return weights


def normal_input(config, batch: int, seed: int) -> np.ndarray:
    shape = (batch, *config['input']['output_shape'])
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def max_rel_err(y: np.ndarray, ref: np.ndarray) -> float:
    """max|y - ref| / max|ref|: the metric the tolerances are stated in."""
    ref64 = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(y, dtype=np.float64) - ref64)) / max(np.max(np.abs(ref64)), 1e-30))


# --------------------------------------------------------------------------------------------
# operator arithmetic, NumPy (explicit loops over the window; small cases)
# --------------------------------------------------------------------------------------------
def _act_numpy(y, act):
    if act == 'relu':
        return np.maximum(y, 0)
    if act == 'sigmoid':
        return 1.0 / (1.0 + np.exp(-y))
    if act == 'tanh':
        return np.tanh(y)
    if act == 'identity':
        return y
    raise ValueError(act)


def conv2d_numpy(x, w, b, stride, padding, groups=1, act='identity'):
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    n, cin, h, wd = x.shape
    cout, cin_g, kh, kw = w.shape
    assert cin == cin_g * groups and cout % groups == 0
    oh = 1 + (h - kh + 2 * padding[0]) // stride[0]
    ow = 1 + (wd - kw + 2 * padding[1]) // stride[1]
    xp = np.zeros((n, cin, h + 2 * padding[0], wd + 2 * padding[1]))
    xp[:, :, padding[0]:padding[0] + h, padding[1]:padding[1] + wd] = x
    y = np.zeros((n, cout, oh, ow))
    cout_g = cout // groups
    for g in range(groups):
        xs = xp[:, g * cin_g:(g + 1) * cin_g]
        ws = w[g * cout_g:(g + 1) * cout_g]
        for r in range(kh):
            for s in range(kw):
                patch = xs[:, :, r:r + (oh - 1) * stride[0] + 1:stride[0], s:s + (ow - 1) * stride[1] + 1:stride[1]]
                y[:, g * cout_g:(g + 1) * cout_g] += np.einsum('nchw,oc->nohw', patch, ws[:, :, r, s])
    if b is not None:
        y += np.asarray(b, dtype=np.float64)[None, :, None, None]
    return _act_numpy(y, act)


def pool2d_numpy(x, pool_type, kernel, stride, padding):
    x = np.asarray(x, dtype=np.float64)
    n, c, h, w = x.shape
    if 'global' in pool_type:
        kernel, stride, padding = (h, w), (1, 1), (0, 0)
    is_max = 'max' in pool_type
    oh = 1 + (h - kernel[0] + 2 * padding[0]) // stride[0]
    ow = 1 + (w - kernel[1] + 2 * padding[1]) // stride[1]
    fill = -np.inf if is_max else 0.0
    xp = np.full((n, c, h + 2 * padding[0], w + 2 * padding[1]), fill)
    xp[:, :, padding[0]:padding[0] + h, padding[1]:padding[1] + w] = x
    y = np.full((n, c, oh, ow), fill)
    for r in range(kernel[0]):
        for s in range(kernel[1]):
            patch = xp[:, :, r:r + (oh - 1) * stride[0] + 1:stride[0], s:s + (ow - 1) * stride[1] + 1:stride[1]]
            y = np.maximum(y, patch) if is_max else y + patch
    return y if is_max else y / float(kernel[0] * kernel[1])


# --------------------------------------------------------------------------------------------
# the graph walk (shared by both back-ends)
# --------------------------------------------------------------------------------------------
class _TorchOps:
    def __init__(self, dtype):
        import torch
        self.torch = torch
        self.F = torch.nn.functional
        self.dtype = dtype

    def tensor(self, a):
        return self.torch.from_numpy(np.ascontiguousarray(a)).to(self.dtype)

    def numpy(self, t):
        return t.detach().cpu().numpy()

    def slice(self, t, begin, end):
        return t if begin == 0 and end == t.shape[1] else t[:, begin:end]

    def add(self, xs):
        return xs[0] if len(xs) == 1 else self.torch.sum(self.torch.stack(xs, dim=0), dim=0)

    def mul(self, xs):
        return xs[0] if len(xs) == 1 else self.torch.prod(self.torch.stack(xs, dim=0), dim=0)

    def cat(self, xs):
        return xs[0] if len(xs) == 1 else self.torch.cat(xs, dim=1)

    def act(self, t, act):
        if act == 'relu':
            return self.torch.relu(t)
        if act == 'sigmoid':
            return self.torch.sigmoid(t)
        if act == 'tanh':
            return self.torch.tanh(t)
        if act == 'identity':
            return t
        raise ValueError(act)

    def conv(self, t, w, b, stride, padding, groups, act):
        y = self.F.conv2d(t, self.tensor(w), self.tensor(b), stride=tuple(stride), padding=tuple(padding),
                          groups=groups)
        return self.act(y, act)

    def pool(self, t, pool_type, kernel, stride, padding):
        if 'global' in pool_type:
            kernel, stride, padding = tuple(t.shape[2:]), (1, 1), (0, 0)
        if 'max' in pool_type:
            return self.F.max_pool2d(t, tuple(kernel), tuple(stride), tuple(padding))
        return self.F.avg_pool2d(t, tuple(kernel), tuple(stride), tuple(padding), count_include_pad=True)


class _NumpyOps:
    def tensor(self, a):
        return np.asarray(a, dtype=np.float64)

    def numpy(self, t):
        return t

    def slice(self, t, begin, end):
        return t[:, begin:end]

    def add(self, xs):
        out = xs[0]
        for x in xs[1:]:
            out = out + x
        return out

    def mul(self, xs):
        out = xs[0]
        for x in xs[1:]:
            out = out * x
        return out

    def cat(self, xs):
        return np.concatenate(xs, axis=1)

    def act(self, t, act):
        return _act_numpy(t, act)

    def conv(self, t, w, b, stride, padding, groups, act):
        return conv2d_numpy(t, w, b, stride, padding, groups, act)

    def pool(self, t, pool_type, kernel, stride, padding):
        return pool2d_numpy(t, pool_type, kernel, stride, padding)


def _walk(config, weights: Weights, x, ops, keep=None):
    values = {config['input']['name']: ops.tensor(x)}

    def assemble(node):
        mul = node['type'] == 'element' and node.get('op_type') == 'mul'
        terms = []
        for term in node['inputs']:
            parts = [ops.slice(values[name], begin, end) for name, begin, end in term]
            terms.append(ops.mul(parts) if mul else ops.add(parts))
        return ops.cat(terms)

    def run(node):
        kind = node['type']
        if kind == 'sequential':
            for sub in node['nodes']:
                run(sub)
            values[node['name']] = values[node['nodes'][-1]['name']]
            return
        t = assemble(node)
        if kind == 'conv':
            w, b = weights[node['name']]
            t = ops.conv(t, w, b, node['stride'], node['padding'], node['groups'], node['act'])
        elif kind == 'pool':
            t = ops.pool(t, node['pool_type'], node['kernel'], node['stride'], node['padding'])
        elif kind == 'relu':
            t = ops.act(t, 'relu')
        elif kind == 'activation':
            t = ops.act(t, node['act_type'])
        elif kind in ('identity', 'element'):
            pass
        else:
            raise ValueError(f'unknown node type {kind}')
        values[node['name']] = t

    last = None
    for block in config['blocks']:
        for node in block['inner_nodes']:
            run(node)
        run(block['exit_node'])
        last = block['exit_node']['name']
    if keep is not None:
        return {name: ops.numpy(values[name]) for name in keep}
    return ops.numpy(values[last])


def run_config(config, weights: Weights, x: np.ndarray, double=False, keep=None, threads=None) -> np.ndarray:
    """Execute a graph config on the CPU with torch (float32, or float64 when ``double``)."""
    import torch
    if threads:
        torch.set_num_threads(int(threads))
    ops = _TorchOps(torch.float64 if double else torch.float32)
    with torch.no_grad():
        out = _walk(config, weights, x, ops, keep)
    return out


def run_config_numpy(config, weights: Weights, x: np.ndarray, keep=None) -> np.ndarray:
    """Execute a graph config with explicit NumPy float64 arithmetic (small graphs)."""
    return _walk(config, weights, x, _NumpyOps(), keep)
