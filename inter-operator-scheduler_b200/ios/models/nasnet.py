"""
NASNet-A Large (6 @ 4032) as a single-block IOS graph (reference ``python/ios/models/nasnet.py``).

A cell is written down as a small program: every line creates one operator (or one pair of
separable convolutions) from named earlier results, in the order in which the reference creates
them -- operator names are a running counter, so the order is part of the exported graph.  Line
forms (``dst`` and ``src`` are names local to the cell; channel arguments are ``'L'`` / ``'R'`` for
the cell's left / right width or a plain number):

    ('rc',   dst, src, channels, stride)            ReLU -> 1x1 convolution
    ('sep',  dst, src, channels, k, stride)         two ReLU-separable convolutions, the first keeps the width of src
    ('sep*', dst, src, channels, k, stride)         the same with both at ``channels`` (stem form)
    ('max' | 'avg', dst, src, stride)               3x3 pooling, padding 1
    ('add',  dst, a, b)                             element-wise sum (an identity node over one two-value term)
    ('cat',  dst, a, b)                             channel concat of a and b
    ('out',  [term, ...])                           the cell's result: concat over terms of sums over names

The block is so large (about 370 schedule units) that the search works on it in parts, one per
cell (``block.parts``, reference ``common.py:494-516``).
"""
from .common import *

_STEM0 = (
    ('rc', 'x1', 'x', 'L', 1),
    ('sep', 'c0l', 'x1', 'L', 5, 2), ('sep*', 'c0r', 'x', 'L', 7, 2), ('add', 'c0', 'c0l', 'c0r'),
    ('max', 'c1l', 'x1', 2), ('sep*', 'c1r', 'x', 'L', 7, 2), ('add', 'c1', 'c1l', 'c1r'),
    ('avg', 'c2l', 'x1', 2), ('sep*', 'c2r', 'x', 'L', 5, 2),
    ('avg', 'c3r', 'c0', 1),
    ('sep', 'c4l', 'c0', 'L', 3, 1), ('max', 'c4r', 'x1', 2),
    ('out', [['c1'], ['c2l', 'c2r'], ['c3r', 'c0'], ['c4l', 'c4r']]),
)

# x = the previous cell's result (hp in the reference), p = the one before (h)
_STEM1 = (
    ('rc', 'xl', 'x', 'L', 1),
    ('rc', 'r1', 'p', 'L/2', 2), ('rc', 'r2', 'p', 'L/2', 2), ('add', 'xr', 'r1', 'r2'),
    ('sep', 'c0l', 'xl', 'L', 5, 2), ('sep', 'c0r', 'xr', 'L', 7, 2), ('add', 'c0', 'c0l', 'c0r'),
    ('max', 'c1l', 'xl', 2), ('sep', 'c1r', 'xr', 'L', 7, 2), ('add', 'c1', 'c1l', 'c1r'),
    ('avg', 'c2l', 'xl', 2), ('sep', 'c2r', 'xr', 'L', 5, 2),
    ('avg', 'c3r', 'c0', 1),
    ('sep', 'c4l', 'c0', 'L', 3, 1), ('max', 'c4r', 'xl', 2),
    ('out', [['c1'], ['c2l', 'c2r'], ['c3r', 'c1'], ['c4l', 'c4r']]),
)

_FIRST = (
    ('rc', 'l1', 'p', 'L', 2), ('rc', 'l2', 'p', 'L', 2), ('cat', 'xl', 'l1', 'l2'),
    ('rc', 'xr', 'x', 'R', 1),
    ('sep', 'c0l', 'xr', 'R', 5, 1), ('sep', 'c0r', 'xr', 'R', 3, 1),
    ('sep', 'c1l', 'xl', 'R', 5, 1), ('sep', 'c1r', 'xl', 'R', 3, 1),
    ('avg', 'c2l', 'xr', 1),
    ('avg', 'c3l', 'xl', 1), ('avg', 'c3r', 'xl', 1),
    ('sep', 'c4l', 'xr', 'R', 3, 1),
    ('out', [['xl'], ['c0l', 'c0r'], ['c1l', 'c1r'], ['c2l', 'xl'], ['c3l', 'c3r'], ['c4l', 'xr']]),
)

_NORMAL = (
    ('rc', 'xl', 'p', 'L', 1), ('rc', 'xr', 'x', 'R', 1),
    ('sep', 'c0l', 'xr', 'R', 5, 1), ('sep', 'c0r', 'xl', 'L', 3, 1),
    ('sep', 'c1l', 'xl', 'L', 5, 1), ('sep', 'c1r', 'xl', 'L', 3, 1),
    ('avg', 'c2l', 'xr', 1),
    ('avg', 'c3l', 'xl', 1), ('avg', 'c3r', 'xl', 1),
    ('sep', 'c4l', 'xr', 'R', 3, 1),
    ('out', [['c0l', 'c0r'], ['c1l', 'c1r'], ['c2l', 'xl'], ['c3l', 'c3r'], ['c4l', 'xr']]),
)

_REDUCTION = (
    ('rc', 'xl', 'p', 'L', 1), ('rc', 'xr', 'x', 'R', 1),
    ('sep', 'c0l', 'xr', 'R', 5, 2), ('sep', 'c0r', 'xl', 'R', 7, 2), ('add', 'c0', 'c0l', 'c0r'),
    ('max', 'c1l', 'xr', 2), ('sep', 'c1r', 'xl', 'R', 7, 2), ('add', 'c1', 'c1l', 'c1r'),
    ('avg', 'c2l', 'xr', 2), ('sep', 'c2r', 'xl', 'R', 5, 2),
    ('avg', 'c3r', 'c0', 1),
    ('sep', 'c4l', 'c0', 'R', 3, 1), ('max', 'c4r', 'xr', 2),
    ('out', [['c1l', 'c1r'], ['c2l', 'c2r'], ['c1', 'c3r'], ['c4l', 'c4r']]),
)


def _run_cell(block, program, x, p, left, right):
    """Execute a cell program; ``x`` is the latest cell result, ``p`` the one before it."""
    env = {'x': x, 'p': p}
    widths = {'L': left, 'R': right, 'L/2': left // 2}

    def width(arg):
        return widths[arg] if isinstance(arg, str) else arg

    for line in program:
        op = line[0]
        if op == 'out':
            return identity(block, [[env[name] for name in term] for term in line[1]])
        dst, src = line[1], env[line[2]]
        if op == 'rc':
            env[dst] = relu_conv(block, [[src]], width(line[3]), kernel=(1, 1), stride=(line[4], line[4]), padding=(0, 0))
        elif op in ('sep', 'sep*'):
            k, s = line[4], line[5]
            first = src.node.output_shape[0] if op == 'sep' else width(line[3])
            v = relu_sep_conv(block, [[src]], first, (k, k), (s, s), (k // 2, k // 2))
            env[dst] = relu_sep_conv(block, [[v]], width(line[3]), (k, k), (1, 1), (k // 2, k // 2))
        elif op in ('max', 'avg'):
            env[dst] = pool2d(block, [[src]], pool_type=op, kernel=(3, 3), stride=(line[3], line[3]), padding=(1, 1))
        elif op == 'add':
            env[dst] = identity(block, [[src, env[line[3]]]])
        elif op == 'cat':
            env[dst] = identity(block, [[src], [env[line[3]]]])
        else:
            raise ValueError(op)
    raise ValueError('a cell program must end with an out line')


def nasnet_large(stem_filters=96, filters=168) -> Graph:
    reset_name()
    v0 = placeholder(output_shape=(3, 331, 331))
    block = Block(v0.node, None, [], None)
    v1 = conv2d(block, [[v0]], out_channels=stem_filters, kernel=(3, 3), stride=(2, 2), padding=(0, 0), act='identity')
    cells = [v0, v1]
    cells.append(_run_cell(block, _STEM0, v1, None, filters // 4, filters // 4))
    cells.append(_run_cell(block, _STEM1, cells[-1], v1, filters // 2, filters // 2))
    # (program, index of the older input counted back from the newest result, left width, right width) per cell
    f = filters
    plan = [(_FIRST, 2, f // 2, f)] + [(_NORMAL, 2, f, f)] * 5 + \
           [(_REDUCTION, 2, 2 * f, 2 * f), (_FIRST, 3, f, 2 * f)] + [(_NORMAL, 2, 2 * f, 2 * f)] * 5 + \
           [(_REDUCTION, 2, 4 * f, 4 * f), (_FIRST, 3, 2 * f, 4 * f)] + [(_NORMAL, 2, 4 * f, 4 * f)] * 5
    for program, back, left, right in plan:
        cells.append(_run_cell(block, program, cells[-1], cells[-back], left, right))
    cells.append(relu(block, [[cells[-1]]]))
    cells.append(pool2d(block, [[cells[-1]]], pool_type='global_avg', is_exit=True))
    block.parts = get_parts(block, split_vars=cells)
    graph = Graph('nasnet_large', v0.node, [block])
    graph.init_weights()
    return graph
