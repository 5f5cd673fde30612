"""
Inception V3 (reference ``python/ios/models/inception_v3.py``): stem, 3 x A, reduction B, 4 x C
(factorised 7x7), reduction D, 2 x E, global average pool -> 2048 x 1 x 1.  Every convolution has
bias + ReLU (batch norm is folded into the bias).
"""
from .common import *


def _block(v: Value) -> Block:
    return Block(v.node, None, [], None)


def _chain(block, v, layers):
    """Apply ``(out_channels, kernel, padding)`` or ``(out_channels, kernel, padding, stride)`` convs in order."""
    for spec in layers:
        out_channels, kernel, padding = spec[:3]
        stride = spec[3] if len(spec) > 3 else (1, 1)
        v = conv2d(block, [[v]], out_channels=out_channels, kernel=kernel, stride=stride, padding=padding)
    return v


def _avg_branch(block, v, out_channels):
    p = pool2d(block, [[v]], pool_type='avg', kernel=(3, 3), stride=(1, 1), padding=(1, 1))
    return conv2d(block, [[p]], out_channels=out_channels, kernel=(1, 1))


def inception_front(v: Value) -> Tuple[Value, Block]:  # 3 x 299 x 299 -> 192 x 35 x 35
    block = _block(v)
    v = _chain(block, v, [(32, (3, 3), (0, 0), (2, 2)), (32, (3, 3), (0, 0)), (64, (3, 3), (1, 1))])
    v = pool2d(block, [[v]], pool_type='max', kernel=(3, 3), stride=(2, 2))
    v = _chain(block, v, [(80, (1, 1), (0, 0)), (192, (3, 3), (0, 0))])
    v = pool2d(block, [[v]], pool_type='max', kernel=(3, 3), stride=(2, 2), is_exit=True)
    return v, block


def inception_a(v: Value, pool_features) -> Tuple[Value, Block]:
    block = _block(v)
    b1 = _chain(block, v, [(64, (1, 1), (0, 0))])
    b5 = _chain(block, v, [(48, (1, 1), (0, 0)), (64, (5, 5), (2, 2))])
    b3 = _chain(block, v, [(64, (1, 1), (0, 0)), (96, (3, 3), (1, 1)), (96, (3, 3), (1, 1))])
    bp = _avg_branch(block, v, pool_features)
    return identity(block, [[b1], [b5], [b3], [bp]], is_exit=True), block


def inception_b(v: Value) -> Tuple[Value, Block]:
    block = _block(v)
    b3 = _chain(block, v, [(384, (3, 3), (0, 0), (2, 2))])
    bd = _chain(block, v, [(64, (1, 1), (0, 0)), (96, (3, 3), (1, 1)), (96, (3, 3), (0, 0), (2, 2))])
    bp = pool2d(block, [[v]], pool_type='max', kernel=(3, 3), stride=(2, 2))
    return identity(block, [[b3], [bd], [bp]], is_exit=True), block


def inception_c(v, channels_7x7):
    block = _block(v)
    c7 = channels_7x7
    row, col = ((1, 7), (0, 3)), ((7, 1), (3, 0))
    b1 = _chain(block, v, [(192, (1, 1), (0, 0))])
    b7 = _chain(block, v, [(c7, (1, 1), (0, 0)), (c7, *row), (192, *col)])
    bd = _chain(block, v, [(c7, (1, 1), (0, 0)), (c7, *col), (c7, *row), (c7, *col), (192, *row)])
    bp = _avg_branch(block, v, 192)
    return identity(block, [[b1], [b7], [bd], [bp]], is_exit=True), block


def inception_d(v):
    block = _block(v)
    b3 = _chain(block, v, [(192, (1, 1), (0, 0)), (320, (3, 3), (0, 0), (2, 2))])
    b7 = _chain(block, v, [(192, (1, 1), (0, 0)), (192, (1, 7), (0, 3)), (192, (7, 1), (3, 0)),
                           (192, (3, 3), (0, 0), (2, 2))])
    bp = pool2d(block, [[v]], pool_type='max', kernel=(3, 3), stride=(2, 2))
    return identity(block, [[b3], [b7], [bp]], is_exit=True), block


def inception_e(v):
    block = _block(v)
    b1 = _chain(block, v, [(320, (1, 1), (0, 0))])
    t3 = _chain(block, v, [(384, (1, 1), (0, 0))])
    b3a = _chain(block, t3, [(384, (1, 3), (0, 1))])
    b3b = _chain(block, t3, [(384, (3, 1), (1, 0))])
    td = _chain(block, v, [(448, (1, 1), (0, 0)), (384, (3, 3), (1, 1))])
    bda = _chain(block, td, [(384, (1, 3), (0, 1))])
    bdb = _chain(block, td, [(384, (3, 1), (1, 0))])
    bp = _avg_branch(block, v, 192)
    return identity(block, [[b1], [b3a], [b3b], [bda], [bdb], [bp]], is_exit=True), block


def inception_logits(v):
    block = _block(v)
    v = pool2d(block, [[v]], pool_type='global_avg', is_exit=True)
    return v, block


def inception_v3() -> Graph:
    reset_name()
    pv = placeholder(output_shape=(3, 299, 299))
    blocks = []
    v = pv
    plan = [(inception_front,), (inception_a, 32), (inception_a, 64), (inception_a, 64), (inception_b,),
            (inception_c, 128), (inception_c, 160), (inception_c, 160), (inception_c, 192), (inception_d,),
            (inception_e,), (inception_e,), (inception_logits,)]
    for maker, *args in plan:
        v, block = maker(v, *args)
        blocks.append(block)
    graph = Graph("inception_v3", pv.node, blocks)
    graph.init_weights()
    return graph
