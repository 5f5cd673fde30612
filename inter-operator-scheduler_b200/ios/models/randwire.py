"""
RandWire networks (reference ``python/ios/models/randwire.py``).  A stage is a Watts-Strogatz
random graph oriented by node index; every node sums its inputs (one term with several values) and
applies ReLU -> depthwise 3x3 -> pointwise 1x1; nodes without a predecessor read the stage input
with stride 2; the stage output is the sum of all nodes without a successor.

``randwire_large`` follows the reference's regular regime (C=154, stages of 16/32/32/32 nodes,
one-convolution stem); ``randwire_small`` is the small regime assembled from the same pieces
(two stride-2 stem convolutions, three 32-node stages at C, 2C, 4C with C=78).
"""
import os

from .common import *

cur_dir = os.path.dirname(os.path.abspath(__file__))
graph_dir = os.path.join(cur_dir, "randwire_graphs/generated")


def read_graph(fname):
    """Read ``n``, ``m`` and ``m`` edge lines ``u v`` (reference ``randwire.py:8-17``)."""
    with open(fname, 'r') as f:
        n = int(f.readline())
        m = int(f.readline())
        edges = [tuple(int(t) for t in f.readline().split()) for _ in range(m)]
    return n, edges


def randwire_small_front(v: Value, ch: int) -> Tuple[Value, Block]:
    block = Block(v.node, None, [], None)
    v = conv2d(block, [[v]], out_channels=ch // 2, kernel=(3, 3), stride=(2, 2), padding=(1, 1), act="relu")
    v = conv2d(block, [[v]], out_channels=ch, kernel=(3, 3), stride=(2, 2), padding=(1, 1), act="identity",
               is_exit=True)
    return v, block


def randwire_regular_front(v: Value, ch: int) -> Tuple[Value, Block]:
    block = Block(v.node, None, [], None)
    v = conv2d(block, [[v]], out_channels=ch // 2, kernel=(3, 3), stride=(2, 2), padding=(1, 1), act="identity",
               is_exit=True)
    return v, block


def randwire_tail(v: Value) -> Tuple[Value, Block]:
    block = Block(v.node, None, [], None)
    v = relu(block, [[v]])
    v = conv2d(block, [[v]], out_channels=1280, kernel=(1, 1), stride=(1, 1), padding=(0, 0), act="identity")
    v = pool2d(block, [[v]], pool_type='global_avg', is_exit=True)
    return v, block


def randwire_stage(r: Value, ch: int, graph_fname) -> Tuple[Value, Block]:
    """Build one random-graph stage; nodes are emitted in the LIFO topological order of the reference (``randwire.py:44-69``)."""
    block = Block(r.node, None, [], None)
    n, edges = read_graph(graph_fname)
    preds = [[] for _ in range(n)]
    succs = [[] for _ in range(n)]
    for u, v in edges:
        succs[u].append(v)
        preds[v].append(u)
    waiting = [len(p) for p in preds]
    produced = [None] * n
    stack = [u for u in range(n) if waiting[u] == 0]
    while stack:
        u = stack.pop()
        if not preds[u]:
            produced[u] = rwconv2d(block, [[r]], out_channels=ch, stride=(2, 2))
        else:
            produced[u] = rwconv2d(block, [[produced[v] for v in preds[u]]], out_channels=ch, stride=(1, 1))
        for v in succs[u]:
            waiting[v] -= 1
            if waiting[v] == 0:
                stack.append(v)
    sinks = [[produced[u] for u in range(n) if not succs[u]]]
    return identity(block, sinks, is_exit=True), block


def _assemble(name, front, ch, stage_specs):
    reset_name()
    pv = placeholder(output_shape=(3, 224, 224))
    v, first = front(pv, ch)
    blocks = [first]
    for mult, fname in stage_specs:
        v, b = randwire_stage(v, mult * ch, os.path.join(graph_dir, fname))
        blocks.append(b)
    v, last = randwire_tail(v)
    blocks.append(last)
    graph = Graph(name, pv.node, blocks)
    graph.init_weights()
    return graph


def randwire_large(graph_files=('ws-16-4-0.75-s0.txt', 'ws-32-4-0.75-s0.txt', 'ws-32-4-0.75-s1.txt',
                                'ws-32-4-0.75-s2.txt')):
    """Regular regime: C=154, four stages at C, 2C, 4C, 8C (reference ``randwire.py:72-87``)."""
    return _assemble("randwire_large", randwire_regular_front, 154, list(zip((1, 2, 4, 8), graph_files)))


def randwire_small(graph_files=('ws-32-4-0.75-s0.txt', 'ws-32-4-0.75-s1.txt', 'ws-32-4-0.75-s2.txt')):
    """Small regime: C=78, two-convolution stem, three 32-node stages at 78/156/312 channels, 28/14/7 pixels."""
    return _assemble("randwire_small", randwire_small_front, 78, list(zip((1, 2, 4), graph_files)))
