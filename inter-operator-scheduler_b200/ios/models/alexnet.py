"""
AlexNet's convolutional trunk as a single-block IOS graph (reference ``python/ios/models/alexnet.py``).
The pooling type is spelled ``max_pool`` there; the runtime recognises pooling types by the
substrings ``max`` and ``global`` (reference ``src/ios/ios_runtime.cu:1047-1051``), so it is kept.
"""
from .common import *

# (kind, channels or None, kernel, stride, padding)
_LAYERS = (
    ('conv', 64, (11, 11), (4, 4), (2, 2)),
    ('pool', None, (3, 3), (2, 2), (1, 1)),
    ('conv', 192, (5, 5), (1, 1), (2, 2)),
    ('pool', None, (3, 3), (2, 2), (1, 1)),
    ('conv', 384, (3, 3), (1, 1), (0, 0)),
    ('conv', 256, (3, 3), (1, 1), (0, 0)),
    ('conv', 256, (3, 3), (1, 1), (0, 0)),
)


def alexnet() -> Graph:
    reset_name()
    pv = placeholder(output_shape=(3, 224, 224))
    block = Block(pv.node, None, [], None)
    v = pv
    for index, (kind, channels, kernel, stride, padding) in enumerate(_LAYERS):
        last = index == len(_LAYERS) - 1
        if kind == 'conv':
            v = conv2d(block, [[v]], channels, kernel, stride=stride, padding=padding, is_exit=last)
        else:
            v = pool2d(block, [[v]], 'max_pool', kernel, stride, padding, is_exit=last)
    graph = Graph('alexnet', pv.node, [block])
    graph.init_weights()
    return graph
