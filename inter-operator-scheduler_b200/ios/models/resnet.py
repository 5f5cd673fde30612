"""
ResNet-18 / 34 / 50 as IOS graphs (reference ``python/ios/models/resnet.py``): a 7x7 stem block, then
four blocks of residual units.  A unit's shortcut is the block input, or -- in the first unit of a
block that changes resolution or width -- a 1x1 convolution of it (with ReLU, as the reference builds
it); the sum is an ``element`` add node, followed in the bottleneck variant by a separate ReLU.
The graphs come back with the sequential schedule, like the reference's.
"""
from .common import *

# network -> (unit kind, width multiplier of the unit's output, units per block)
_VARIANTS = {
    'resnet18': ('basic', 1, (2, 2, 2, 2)),
    'resnet34': ('basic', 1, (3, 4, 6, 3)),
    'resnet50': ('bottleneck', 4, (3, 4, 6, 3)),
}
_WIDTHS = (64, 128, 256, 512)


def _unit(kind, block, v, width, stride, shortcut, is_exit):
    """One residual unit.  basic: 3x3, 3x3, add.  bottleneck: 1x1, 3x3, 1x1, add, relu."""
    skip = v if shortcut is None else shortcut
    if kind == 'basic':
        v = conv2d(block, [[v]], out_channels=width, kernel=(3, 3), stride=stride, padding=(1, 1), act='relu')
        v = conv2d(block, [[v]], out_channels=width, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='identity')
        return addition(block, [[v, skip]], is_exit=is_exit)
    v = conv2d(block, [[v]], out_channels=width, kernel=(1, 1), stride=stride, padding=(0, 0), act='relu')
    v = conv2d(block, [[v]], out_channels=width, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
    v = conv2d(block, [[v]], out_channels=width, kernel=(1, 1), stride=(1, 1), padding=(0, 0), act='identity')
    v = addition(block, [[v, skip]])
    return activation(block, [[v]], act_type='relu', inplace=True, is_exit=is_exit)


def _stage(v, kind, expansion, width, units, in_channels, stride):
    block = Block(v.node, None, [], None)
    shortcut = None
    if max(stride) != 1 or in_channels != width * expansion:
        shortcut = conv2d(block, [[v]], out_channels=width * expansion, kernel=(1, 1), stride=stride, padding=(0, 0),
                          act='relu')
    v = _unit(kind, block, v, width, stride, shortcut, is_exit=False)
    for index in range(1, units):
        v = _unit(kind, block, v, width, (1, 1), None, is_exit=(index == units - 1))
    return v, block, width


def _resnet(name):
    kind, expansion, depths = _VARIANTS[name]
    reset_name()
    pv = placeholder(output_shape=(3, 224, 224))
    stem = Block(pv.node, None, [], None)
    v = conv2d(stem, [[pv]], out_channels=64, kernel=(7, 7), stride=(2, 2), padding=(3, 3), act='relu')
    v = pool2d(stem, [[v]], pool_type='max', kernel=(3, 3), stride=(2, 2), padding=(1, 1), is_exit=True)
    blocks, channels = [stem], 64
    for index, (width, units) in enumerate(zip(_WIDTHS, depths)):
        stride = (1, 1) if index == 0 else (2, 2)
        v, block, channels = _stage(v, kind, expansion, width, units, channels, stride)
        blocks.append(block)
    graph = Graph(name, pv.node, blocks)
    graph.init_weights()
    graph.sequential_schedule()
    return graph


def resnet18():
    return _resnet('resnet18')


def resnet34():
    return _resnet('resnet34')


def resnet50():
    return _resnet('resnet50')
