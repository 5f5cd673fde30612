"""
VGG-11 / 13 / 16 / 19 feature extractors as single-block IOS graphs (reference
``python/ios/models/vgg.py``): 3x3 convolutions with ReLU, 2x2 max pooling between the groups and a
global average pool as exit.
"""
from .common import *

# convolutions per resolution group; widths are 64, 128, 256, 512, 512
_DEPTHS = {'vgg_11': (1, 1, 2, 2, 2), 'vgg_13': (2, 2, 2, 2, 2), 'vgg_16': (2, 2, 3, 3, 3), 'vgg_19': (2, 2, 4, 4, 4)}
_WIDTHS = (64, 128, 256, 512, 512)


def vgg_net(name):
    reset_name()
    pv = placeholder(output_shape=(3, 224, 224))
    block = Block(pv.node, None, [], None)
    v = pv
    for width, depth in zip(_WIDTHS, _DEPTHS[name]):
        for _ in range(depth):
            v = conv2d(block, [[v]], width, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
        v = pool2d(block, [[v]], pool_type='max', kernel=(2, 2), stride=(2, 2))
    pool2d(block, [[v]], pool_type='global_avg', is_exit=True)
    graph = Graph(name, pv.node, [block])
    graph.init_weights()
    return graph


def vgg_11():
    return vgg_net('vgg_11')


def vgg_13():
    return vgg_net('vgg_13')


def vgg_16():
    return vgg_net('vgg_16')


def vgg_19():
    return vgg_net('vgg_19')
