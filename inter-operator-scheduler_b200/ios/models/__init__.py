from .inception_v3 import inception_v3
from .randwire import randwire_large, randwire_small
from .squeezenet import squeezenet
from .nasnet import nasnet_large
from .resnet import resnet18, resnet34, resnet50
from .vgg import vgg_11, vgg_13, vgg_16, vgg_19
from .alexnet import alexnet
