from .inception_v3 import inception_v3
from .randwire import randwire_large, randwire_small
from .squeezenet import squeezenet
