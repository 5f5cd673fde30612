"""
Drop-in ``ios`` package for the B200-native IOS runtime.

Same user-facing surface as the reference's ``python/ios/__init__.py``: graph builders, ``Graph``,
``optimize``, the cost models and ``ios.ios_runtime`` (the ctypes front-end of ``libios_runtime.so``).
"""
from .optimizer import optimize
from .ir import Graph
from .cost_model import IOSCostModel, RandomCostModel
from .models.common import Graph, Block, placeholder, reset_name
from .models.common import conv2d, pool2d, identity, relu, activation, multiply, addition, element, sequential
from .contrib import ios_runtime
from .visualizer import draw
from . import models

__version__ = "0.1.dev0"
