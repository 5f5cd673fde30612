"""Python -> C marshalling helpers for the runtime's C-ABI (reference ``python/ios/contrib/ctypes_utils.py``)."""
from typing import Iterable, List
import ctypes

import numpy as np

from ios.ir import Sequential, Node


def c_int(i: int):
    return ctypes.c_int(i)


def c_string(s: str):
    """``char *`` to a private NUL-terminated copy of ``s``."""
    return ctypes.cast(ctypes.create_string_buffer(s.encode()), ctypes.c_char_p)


def c_string_list(sl: List[str]):
    """``char **`` with one entry per string."""
    array = (ctypes.c_char_p * len(sl))(*[s.encode() for s in sl])
    return ctypes.cast(array, ctypes.POINTER(ctypes.c_char_p))


def c_ndarray_list(al: List[np.ndarray]):
    """``float **``; entries that are not arrays become NULL."""
    ptrs = [a.ctypes.data_as(ctypes.c_void_p) if isinstance(a, np.ndarray) else ctypes.c_void_p(None) for a in al]
    return ctypes.cast((ctypes.c_void_p * len(al))(*ptrs), ctypes.POINTER(ctypes.c_void_p))


def c_ndarray(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def get_nodes_by_type(nodes: Iterable[Node], node_type):
    """Nodes of ``node_type`` in order, looking inside Sequential operators."""
    for node in nodes:
        if isinstance(node, node_type):
            yield node
        elif isinstance(node, Sequential):
            yield from get_nodes_by_type(node.nodes, node_type)
