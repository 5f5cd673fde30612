"""
ctypes front-end of ``libios_runtime.so``.

Same functions, arguments and return shapes as the reference's
``python/ios/contrib/ios_runtime.py`` (``graph_latency`` :26, ``block_latency`` :53,
``stage_latency`` :80, ``graph_inference`` :114).  Differences that a caller can observe:

* failures raise ``RuntimeError`` with the library's message instead of ending the interpreter
  (the reference's ``FatalError`` calls ``exit(1)``);
* ``graph_inference`` converts its input to C-contiguous float32 first (the reference passes the
  raw buffer of whatever array it is given, ``ios_runtime.py:126``);
* there is no CPU path: without a CUDA device every call raises.

``Engine`` is the build-once / run-many handle used for serving and benchmarking.
"""
import ctypes
import json
import os
from typing import List

import numpy as np

from ios.ir import Conv, Graph, Block, Node
from .ctypes_utils import c_string, c_string_list, c_ndarray_list, get_nodes_by_type

cur_dir = os.path.dirname(os.path.abspath(os.path.realpath(__file__)))

libname_list = [
    'libios_runtime.so',
    '../libios_runtime.so',
    '../../libios_runtime.so',
    '../build/libios_runtime.so',
    '../../build/libios_runtime.so',
    '../../../build/libios_runtime.so',
]
lib = None

_INT, _FLOATP, _CHARP = ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.c_char_p
_VOIDPP = ctypes.POINTER(ctypes.c_void_p)
_LATENCY_ARGS = [_CHARP, _INT, _INT, _INT, _INT, _INT, _FLOATP, _FLOATP]


def load_ios_library():
    """Find and load the runtime next to this package (same search list as the reference, :8-23)."""
    override = os.environ.get('IOS_RUNTIME_LIBRARY')
    candidates = [override] if override else [os.path.join(cur_dir, name) for name in libname_list]
    for path in candidates:
        try:
            handle = ctypes.cdll.LoadLibrary(path)
        except OSError:
            continue
        handle.ios_last_error.restype = ctypes.c_char_p
        handle.ios_graph_latency.argtypes = _LATENCY_ARGS
        handle.ios_block_latency.argtypes = _LATENCY_ARGS
        handle.ios_stage_latency.argtypes = [_CHARP] + _LATENCY_ARGS
        handle.ios_graph_inference.argtypes = [_CHARP, _INT, ctypes.c_void_p, _INT, ctypes.POINTER(_CHARP), _VOIDPP,
                                               _VOIDPP, ctypes.c_void_p]
        handle.ios_engine_create.argtypes = [_CHARP, _INT, _INT, ctypes.POINTER(_CHARP), _VOIDPP, _VOIDPP,
                                             ctypes.POINTER(ctypes.c_void_p)]
        handle.ios_engine_destroy.argtypes = [ctypes.c_void_p]
        handle.ios_engine_save.argtypes = [ctypes.c_void_p, _CHARP]
        handle.ios_engine_load.argtypes = [_CHARP, ctypes.POINTER(ctypes.c_void_p)]
        handle.ios_engine_run.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        handle.ios_engine_run_pipelined.argtypes = [ctypes.c_void_p, _INT, _VOIDPP, _VOIDPP]
        handle.ios_engine_time.argtypes = [ctypes.c_void_p, _INT, _FLOATP]
        handle.ios_engine_describe.argtypes = [ctypes.c_void_p, ctypes.c_char_p, _INT]
        handle.ios_plan_describe.argtypes = [ctypes.c_char_p, _INT, _INT, ctypes.c_char_p, _INT]
        handle.ios_plan_describe.restype = _INT
        handle.ios_engine_profile.argtypes = [ctypes.c_void_p, _INT, _INT, ctypes.POINTER(_INT), _FLOATP,
                                              ctypes.POINTER(_INT), ctypes.POINTER(ctypes.c_double)]
        handle.ios_engine_set_input.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        handle.ios_engine_get_output.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        handle.ios_set_option.argtypes = [_CHARP, _CHARP]
        handle.ios_get_option.argtypes = [_CHARP, ctypes.c_char_p, _INT]
        handle.ios_set_device.argtypes = [_INT]
        handle.ios_device_count.argtypes = [ctypes.POINTER(_INT)]
        handle.ios_host_register.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
        handle.ios_host_unregister.argtypes = [ctypes.c_void_p]
        handle.ios_conv2d.argtypes = [ctypes.c_void_p] * 4 + [_INT] * 14
        return handle
    raise FileNotFoundError('IOS Backend library not found (build it with inter-operator-scheduler_b200/build.py)')


def _library():
    global lib
    if lib is None:
        lib = load_ios_library()
    return lib


def _check(status):
    if status != 0:
        message = _library().ios_last_error().decode(errors='replace')
        raise RuntimeError(f'ios_runtime error {status}: {message}')


def set_option(key: str, value: str):
    """Run-time switches: precision tf32x3|tf32|bf16|fp32, executor graph|streams, conv auto|direct, pdl 0|1."""
    _check(_library().ios_set_option(key.encode(), str(value).encode()))


def plan_describe(graph: Graph, batch_size: int, sm_count: int = 0) -> dict:
    """
    The plan the current options would build for `graph`: arena size, launches per forward, and for every convolution
    its kernel and tiling.  Touches no device (works on a machine without a GPU).
    """
    text = json.dumps(graph.export_config()).encode()
    capacity = 1 << 20
    buf = ctypes.create_string_buffer(capacity)
    _check(_library().ios_plan_describe(text, batch_size, sm_count, buf, capacity))
    return json.loads(buf.value.decode())


def get_option(key: str) -> str:
    buf = ctypes.create_string_buffer(64)
    _check(_library().ios_get_option(key.encode(), buf, 64))
    return buf.value.decode()


def set_device(device: int):
    _check(_library().ios_set_device(int(device)))


def device_count() -> int:
    n = ctypes.c_int(0)
    _check(_library().ios_device_count(ctypes.byref(n)))
    return n.value


def host_register(array: np.ndarray) -> bool:
    """Page-lock the memory of ``array`` so that copies from / to it overlap with compute.  False if refused."""
    return _library().ios_host_register(ctypes.c_void_p(array.ctypes.data), array.nbytes) == 0


def host_unregister(array: np.ndarray) -> bool:
    return _library().ios_host_unregister(ctypes.c_void_p(array.ctypes.data)) == 0


def _timed(entry, head_args, batch_size, warmup, number, repeat, profile_stage, num_stage_slots):
    results = (ctypes.c_float * int(repeat))()
    stage_results = (ctypes.c_float * max(1, int(num_stage_slots)))()
    _check(entry(*head_args, int(batch_size), int(warmup), int(number), int(repeat), 1 if profile_stage else 0,
                 ctypes.cast(results, _FLOATP), ctypes.cast(stage_results, _FLOATP)))
    values = [float(v) for v in results]
    if profile_stage:
        return values, [float(v) for v in stage_results][:int(num_stage_slots)]
    return values


def graph_latency(graph: Graph, batch_size=1, warmup=2, number=6, repeat=6, profile_stage=False):
    """
    Latency of the whole graph under its schedule: ``repeat`` samples in ms, each the mean of
    ``number`` forwards after ``warmup`` untimed ones.  With ``profile_stage`` also returns the
    flattened ``repeat x num_stages`` per-stage times.
    """
    num_stages = sum(len(b.stages or []) for b in graph.blocks)
    text = json.dumps(graph.export_config()).encode()
    return _timed(_library().ios_graph_latency, (text,), batch_size, warmup, number, repeat, profile_stage,
                  repeat * num_stages)


def block_latency(block: Block, batch_size, warmup, number, repeat, profile_stage=False):
    text = json.dumps(block.export_config()).encode()
    return _timed(_library().ios_block_latency, (text,), batch_size, warmup, number, repeat, profile_stage,
                  repeat * len(block.stages or []))


def stage_config(stage: List[List[Node]]):
    """(stage json, input json) of a candidate stage: full node configs plus the shapes of outside producers."""
    groups = [[node.export_config() for node in group] for group in stage]
    inside = {node.name for group in stage for node in group}
    producers = {}
    for group in stage:
        for node in group:
            for term in node.inputs:
                for value in term:
                    if value.node.name not in inside:
                        producers.setdefault(value.node.name, value.node.output_shape)
    return json.dumps(groups), json.dumps({name: list(shape) for name, shape in producers.items()})


def canonical_stage_key(stage_text: str, input_text: str) -> str:
    """
    A key that is equal for candidate stages of the same structure whatever their operators are called:
    names are replaced by their order of first appearance and hint names dropped.  Networks repeat their
    blocks (three Inception-A, four Inception-C ...), so a search meets every such stage several times
    and needs to measure it once.
    """
    groups, producers = json.loads(stage_text), json.loads(input_text)
    order = {}

    def canon(name):
        return order.setdefault(name, f'n{len(order)}')

    def walk(node):
        node = dict(node)
        node['hint_name'] = ''
        node['inputs'] = [[[canon(v[0]), v[1], v[2]] for v in term] for term in node.get('inputs', [])]
        if 'nodes' in node:
            node['nodes'] = [walk(sub) for sub in node['nodes']]
        node['name'] = canon(node['name'])
        return node

    body = [[walk(node) for node in group] for group in groups]
    shapes = sorted((canon(name), list(shape)) for name, shape in producers.items() if name in order)
    return json.dumps([body, shapes])


def stage_latency(stage: List[List[Node]], batch_size, warmup, number, repeat, profile_stage=False):
    """Latency of one candidate stage (groups x operators) on synthetic inputs; what the DP search calls."""
    stage_text, input_text = stage_config(stage)
    return _timed(_library().ios_stage_latency, (stage_text.encode(), input_text.encode()), batch_size, warmup,
                  number, repeat, profile_stage, repeat)


def pick_faster(graphs, batch_size, warmup=2, number=6, repeat=6):
    """
    Time each scheduled graph with ``graph_latency`` and return ``(best graph, [mean latency ms of each])``.
    A DP schedule is assembled from stage latencies measured one by one; where those do not add up (wide
    graphs of tiny operators) a heuristic schedule can still win, and a caller that wants the fastest
    schedule it has should measure the candidates whole.
    """
    means = [float(np.mean(graph_latency(g, batch_size, warmup, number, repeat))) for g in graphs]
    return graphs[int(np.argmin(means))], means


def _conv_arrays(graph: Graph):
    convs: List[Conv] = list(get_nodes_by_type(graph.nodes(), Conv))
    weights, biases = [], []
    for node in convs:
        if node.weight is None or node.bias is None:
            raise RuntimeError(f'conv {node.name} has no weights: call graph.init_weights() '
                               f'(or optimize(..., compute_weight=True))')
        weights.append(np.ascontiguousarray(node.weight, dtype=np.float32))
        biases.append(np.ascontiguousarray(node.bias, dtype=np.float32))
    return convs, weights, biases


def graph_inference(graph: Graph, batch_size, input: np.ndarray):
    """Execute the graph once on ``input`` (N, C, H, W) and return the exit node's output as float32."""
    output = np.empty(shape=(batch_size, *graph.blocks[-1].exit_node.output_shape), dtype=np.float32)
    convs, weights, biases = _conv_arrays(graph)
    data = np.ascontiguousarray(input, dtype=np.float32)
    expected = (batch_size, *graph.input.output_shape)
    if tuple(data.shape) != tuple(expected):
        raise ValueError(f'input has shape {tuple(data.shape)}, the graph expects {tuple(expected)}')
    _check(_library().ios_graph_inference(
        json.dumps(graph.export_config()).encode(), int(batch_size), data.ctypes.data_as(ctypes.c_void_p),
        len(convs), c_string_list([node.name for node in convs]), c_ndarray_list(weights), c_ndarray_list(biases),
        output.ctypes.data_as(ctypes.c_void_p)))
    return output


def conv2d(x: np.ndarray, weight: np.ndarray, bias=None, stride=(1, 1), padding=(0, 0), groups=1, act='identity',
           impl='auto'):
    """
    One convolution through the runtime (testing aid).  x: NCHW, weight: OIHW.  impl: 'auto',
    'direct' (CUDA cores), 'tensor' (tensor cores, current precision option), 'tensor1' (tensor
    cores, single-pass TF32), 'bf16' (tensor cores, bfloat16 operands and activations).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    n, cin, h, w = x.shape
    cout, _, kh, kw = weight.shape
    oh = 1 + (h - kh + 2 * padding[0]) // stride[0]
    ow = 1 + (w - kw + 2 * padding[1]) // stride[1]
    y = np.empty((n, cout, oh, ow), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    _check(_library().ios_conv2d(
        x.ctypes.data_as(ctypes.c_void_p), weight.ctypes.data_as(ctypes.c_void_p),
        None if b is None else b.ctypes.data_as(ctypes.c_void_p), y.ctypes.data_as(ctypes.c_void_p),
        n, cin, h, w, cout, kh, kw, stride[0], stride[1], padding[0], padding[1], groups,
        ['identity', 'relu', 'sigmoid', 'tanh'].index(act), ['auto', 'direct', 'tensor', 'tensor1', 'bf16'].index(impl)))
    return y


class Engine:
    """
    A graph bound to one GPU: weights packed and resident, schedule captured once.  ``run`` takes
    host NCHW input and returns host NCHW output; ``time`` replays the resident forward.
    """

    def __init__(self, graph: Graph, batch_size: int, synthetic_weights=False):
        self._lib = _library()
        self._handle = ctypes.c_void_p(None)
        self.batch_size = int(batch_size)
        self.input_shape = (self.batch_size, *graph.input.output_shape)
        self.output_shape = (self.batch_size, *graph.blocks[-1].exit_node.output_shape)
        text = json.dumps(graph.export_config()).encode()
        if synthetic_weights:
            status = self._lib.ios_engine_create(text, self.batch_size, 0, None, None, None, ctypes.byref(self._handle))
        else:
            convs, weights, biases = _conv_arrays(graph)
            status = self._lib.ios_engine_create(text, self.batch_size, len(convs),
                                                 c_string_list([node.name for node in convs]),
                                                 c_ndarray_list(weights), c_ndarray_list(biases),
                                                 ctypes.byref(self._handle))
        _check(status)

    def save(self, path: str):
        """Write the engine artefact (scheduled graph, options, packed parameters); see ``Engine.load``."""
        _check(self._lib.ios_engine_save(self._handle, os.fsencode(path)))

    @classmethod
    def load(cls, path: str) -> 'Engine':
        """
        Rebuild an engine from an artefact written by ``save`` on the current device: no float32 weights, no
        packing, no schedule search.  Refused if this library would tile any convolution differently.
        """
        self = cls.__new__(cls)
        self._lib = _library()
        self._handle = ctypes.c_void_p(None)
        _check(self._lib.ios_engine_load(os.fsencode(path), ctypes.byref(self._handle)))
        info = self.describe()
        self.batch_size = info['output_shape'][0]
        self.output_shape = tuple(info['output_shape'])
        self.input_shape = tuple(info['input_shape'])
        return self

    def run(self, input, output=None):
        """``input`` / ``output`` may be numpy arrays or raw host addresses (ints) of float32 NCHW buffers."""
        if isinstance(input, np.ndarray):
            data = np.ascontiguousarray(input, dtype=np.float32)
            if tuple(data.shape) != tuple(self.input_shape):
                raise ValueError(f'input has shape {tuple(data.shape)}, the engine expects {self.input_shape}')
            in_ptr = data.ctypes.data_as(ctypes.c_void_p)
        else:
            in_ptr = ctypes.c_void_p(int(input))
        result = output
        if output is None:
            result = np.empty(self.output_shape, dtype=np.float32)
        out_ptr = result.ctypes.data_as(ctypes.c_void_p) if isinstance(result, np.ndarray) else ctypes.c_void_p(int(result))
        _check(self._lib.ios_engine_run(self._handle, in_ptr, out_ptr))
        return result

    def run_pipelined(self, inputs, outputs=None):
        """
        Several batches in a row with the host copies overlapped with compute (upload of batch i + 1 and
        download of batch i - 1 beside the forward of batch i).  ``inputs`` / ``outputs``: sequences of
        float32 NCHW numpy arrays or raw host addresses; page-locked buffers are needed for the overlap.
        """
        count = len(inputs)
        keep = []

        def address(item, shape):
            if isinstance(item, np.ndarray):
                if item.dtype != np.float32 or not item.flags['C_CONTIGUOUS'] or tuple(item.shape) != tuple(shape):
                    raise ValueError(f'expected a C-contiguous float32 array of shape {tuple(shape)}')
                keep.append(item)
                return item.ctypes.data
            return int(item)

        results = outputs
        if outputs is None:
            results = [np.empty(self.output_shape, dtype=np.float32) for _ in range(count)]
        in_ptrs = (ctypes.c_void_p * count)(*[address(x, self.input_shape) for x in inputs])
        out_ptrs = (ctypes.c_void_p * count)(*[address(y, self.output_shape) for y in results])
        _check(self._lib.ios_engine_run_pipelined(self._handle, count, in_ptrs, out_ptrs))
        return results

    def set_input(self, input: np.ndarray):
        data = np.ascontiguousarray(input, dtype=np.float32)
        _check(self._lib.ios_engine_set_input(self._handle, data.ctypes.data_as(ctypes.c_void_p)))

    def get_output(self):
        out = np.empty(self.output_shape, dtype=np.float32)
        _check(self._lib.ios_engine_get_output(self._handle, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def time(self, iters=10) -> float:
        """Milliseconds per forward over ``iters`` back-to-back replays (CUDA events, resident input)."""
        ms = ctypes.c_float(0.0)
        _check(self._lib.ios_engine_time(self._handle, int(iters), ctypes.byref(ms)))
        return float(ms.value)

    def describe(self) -> dict:
        buf = ctypes.create_string_buffer(2048)
        _check(self._lib.ios_engine_describe(self._handle, buf, 2048))
        return json.loads(buf.value.decode())

    STEP_KINDS = ('sum_act', 'pool', 'conv_tc', 'conv_direct', 'conv_depthwise')

    def profile(self, iters=5):
        """
        Device time of the launches of one forward: the launches of each kind are replayed one after
        another as a graph of their own and every launch is credited with its kind's mean.
        Returns a list of ``(kind, ms, work)``; ``work`` is algorithmic FLOPs for the
        convolutions on ``conv_tc`` / ``conv_direct`` and algorithmic bytes for the other kinds.
        """
        capacity = 4096
        count = ctypes.c_int(0)
        ms = (ctypes.c_float * capacity)()
        kinds = (ctypes.c_int * capacity)()
        work = (ctypes.c_double * capacity)()
        _check(self._lib.ios_engine_profile(self._handle, int(iters), capacity, ctypes.byref(count), ms, kinds, work))
        return [(self.STEP_KINDS[kinds[i]], float(ms[i]), float(work[i])) for i in range(count.value)]

    def close(self):
        if self._handle:
            self._lib.ios_engine_destroy(self._handle)
            self._handle = ctypes.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
