"""
Computation-graph IR and schedule representation.

Behavioural counterpart of the reference's ``python/ios/ir.py``: the class names, attribute names,
JSON wire format (``export_config`` / ``from_config``), shape inference, work counters, schedule
helpers and the pretty printer are kept so that user scripts and the C-ABI runtime see the same
thing.  The implementation is table-driven: every operator declares the attribute list it
serialises, and one generic loader / exporter in :class:`Node` serves all of them.

A graph is a chain of blocks.  A block is a DAG of operators with one enter node (owned by the
previous block) and one exit node.  Each operator's input is *concat over terms (sum over values
(channel slice of a producer))*, written ``inputs = [[Value, ...], ...]``
(reference ``python/ios/ir.py:99-102``).
"""
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np


class Value:
    """Channel slice ``[begin, end)`` of the output of ``node`` (reference ``ir.py:19-80``)."""
    __slots__ = ['node', 'begin', 'end']

    def __init__(self, node, begin, end):
        self.node = node
        self.begin = begin
        self.end = end

    @property
    def length(self):
        return self.end - self.begin

    @staticmethod
    def from_config(config, name2nodes):
        return Value(name2nodes[config[0]], config[1], config[2])

    def export_config(self):
        return [self.node.name, self.begin, self.end]

    def __eq__(self, other):
        return (isinstance(other, Value) and self.node == other.node
                and self.begin == other.begin and self.end == other.end)

    def __hash__(self):
        return hash((id(self.node), self.begin, self.end))

    def __repr__(self):
        return f'({self.node.hint_name}:{self.begin}:{self.end})'

    __str__ = __repr__


def _spatial_out(size, kernel, padding, stride):
    return 1 + (size - kernel + 2 * padding) // stride


class Node:
    """
    Base class of all operators (reference ``ir.py:83-237``).

    ``_extra`` lists the operator-specific attributes in the order they appear in the exported
    config, between ``inputs`` and ``output_shape``.
    """
    __slots__ = ['type', 'name', 'hint_name', 'inputs', 'output_shape', 'uses']
    _extra: Tuple[str, ...] = ()
    _registry: Dict[str, type] = {}

    def __init__(self, type, name, hint_name, inputs, output_shape):
        self.type = type
        self.name = name
        self.hint_name = hint_name
        self.inputs = inputs
        self.output_shape = output_shape
        self.uses: List[Tuple['Node', int, int]] = []

    # ---- construction from / export to the JSON wire format --------------------------------
    @staticmethod
    def from_config(config, name2node):
        kind = config['type']
        cls = Node._registry.get(kind)
        if cls is None:
            raise ValueError(f"unrecognized node type {kind}")
        return cls.from_config(config, name2node)

    @classmethod
    def _load(cls, config, name2node):
        terms = [[Value.from_config(vc, name2node) for vc in tc] for tc in config['inputs']]
        kwargs = {key: config[key] for key in cls._extra}
        node = cls(config['name'], config['hint_name'], terms, output_shape=config['output_shape'], **kwargs)
        node._register_uses(name2node)
        return node

    def _register_uses(self, name2node=None):
        for ti, term in enumerate(self.inputs):
            for vi, value in enumerate(term):
                owner = value.node if name2node is None else name2node[value.node.name]
                owner.uses.append((self, ti, vi))

    def _export_inputs(self):
        return [[value.export_config() for value in term] for term in self.inputs]

    def export_config(self):
        config = {'type': self.type, 'name': self.name, 'hint_name': self.hint_name,
                  'inputs': self._export_inputs()}
        for key in self._extra:
            config[key] = getattr(self, key)
        config['output_shape'] = self.output_shape
        return config

    # ---- shapes -------------------------------------------------------------------------------
    @property
    def input_shape(self):
        first = self.inputs[0][0].node.output_shape
        return (sum(term[0].length for term in self.inputs), first[1], first[2])

    def infer_shape(self):
        self.output_shape = self.input_shape

    # ---- work counters (reference ir.py:158-208) -------------------------------------------
    def _term_sizes(self):
        return [t[0].node.output_shape[1] * t[0].node.output_shape[2] * t[0].length for t in self.inputs]

    def input_flops(self):
        return sum(len(term) * size for term, size in zip(self.inputs, self._term_sizes()))

    def input_memory_access(self):
        sizes = self._term_sizes()
        total = sum(size * len(term) for term, size in zip(self.inputs, sizes) if len(term) > 1)
        if len(self.inputs) > 1:
            total += sum(sizes)
        return total

    def input_kernels(self):
        return sum(1 for term in self.inputs if len(term) > 1) + (1 if len(self.inputs) > 1 else 0)

    def _input_volume(self):
        c, h, w = self.input_shape
        return c * h * w

    def flops(self):
        return 0.0 + self.input_flops()

    def memory_access(self):
        return 0.0 + self.input_memory_access()

    def kernels(self):
        return self.input_kernels()

    # ---- printing -----------------------------------------------------------------------------
    def input_readable_str(self, merge_op='+'):
        terms = [merge_op.join(v.node.hint_name for v in term) for term in self.inputs]
        if len(terms) > 1:
            return "Concat(" + ",".join(terms) + ")"
        return '(' + terms[0] + ')' if len(self.inputs[0]) > 1 else terms[0]

    def readable_lines(self, indent) -> List[str]:
        raise NotImplementedError

    def __repr__(self):
        return self.name


def _op(kind):
    def register(cls):
        Node._registry[kind] = cls
        return cls
    return register


@_op('placeholder')
class Placeholder(Node):
    """Graph input (reference ``ir.py:240-273``)."""
    __slots__ = []

    def __init__(self, name, hint_name, output_shape):
        super().__init__('placeholder', name, hint_name, [[]], output_shape)

    @staticmethod
    def from_config(config, name2node):
        return Placeholder(config['name'], config['hint_name'], output_shape=config['output_shape'])

    def export_config(self):
        return {'type': 'placeholder', 'name': self.name, 'hint_name': self.hint_name,
                'output_shape': self.output_shape}

    def infer_shape(self):
        pass

    def flops(self):
        return 0.0

    def memory_access(self):
        return 0.0

    def kernels(self):
        return 0

    def readable_lines(self, indent):
        return [f'[{self.hint_name}]Placeholder']


@_op('conv')
class Conv(Node):
    """
    2-D cross-correlation + bias + activation (reference ``ir.py:276-396``).  ``weight`` is OIHW
    ``(Cout, Cin/groups, kh, kw)`` float32, ``bias`` is ``(Cout,)`` float32; both may be ``None``
    when a graph is only timed.
    """
    __slots__ = ['out_channels', 'kernel', 'stride', 'padding', 'groups', 'act', 'weight', 'bias']
    _extra = ('out_channels', 'kernel', 'stride', 'padding', 'groups', 'act')

    def __init__(self, name, hint_name, inputs, out_channels, kernel, stride, padding, groups, act, output_shape):
        super().__init__('conv', name, hint_name, inputs, output_shape)
        assert act in ('relu', 'sigmoid', 'tanh', 'identity')
        self.out_channels = out_channels
        self.kernel = kernel
        self.stride = stride
        self.padding = padding
        self.groups = groups
        self.act = act
        self.weight = None
        self.bias = None

    @classmethod
    def from_config(cls, config, name2node):
        return cls._load(config, name2node)

    def _export_inputs(self):
        return None if self.inputs is None else super()._export_inputs()

    @property
    def weight_shape(self):
        return (self.out_channels, self.input_shape[0] // self.groups, *self.kernel)

    @property
    def bias_shape(self):
        return self.out_channels,

    def init_weights(self):
        """Unseeded U(-b, b), b = 1/sqrt(fan_in), for weight and bias (reference ``ir.py:360-363``)."""
        bound = 1.0 / np.sqrt(self.kernel[0] * self.kernel[1] * self.input_shape[0] // self.groups)
        self.weight = np.random.uniform(low=-bound, high=bound, size=self.weight_shape).astype(np.float32)
        self.bias = np.random.uniform(low=-bound, high=bound, size=self.bias_shape).astype(np.float32)

    def infer_shape(self):
        _, h, w = self.input_shape
        self.output_shape = (self.out_channels,
                             _spatial_out(h, self.kernel[0], self.padding[0], self.stride[0]),
                             _spatial_out(w, self.kernel[1], self.padding[1], self.stride[1]))

    def flops(self):
        per_output = 1 + self.kernel[0] * self.kernel[1] * self.input_shape[0] // self.groups
        c, h, w = self.output_shape
        return c * h * w * per_output + self.input_flops()

    def memory_access(self):
        return self._input_volume() + self.input_memory_access()

    def kernels(self):
        return 1 + self.input_kernels()

    def readable_lines(self, indent):
        return [f'[{self.hint_name}]Conv2d({self.input_readable_str()})']


@_op('sequential')
class Sequential(Node):
    """Compound operator: inner nodes run in order as one schedule unit (reference ``ir.py:399-459``)."""
    __slots__ = ['nodes']

    def __init__(self, name, hint_name, nodes: List[Node], output_shape):
        super().__init__('sequential', name, hint_name, nodes[0].inputs, output_shape)
        self.nodes = nodes

    @staticmethod
    def from_config(config, name2node):
        inner = []
        for sub in config['nodes']:
            node = Node.from_config(sub, name2node)
            name2node[node.name] = node
            inner.append(node)
        seq = Sequential(config['name'], config['hint_name'], inner, config['output_shape'])
        seq._register_uses(name2node)
        return seq

    def export_config(self):
        return {'type': self.type, 'name': self.name, 'hint_name': self.hint_name,
                'nodes': [node.export_config() for node in self.nodes], 'output_shape': self.output_shape}

    def infer_shape(self):
        for node in self.nodes:
            node.infer_shape()
        self.output_shape = self.nodes[-1].output_shape

    def flops(self):
        return sum(node.flops() for node in self.nodes)

    def memory_access(self):
        return sum(node.memory_access() for node in self.nodes)

    def kernels(self):
        return sum(node.kernels() for node in self.nodes)

    def readable_lines(self, indent):
        lines = [f'[{self.hint_name}]Sequential(']
        for node in self.nodes:
            lines.extend(' ' * indent + line for line in node.readable_lines(indent))
        lines.append(')')
        return lines


_POOL_TITLES = {'max': 'MaxPool2d', 'avg': 'AvgPool2d', 'global_max': 'GlobalMaxPool2d',
                'global_avg': 'GlobalAvgPool2d'}


@_op('pool')
class Pool(Node):
    """max / avg (padding counted) / global pooling (reference ``ir.py:462-567``)."""
    __slots__ = ['pool_type', 'kernel', 'stride', 'padding']
    _extra = ('pool_type', 'kernel', 'stride', 'padding')

    def __init__(self, name, hint_name, inputs, pool_type, kernel, stride, padding, output_shape):
        super().__init__('pool', name, hint_name, inputs, output_shape)
        self.pool_type = pool_type
        self.kernel = kernel
        self.stride = stride
        self.padding = padding

    @classmethod
    def from_config(cls, config, name2node):
        return cls._load(config, name2node)

    def infer_shape(self):
        c, h, w = self.input_shape
        if self.pool_type == 'global_avg':
            # the whole map is one window (reference ir.py:532-535)
            self.stride = (1, 1)
            self.padding = (0, 0)
            self.kernel = (h, w)
        self.output_shape = [c,
                             _spatial_out(h, self.kernel[0], self.padding[0], self.stride[0]),
                             _spatial_out(w, self.kernel[1], self.padding[1], self.stride[1])]

    def flops(self):
        volume = self._input_volume()
        if 'global' in self.pool_type:
            return volume + self.input_flops()
        return volume * self.kernel[0] * self.kernel[1] + self.input_flops()

    def memory_access(self):
        return self._input_volume() + self.input_memory_access()

    def kernels(self):
        return 1 + self.input_kernels()

    def readable_lines(self, indent):
        return [f'[{self.hint_name}]{_POOL_TITLES[self.pool_type]}({self.input_readable_str()})']


@_op('element')
class Element(Node):
    """Element-wise sum (``add``) or product (``mul``) of the values of each term (reference ``ir.py:570-629``)."""
    __slots__ = ['op_type']
    _extra = ('op_type',)

    def __init__(self, name, hint_name, inputs, op_type, output_shape):
        super().__init__('element', name, hint_name, inputs, output_shape)
        self.op_type = op_type

    @classmethod
    def from_config(cls, config, name2node):
        return cls._load(config, name2node)

    def readable_lines(self, indent):
        return [f"[{self.hint_name}]{self.input_readable_str('*' if self.op_type == 'mul' else '+')}"]


@_op('identity')
class Identity(Node):
    """Materialises its input; with several terms it is the concat operator (reference ``ir.py:632-686``)."""
    __slots__ = []

    def __init__(self, name, hint_name, inputs, output_shape):
        super().__init__('identity', name, hint_name, inputs, output_shape)

    @classmethod
    def from_config(cls, config, name2node):
        return cls._load(config, name2node)

    def readable_lines(self, indent):
        text = self.input_readable_str()
        if text[0] != 'C':
            text = '(' + text + ')'
        return [f'[{self.hint_name}]{text}']


class _Pointwise(Node):
    __slots__ = []

    def flops(self):
        return 4 * self._input_volume() + self.input_flops()

    def memory_access(self):
        return self._input_volume() + self.input_memory_access()

    def kernels(self):
        return 1 + self.input_kernels()


@_op('activation')
class Activation(_Pointwise):
    """Stand-alone relu / tanh / sigmoid, optionally in place (reference ``ir.py:689-750``)."""
    __slots__ = ['act_type', 'inplace']
    _extra = ('act_type', 'inplace')

    def __init__(self, name, hint_name, inputs, act_type, inplace, output_shape):
        super().__init__('activation', name, hint_name, inputs, output_shape)
        self.act_type = act_type
        self.inplace = inplace

    @classmethod
    def from_config(cls, config, name2node):
        return cls._load(config, name2node)

    def readable_lines(self, indent):
        return [f'{self.act_type.capitalize()}@{self.hint_name}({self.input_readable_str()})']


@_op('relu')
class Relu(_Pointwise):
    """ReLU operator (reference ``ir.py:753-802``)."""
    __slots__ = []

    def __init__(self, name, hint_name, inputs, output_shape):
        super().__init__('relu', name, hint_name, inputs, output_shape)

    @classmethod
    def from_config(cls, config, name2node):
        return cls._load(config, name2node)

    def readable_lines(self, indent):
        return [f'[{self.hint_name}]Relu({self.input_readable_str()})']


class Block:
    """
    A DAG of operators between one enter node and one exit node, plus its schedule
    ``stages[stage][group] = [operator name, ...]``: stages run one after another, the groups of a
    stage run concurrently, the operators of a group run in order (reference ``ir.py:805-977``).
    """
    __slots__ = ['enter_node', 'exit_node', 'inner_nodes', 'stages', 'parts']

    def __init__(self, enter_node, exit_node=None, inner_nodes=None, stages=None):
        self.enter_node: Optional[Node] = enter_node
        self.exit_node: Optional[Node] = exit_node
        self.inner_nodes: List[Node] = [] if inner_nodes is None else inner_nodes
        self.stages = stages
        self.parts = None

    def _all_nodes(self) -> List[Node]:
        return self.inner_nodes + [self.exit_node]

    @staticmethod
    def from_config(config, name2node):
        enter = name2node[config['enter_name']]
        inner = []
        for node_config in config['inner_nodes']:
            node = Node.from_config(node_config, name2node)
            name2node[node.name] = node
            inner.append(node)
        exit_node = Node.from_config(config['exit_node'], name2node)
        name2node[exit_node.name] = exit_node
        return Block(enter, exit_node, inner, config['stages'])

    def export_config(self):
        return {
            'enter_name': self.enter_node.name,
            'enter_node': self.enter_node.export_config(),
            'inner_nodes': [node.export_config() for node in self.inner_nodes],
            'exit_node': self.exit_node.export_config(),
            'stages': self.stages,
        }

    def sequential_schedule(self):
        """One single-operator stage per node in definition order (reference ``ir.py:867-874``)."""
        self.stages = [[[node.name]] for node in self._all_nodes()]

    def greedy_schedule(self, max_num_stream):
        """Topological wavefronts, at most ``max_num_stream`` groups per stage (reference ``ir.py:876-907``)."""
        members = self._all_nodes()
        pending = {node: sum(len(term) for term in node.inputs) for node in members}
        frontier = [self.enter_node] + [node for node in members if len(node.inputs) == 0]
        self.stages = []
        while frontier:
            ready = [node for node in frontier if node is not self.enter_node]
            held = []
            if ready:
                ready, held = ready[:max_num_stream], ready[max_num_stream:]
                self.stages.append([[node.name] for node in ready])
                for node in held:
                    frontier.remove(node)
            released = []
            for node in frontier:
                if node is self.exit_node:
                    continue
                for user, _, _ in node.uses:
                    if user not in pending:
                        continue
                    pending[user] -= 1
                    if pending[user] == 0:
                        released.append(user)
            frontier = held + released
        assert sum(len(stage) for stage in self.stages) == len(members)

    def flops(self):
        return sum(node.flops() for node in self._all_nodes())

    def memory_access(self):
        return sum(node.memory_access() for node in self._all_nodes())

    def kernels(self):
        return sum(node.kernels() for node in self._all_nodes())

    def schedule_operators(self):
        return len(self._all_nodes())

    def readable_lines(self, indent=0):
        by_name = {node.name: node for node in self._all_nodes()}

        def shifted(lines):
            return [' ' * indent + line for line in lines]

        def group_lines(group):
            if len(group) == 1:
                return by_name[group[0]].readable_lines(indent)
            out = ['Sequential (']
            for name in group:
                out.extend(shifted(by_name[name].readable_lines(indent)))
            return out + [')']

        lines = []
        for stage in self.stages:
            if len(stage) == 1:
                lines.extend(group_lines(stage[0]))
            else:
                lines.append('Parallel(')
                for group in stage:
                    lines.extend(shifted(group_lines(group)))
                lines.append(')')
        return lines


class Graph:
    """A chain of blocks behind one placeholder (reference ``ir.py:980-1132``)."""
    __slots__ = ['name', 'input', 'input_shape', 'blocks']

    def __init__(self, name, input, blocks):
        self.name = name
        self.input: Placeholder = input
        self.blocks: List[Block] = blocks

    def nodes(self) -> Iterable[Node]:
        """Enter node, then every block's inner nodes and exit node: a topological order."""
        if not self.blocks:
            return
        yield self.blocks[0].enter_node
        for block in self.blocks:
            yield from block.inner_nodes
            yield block.exit_node

    @property
    def enter_node(self) -> Node:
        return self.blocks[0].enter_node

    @property
    def exit_node(self) -> Node:
        return self.blocks[-1].exit_node

    @staticmethod
    def from_config(config):
        name2node = {}
        source = Placeholder.from_config(config['input'], name2node)
        name2node[source.name] = source
        blocks = [Block.from_config(block_config, name2node) for block_config in config['blocks']]
        graph = Graph(config['name'], source, blocks)
        graph.infer_shape()
        return graph

    def export_config(self):
        return {'name': self.name, 'input': self.input.export_config(),
                'blocks': [block.export_config() for block in self.blocks]}

    def infer_shape(self):
        enter = self.blocks[0].enter_node
        for node in self.nodes():
            if node != enter:
                node.infer_shape()

    def convs(self) -> Iterable[Conv]:
        """Every Conv of the graph, those inside Sequential operators included, in graph order."""
        def walk(nodes):
            for node in nodes:
                if isinstance(node, Conv):
                    yield node
                elif isinstance(node, Sequential):
                    yield from walk(node.nodes)
        return walk(self.nodes())

    def init_weights(self):
        for conv in self.convs():
            conv.init_weights()

    def sequential_schedule(self):
        for block in self.blocks:
            block.sequential_schedule()

    def greedy_schedule(self, max_num_stream=10):
        for block in self.blocks:
            block.greedy_schedule(max_num_stream)

    def flops(self):
        return sum(block.flops() for block in self.blocks)

    def memory_access(self):
        return sum(block.memory_access() for block in self.blocks)

    def kernels(self):
        return sum(block.kernels() for block in self.blocks)

    def schedule_operators(self):
        return sum(block.schedule_operators() for block in self.blocks)

    def readable_lines(self, indent=0):
        lines = ['Sequential(']
        for block in self.blocks:
            lines.extend(' ' * indent + line for line in block.readable_lines(indent))
        lines.append(')')
        return lines

    def __str__(self):
        return "\n".join(self.readable_lines(2))
