"""
Graph-builder helpers: the functions user scripts call to append operators to a block.

Behavioural counterpart of the reference's ``python/ios/models/common.py``.  Operators are named by
a process-wide counter rendered as a decimal string; ``placeholder`` consumes a name too, compound
operators consume one name per inner node and then one for the Sequential
(reference ``common.py:9-27, 347, 395, 435``).
"""
from typing import List, Tuple

from ios.ir import (Placeholder, Conv, Pool, Relu, Identity, Value, Node, Block, Sequential, Activation,
                    Element, Graph)

name_index = 0


def new_name():
    global name_index
    name = str(name_index)
    name_index += 1
    return name


def reset_name():
    global name_index
    name_index = 0


def _attach(block: Block, node: Node, is_exit: bool, users_of=None) -> Value:
    """Infer the shape, register the node with its producers and with the block, return its full Value."""
    node.infer_shape()
    for ti, term in enumerate(node.inputs if users_of is None else users_of):
        for vi, value in enumerate(term):
            value.node.uses.append((node, ti, vi))
    if is_exit:
        block.exit_node = node
    else:
        block.inner_nodes.append(node)
    return Value(node, 0, node.output_shape[0])


def placeholder(output_shape):
    name = new_name()
    holder = Placeholder(name, name, output_shape)
    return Value(holder, 0, holder.output_shape[0])


def conv2d(block: Block, inputs, out_channels, kernel=(1, 1), stride=(1, 1), padding=(0, 0), groups=1, act="relu",
           is_exit=False):
    name = new_name()
    return _attach(block, Conv(name, name, inputs, out_channels, kernel, stride, padding, groups, act, None), is_exit)


def pool2d(block: Block, inputs, pool_type, kernel=(1, 1), stride=(1, 1), padding=(0, 0), is_exit=False):
    name = new_name()
    return _attach(block, Pool(name, name, inputs, pool_type, kernel, stride, padding, None), is_exit)


def identity(block: Block, inputs, is_exit=False):
    name = new_name()
    return _attach(block, Identity(name, name, inputs, None), is_exit)


def relu(block: Block, inputs, is_exit=False):
    name = new_name()
    return _attach(block, Relu(name, name, inputs, None), is_exit)


def activation(block: Block, inputs, act_type, inplace, is_exit=False):
    name = new_name()
    return _attach(block, Activation(name, name, inputs, act_type=act_type, inplace=inplace, output_shape=None),
                   is_exit)


def sigmoid(block: Block, inputs, inplace=False, is_exit=False):
    return activation(block, inputs, 'sigmoid', inplace, is_exit)


def tanh(block: Block, inputs, inplace=False, is_exit=False):
    return activation(block, inputs, 'tanh', inplace, is_exit)


def element(block: Block, inputs, op_type, is_exit=False):
    name = new_name()
    return _attach(block, Element(name, name, inputs, op_type=op_type, output_shape=None), is_exit)


def multiply(block: Block, inputs, is_exit=False):
    return element(block, inputs, op_type='mul', is_exit=is_exit)


def addition(block: Block, inputs, is_exit=False):
    return element(block, inputs, op_type='add', is_exit=is_exit)


def sequential(block: Block, hint_name, nodes: List[Node], is_exit=False):
    """Chain ``nodes`` (each takes the previous one as its only input) into one schedule unit."""
    name = new_name()
    for prev, nxt in zip(nodes, nodes[1:]):
        prev.infer_shape()
        nxt.inputs = [[Value(prev, 0, prev.output_shape[0])]]
    seq = Sequential(name, name if hint_name is None else hint_name, nodes, None)
    return _attach(block, seq, is_exit, users_of=nodes[0].inputs)


def _depthwise_then_pointwise(inputs, out_channels, kernel, stride, padding):
    in_channels = sum(term[0].node.output_shape[0] for term in inputs)
    dw_name, pw_name = new_name(), new_name()
    return [
        Conv(dw_name, dw_name, inputs, out_channels=in_channels, kernel=kernel, stride=stride, padding=padding,
             groups=in_channels, act="identity", output_shape=None),
        Conv(pw_name, pw_name, None, out_channels=out_channels, kernel=(1, 1), stride=(1, 1), padding=(0, 0),
             groups=1, act="identity", output_shape=None),
    ]


def sep_conv(block: Block, inputs: List[List[Value]], out_channels, kernel, stride, padding, is_exit=False):
    """Depthwise k x k followed by pointwise 1 x 1, no activation (reference ``common.py:379-403``)."""
    nodes = _depthwise_then_pointwise(inputs, out_channels, kernel, stride, padding)
    return sequential(block, hint_name='SepConv', nodes=nodes, is_exit=is_exit)


def relu_sep_conv(block: Block, inputs: List[List[Value]], out_channels, kernel, stride, padding, is_exit=False):
    """ReLU, depthwise k x k, pointwise 1 x 1 (reference ``common.py:406-444``)."""
    relu_name = new_name()
    head = Relu(relu_name, relu_name, inputs, None)
    nodes = [head] + _depthwise_then_pointwise(inputs, out_channels, kernel, stride, padding)
    nodes[1].inputs = None
    return sequential(block, hint_name='ReluSepConv', nodes=nodes, is_exit=is_exit)


def relu_conv(block: Block, inputs, out_channels, kernel=(1, 1), stride=(1, 1), padding=(0, 0), groups=1,
              is_exit=False):
    relu_name, conv_name = new_name(), new_name()
    nodes = [
        Relu(relu_name, relu_name, inputs, None),
        Conv(conv_name, conv_name, None, out_channels=out_channels, kernel=kernel, stride=stride, padding=padding,
             groups=groups, act="identity", output_shape=None),
    ]
    return sequential(block, hint_name='ReluConv', nodes=nodes, is_exit=is_exit)


def rwconv2d(block: Block, inputs, out_channels, stride=(1, 1), is_exit=False):
    """The RandWire node operator: ReLU -> depthwise 3x3 -> pointwise 1x1."""
    return relu_sep_conv(block, inputs, out_channels, (3, 3), stride, (1, 1), is_exit)


def get_parts(block, split_vars: List[Value]):
    """
    Split a block's nodes into parts delimited by the (integer) names of ``split_vars``: part i
    holds the nodes whose name n satisfies ``split[i] < n <= split[i+1]`` (reference ``common.py:494-516``).
    """
    marks = [int(v.node.name) for v in split_vars]
    parts = [[] for _ in range(len(marks) - 1)]
    for node in block.inner_nodes + [block.exit_node]:
        idx = int(node.name)
        where = [i for i in range(len(marks) - 1) if marks[i] < idx <= marks[i + 1]]
        assert where, f'node {node.name} lies outside the split points {marks}'
        parts[where[-1]].append(node)
    return parts
