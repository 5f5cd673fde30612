"""
The IOS dynamic-programming schedule search.

Behavioural counterpart of the reference's ``python/ios/optimizer.py``: a block's operators are
indexed 0..n-1, a DP state is the bitmask of operators that are still unscheduled, and a
transition removes an *ending* -- a set of operators closed under successors inside the state --
which becomes the last stage.  Two kinds of stage are tried (reference ``optimizer.py:513-593``):

* ``merge``: a subset of the sink operators that are convolutions reading the same value with equal
  stride / activation / resolution; it is timed (and later built) as ONE convolution whose output
  channels are the concatenation (``optimizer.py:245-278, 297-327``);
* ``parallel``: up to ``max_num_groups`` pairwise-disjoint groups, each the successor closure of
  one operator picked from a chain of a chain decomposition of the state, each at most
  ``max_group_size`` operators long (``optimizer.py:450-510``).

``cost(state) = min over endings (cost(state - ending) + latency(ending))`` and the chosen endings
are replayed front to back to rebuild the block (``optimizer.py:596-745``).  Enumeration order and
tie-breaking (strict ``<``, merge candidates first) follow the reference so that both produce the
same schedule from the same sequence of measurements.
"""
from typing import Dict, List, Optional, Set, Tuple
import functools
import itertools
import logging
import operator

import numpy as np

from ios.ir import Graph, Block, Conv, Value, Placeholder, Node, Sequential
from ios.cost_model import CostModel, IOSCostModel, RandomCostModel
from ios.utils import iter_subset

logging.disable(logging.WARNING)

IGraph = Dict[int, List[int]]
Stage = Tuple[List[List[int]], str]


# --------------------------------------------------------------------------------------------
# small bitmask / index-graph helpers
# --------------------------------------------------------------------------------------------
def count_bits(s):
    return bin(s).count('1')


def state2iset(s):
    """Indices of the set bits of ``s`` in increasing order."""
    out, i = [], 0
    while s:
        if s & 1:
            out.append(i)
        s >>= 1
        i += 1
    return out


def state2nset(s, idn):
    return [idn[i] for i in state2iset(s)]


def _mask(indices):
    return sum(1 << u for u in indices)


def log(info, verbose):
    if verbose:
        print(info)


def build_graph(all_nodes: List[Node], nid) -> IGraph:
    """Successor lists (by index) restricted to ``all_nodes`` (reference ``optimizer.py:343-354``)."""
    members = set(all_nodes)
    g: IGraph = {}
    for node in all_nodes:
        targets = []
        for user, _, _ in node.uses:
            if user in members:
                targets.append(nid[user])
        g[nid[node]] = list(set(targets))
    return g


def topological_order(graph: IGraph) -> List[int]:
    indeg = {u: 0 for u in graph}
    for u in graph:
        for v in graph[u]:
            indeg[v] += 1
    stack = [u for u in graph if indeg[u] == 0]
    order = []
    while stack:
        u = stack.pop()
        order.append(u)
        for v in graph[u]:
            indeg[v] -= 1
            if indeg[v] == 0:
                stack.append(v)
    assert len(order) == len(graph), 'the operator graph has a cycle'
    return order


def graph_transitive_closure(graph: IGraph, include_self=False) -> Dict[int, Set[int]]:
    closure: Dict[int, Set[int]] = {u: set() for u in graph}
    for u in reversed(topological_order(graph)):
        if include_self:
            closure[u].update([u])
        for v in graph[u]:
            closure[u].update(closure[v])
            closure[u].update([v])
    return closure


def transitive_closure_to_graph(tc) -> IGraph:
    return {u: list(tc[u]) for u in tc}


def longest_chain(graph: IGraph) -> List[int]:
    depth = {u: 1 for u in graph}
    follow: Dict[int, Optional[int]] = {u: None for u in graph}
    for u in reversed(topological_order(graph)):
        for v in graph[u]:
            if depth[u] < depth[v] + 1:
                depth[u] = depth[v] + 1
                follow[u] = v
    u = max(depth.keys(), key=lambda k: depth[k])
    chain = []
    while u is not None:
        chain.append(u)
        u = follow[u]
    return chain


def sub_graph(graph: IGraph, uset) -> IGraph:
    return {u: [v for v in graph[u] if v in uset] for u in graph if u in uset}


def graph_chain_decomposition(graph: IGraph) -> List[List[int]]:
    """Repeatedly peel the longest path off the transitive closure (reference ``optimizer.py:435-447``)."""
    chains = []
    graph = transitive_closure_to_graph(graph_transitive_closure(graph))
    while graph:
        chain = longest_chain(graph)
        chains.append(chain)
        graph = sub_graph(graph, set(graph.keys()) - set(chain))
    return chains


def get_input(ssnodes, block, nid, idn):
    """De-duplicated terms of several operators, sorted by (length, indices) (reference ``optimizer.py:222-233``)."""
    keyed = []
    for node in ssnodes:
        for term in node.inputs:
            keyed.append(tuple((-1 if v.node is block.enter_node else nid[v.node], v.begin, v.end) for v in term))
    unique = dict.fromkeys(sorted(keyed, key=lambda it: (len(it), it)))
    return [[Value(block.enter_node if src == -1 else idn[src], b, e) for src, b, e in it] for it in unique]


def check_merge(s, idn) -> bool:
    """Can the operators of ``s`` run as one merged convolution? (reference ``optimizer.py:245-278``)."""
    nodes = state2nset(s, idn)
    if len(nodes) == 1:
        return True
    head = None
    for node in nodes:
        if not isinstance(node, Conv):
            return False
        if head is None:
            head = node
            continue
        if (node.input_shape[1], node.input_shape[2]) != (head.input_shape[1], head.input_shape[2]):
            return False
        if (node.output_shape[1], node.output_shape[2]) != (head.output_shape[1], head.output_shape[2]):
            return False
        if (node.stride[0], node.stride[1]) != (head.stride[0], head.stride[1]):
            return False
        if node.groups != 1 or node.act != head.act:
            return False
        if len(node.inputs) > 1 or len(node.inputs[0]) > 1 or not (node.inputs[0][0] == nodes[0].inputs[0][0]):
            return False
    return True


def check_parallel(ss, successor_dict, max_num_streams):
    members = state2iset(ss)
    if len(members) > max_num_streams:
        return False
    closures = [successor_dict[u] for u in members]
    return all(a.isdisjoint(b) for a, b in itertools.combinations(closures, 2))


def _merged_conv_params(convs):
    """(out_channels, kernel, stride, padding) of the convolution that computes all of ``convs`` at once."""
    return (sum(c.out_channels for c in convs),
            (max(c.kernel[0] for c in convs), max(c.kernel[1] for c in convs)),
            (convs[0].stride[0], convs[0].stride[1]),
            (max(c.padding[0] for c in convs), max(c.padding[1] for c in convs)))


def ending_iterator(s: int, chains: List[List[int]], nid, idn, max_group_size: int, max_num_groups: int):
    """
    Enumerate the parallel endings of state ``s``: per chain pick nothing or one of the last
    ``max_group_size`` operators of the chain's prefix inside ``s``; the picks' successor closures
    must be pairwise disjoint and short enough (reference ``optimizer.py:450-510``).
    """
    members = state2iset(s)
    begins, lengths = [], []
    for chain in chains:
        end = 0
        for pos, u in enumerate(chain):
            if u not in members:
                break
            end = pos + 1
        begin = max(0, end - max_group_size)
        begins.append(begin)
        lengths.append(end - begin)
    radix = list(itertools.accumulate([n + 1 for n in lengths], operator.mul))
    closure = graph_transitive_closure(build_graph(state2nset(s, idn), nid), include_self=True)

    for code in range(radix[-1]):
        picks = []
        for i, chain in enumerate(chains):
            digit = (code % radix[i]) // (radix[i - 1] if i else 1)
            if digit != lengths[i]:
                picks.append(chain[begins[i] + digit])
        if not picks or len(picks) > max_num_groups:
            continue
        if any(not closure[a].isdisjoint(closure[b]) for a, b in itertools.combinations(picks, 2)):
            continue
        groups = [sorted(closure[u]) for u in picks]
        if any(len(group) > max_group_size for group in groups):
            continue
        yield groups


def latency(stage: Stage, block, merge_latency, parallel_latency, cost_model, idn, nid,
            batch_size, warmup, number, repeat) -> float:
    """Memoised mean latency of one candidate stage (reference ``optimizer.py:297-340``)."""
    groups, kind = stage
    key = _mask(itertools.chain(*groups))
    if kind == 'merge':
        if key not in merge_latency:
            nodes = state2nset(key, idn)
            if len(groups) == 1:
                assert len(nodes) == 1
                probe = nodes[0]
            else:
                assert all(isinstance(n, Conv) for n in nodes)
                out_channels, kernel, stride, padding = _merged_conv_params(nodes)
                probe = Conv('c', '', inputs=get_input(nodes, block, nid, idn), out_channels=out_channels,
                             kernel=kernel, stride=stride, padding=padding, groups=nodes[0].groups,
                             act=nodes[0].act, output_shape=None)
            merge_latency[key] = float(np.mean(
                cost_model.get_stage_latency([[probe]], batch_size, warmup, number, repeat)))
        return merge_latency[key]
    if kind == 'parallel':
        if key not in parallel_latency:
            stage_nodes = [[idn[u] for u in group] for group in groups]
            parallel_latency[key] = float(np.mean(
                cost_model.get_stage_latency(stage_nodes, batch_size, warmup, number, repeat)))
        return parallel_latency[key]
    raise ValueError(kind)


def dop(s: int, block, chains, on_debug, debug_dp_info, idn, nid, dp, ep, opt_type, max_group_size,
        max_num_groups, merge_latency, parallel_latency, cost_model, batch_size, warmup, number, repeat,
        bar_state) -> float:
    """Optimal latency of scheduling exactly the operators in ``s`` (reference ``optimizer.py:513-593``)."""
    if s == 0:
        return 0.0
    if s in dp:
        return dp[s]
    if on_debug:
        debug_dp_info['#states'][-1] += 1
        debug_dp_info['meta'][-1][s] = 0

    def recurse(rest):
        return dop(rest, block, chains, on_debug, debug_dp_info, idn, nid, dp, ep, opt_type, max_group_size,
                   max_num_groups, merge_latency, parallel_latency, cost_model, batch_size, warmup, number,
                   repeat, bar_state)

    def consider(stage, best):
        used = _mask(itertools.chain(*stage[0]))
        total = recurse(s - used)
        total = total + latency(stage, block, merge_latency, parallel_latency, cost_model, idn, nid,
                                batch_size, warmup, number, repeat)
        if on_debug:
            debug_dp_info['#transitions'][-1] += 1
            debug_dp_info['meta'][-1][s] += debug_dp_info['meta'][-1][s - used]
            if stage[1] == 'parallel':
                debug_dp_info['width'][-1] = max(debug_dp_info['width'][-1], len(stage[0]))
        if total < best:
            ep[s] = stage
            return total
        return best

    members = state2iset(s)
    inside = set(members)
    successors: Dict[int, Set[int]] = {u: set() for u in members}
    for u in reversed(members):
        successors[u].add(u)
        for user, _, _ in idn[u].uses:
            if user in nid and nid[user] in inside:
                successors[u].update(successors[nid[user]])

    best = 1e19
    if 'merge' in opt_type:
        sinks = _mask(u for u in members if len(successors[u]) == 1)
        for ss in iter_subset(sinks):
            if check_merge(ss, idn):
                best = consider(([[u] for u in state2iset(ss)], 'merge'), best)
    if 'parallel' in opt_type:
        for groups in ending_iterator(s, chains, nid, idn, max_group_size, max_num_groups):
            best = consider((groups, 'parallel'), best)
    dp[s] = best
    if bar_state is not None:
        bar_state.update(1)
    return best


# --------------------------------------------------------------------------------------------
# the same search in native code (csrc/dp_search.cc)
# --------------------------------------------------------------------------------------------
NATIVE_PART_LIMIT = 128


def _native_library():
    """The runtime library if it exports the native search, else None."""
    try:
        from ios.contrib import ios_runtime
        lib = ios_runtime._library()
        return lib if hasattr(lib, 'ios_dp_create') else None
    except (OSError, FileNotFoundError):
        return None


def _merge_keys(part: List[Node]):
    """
    Per operator: -1 if it is no convolution, else ``(class << 1) | plain``.  Two convolutions are of one class
    when they read the same first value at the same resolution with equal stride and activation; ``plain`` says
    groups == 1 and a single input value (what ``check_merge`` asks of every operator but the first of a set).
    """
    classes, keys = {}, []
    for node in part:
        if not isinstance(node, Conv):
            keys.append(-1)
            continue
        first = node.inputs[0][0]
        signature = (tuple(node.input_shape[1:]), tuple(node.output_shape[1:]), tuple(node.stride), node.act,
                     id(first.node), first.begin, first.end)
        cls = classes.setdefault(signature, len(classes))
        plain = node.groups == 1 and len(node.inputs) == 1 and len(node.inputs[0]) == 1
        keys.append((cls << 1) | (1 if plain else 0))
    return keys


def search_part_native(lib, part: List[Node], block, nid, idn, opt_type, max_group_size, max_num_groups, cost_model,
                       batch_size, warmup, number, repeat) -> List[Stage]:
    """
    One part of a block through the native search: enumerate the candidate stages (in the order the Python
    search would first ask for them), measure each through ``cost_model`` -- all of them at once if the model
    offers ``get_stage_latencies`` -- and let the native code evaluate the recurrence.  Returns the chosen
    stages, first stage first, with operators as block indices.
    """
    import ctypes
    n = len(part)
    local = {node: i for i, node in enumerate(part)}
    graph = build_graph(part, nid)
    chains = graph_chain_decomposition(graph)
    succ = []
    for node in part:
        mask = 0
        for v in graph[nid[node]]:
            mask |= 1 << local[idn[v]]
        succ.append(mask)
    lo = (ctypes.c_ulonglong * n)(*[m & 0xFFFFFFFFFFFFFFFF for m in succ])
    hi = (ctypes.c_ulonglong * n)(*[m >> 64 for m in succ])
    keys = (ctypes.c_int * n)(*_merge_keys(part))
    flat = [local[idn[u]] for chain in chains for u in chain]
    offsets = list(itertools.accumulate([0] + [len(chain) for chain in chains]))
    handle = ctypes.c_void_p(None)

    def check(status):
        if status != 0:
            lib.ios_last_error.restype = ctypes.c_char_p
            raise RuntimeError(f'native search error {status}: {lib.ios_last_error().decode(errors="replace")}')

    lib.ios_dp_create.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                  ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                  ctypes.POINTER(ctypes.c_void_p)]
    lib.ios_dp_set_latency.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_double]
    for name in ('ios_dp_enumerate', 'ios_dp_stage', 'ios_dp_solve', 'ios_dp_chosen', 'ios_dp_destroy'):
        getattr(lib, name).argtypes = None
    check(lib.ios_dp_create(n, lo, hi, keys, len(chains), (ctypes.c_int * len(offsets))(*offsets),
                            (ctypes.c_int * max(1, len(flat)))(*flat), 1 if 'merge' in opt_type else 0,
                            1 if 'parallel' in opt_type else 0, int(max_group_size), int(max_num_groups), ctypes.byref(handle)))
    try:
        count = ctypes.c_int(0)
        check(lib.ios_dp_enumerate(handle, ctypes.byref(count)))
        kind, groups_n = ctypes.c_int(0), ctypes.c_int(0)
        group_offsets, nodes = (ctypes.c_int * (n + 1))(), (ctypes.c_int * n)()
        candidates: List[Stage] = []
        for index in range(count.value):
            check(lib.ios_dp_stage(handle, index, ctypes.byref(kind), ctypes.byref(groups_n), group_offsets, nodes))
            groups = [[nid[part[nodes[k]]] for k in range(group_offsets[g], group_offsets[g + 1])]
                      for g in range(groups_n.value)]
            candidates.append((groups, 'merge' if kind.value == 0 else 'parallel'))
        # the measurements, in the order of first request
        probes = [_stage_probe(stage, block, idn, nid) for stage in candidates]
        many = getattr(cost_model, 'get_stage_latencies', None)
        if many is not None:
            values = many(probes, batch_size, warmup, number, repeat)
        else:
            values = [cost_model.get_stage_latency(probe, batch_size, warmup, number, repeat) for probe in probes]
        for index, value in enumerate(values):
            check(lib.ios_dp_set_latency(handle, index, ctypes.c_double(float(np.mean(value)))))
        chosen_n = ctypes.c_int(0)
        check(lib.ios_dp_solve(handle, ctypes.byref(chosen_n), None, None, None))
        chosen = (ctypes.c_int * max(1, chosen_n.value))()
        check(lib.ios_dp_chosen(handle, chosen))
        return [candidates[chosen[i]] for i in range(chosen_n.value)]
    finally:
        lib.ios_dp_destroy(handle)


def _stage_probe(stage: Stage, block, idn, nid) -> List[List[Node]]:
    """The operators handed to the cost model for one candidate stage (reference ``optimizer.py:297-340``)."""
    groups, kind = stage
    if kind == 'parallel':
        return [[idn[u] for u in group] for group in groups]
    nodes = [idn[group[0]] for group in groups]
    if len(nodes) == 1:
        return [[nodes[0]]]
    out_channels, kernel, stride, padding = _merged_conv_params(nodes)
    probe = Conv('c', '', inputs=get_input(nodes, block, nid, idn), out_channels=out_channels, kernel=kernel,
                 stride=stride, padding=padding, groups=nodes[0].groups, act=nodes[0].act, output_shape=None)
    return [[probe]]


def get_stage_list(ep, s):
    """Follow the recorded best endings from the full state down to the empty one; first stage first."""
    picked = []
    while s:
        picked.append(ep[s])
        s -= _mask(itertools.chain(*ep[s][0]))
    picked.reverse()
    return picked


# --------------------------------------------------------------------------------------------
# rebuilding a block from the chosen stages
# --------------------------------------------------------------------------------------------
class _BlockBuilder:
    """
    Replays the chosen stages into a new block (reference ``optimizer.py:609-745``).  ``where`` maps
    every old node to ``(new node, channel begin, channel end)``: a merged convolution serves each
    of its originals as a channel slice.
    """

    def __init__(self, block, new_enter, idn, nid, compute_weight):
        self.block, self.idn, self.nid = block, idn, nid
        self.compute_weight = compute_weight
        self.where = {block.enter_node: (new_enter, 0, new_enter.output_shape[0])}
        self.inner: List[Node] = []
        self.stages = []

    @staticmethod
    def fuse_adjacent(inputs: List[List[Value]]):
        """Join consecutive single-value terms that are adjacent slices of one node (``optimizer.py:622-638``)."""
        changed = True
        while changed:
            changed = False
            for i in range(1, len(inputs)):
                if len(inputs[i - 1]) > 1 or len(inputs[i]) > 1:
                    continue
                a, b = inputs[i - 1][0], inputs[i][0]
                if a.node == b.node and a.end == b.begin:
                    inputs = inputs[:i - 1] + [[Value(a.node, a.begin, b.end)]] + inputs[i + 1:]
                    changed = True
                    break
        return inputs

    def remap(self, terms, consumer, do_sort=True):
        mapped = []
        for term in terms:
            row = []
            for value in term:
                node, base, _ = self.where[value.node]
                row.append(Value(node, base + value.begin, base + value.end))
            mapped.append(row)
        if do_sort:
            mapped = sorted(mapped, key=lambda row: (len(row), row[0].node.name))
        for ti, row in enumerate(mapped):
            for vi, value in enumerate(row):
                value.node.uses.append((consumer, ti, vi))
        return mapped

    def _copy_weights(self, dst, src):
        if self.compute_weight and isinstance(dst, Conv):
            assert isinstance(src, Conv)
            dst.weight = src.weight.copy()
            dst.bias = src.bias.copy()

    def add_merged(self, indices):
        convs = [self.idn[i] for i in indices]
        assert all(isinstance(c, Conv) for c in convs)
        out_channels, kernel, stride, padding = _merged_conv_params(convs)
        terms = get_input(convs, self.block, self.nid, self.idn)
        merged = Conv(convs[0].name, " ".join(c.hint_name for c in convs), None, out_channels, kernel, stride,
                      padding, 1, convs[0].act, None)
        merged.inputs = self.remap(terms, merged)
        merged.infer_shape()
        if self.compute_weight:
            merged.weight = np.zeros(merged.weight_shape, dtype=np.float32)
            merged.bias = np.zeros(merged.bias_shape, dtype=np.float32)

        def same_term(ta, tb):
            return len(ta) == len(tb) and all(
                va.node == vb.node and va.begin == vb.begin and va.end == vb.end for va, vb in zip(ta, tb))

        out_begin = 0
        for conv in convs:
            out_end = out_begin + conv.out_channels
            k0 = ((kernel[0] - conv.kernel[0]) // 2, (kernel[1] - conv.kernel[1]) // 2)
            for term in conv.inputs:
                in_begin = 0
                for candidate in terms:
                    if same_term(term, candidate):
                        break
                    in_begin += candidate[0].length
                in_end = in_begin + term[0].length
                if self.compute_weight:
                    # smaller kernels sit centred in the merged kernel, zero elsewhere
                    merged.weight[out_begin:out_end, in_begin:in_end,
                                  k0[0]:k0[0] + conv.kernel[0], k0[1]:k0[1] + conv.kernel[1]] = conv.weight.copy()
                    merged.bias[out_begin:out_end] = conv.bias.copy()
            self.where[conv] = (merged, out_begin, out_end)
            out_begin = out_end
        merged.inputs = self.fuse_adjacent(merged.inputs)
        merged.infer_shape()
        self.inner.append(merged)
        self.stages.append([[merged.name]])

    def add_groups(self, groups):
        stage_names = []
        for group in groups:
            clones = []
            for old in (self.idn[i] for i in group):
                config = old.export_config()
                if isinstance(old, Sequential):
                    config['nodes'][0]['inputs'] = []
                    new = Node.from_config(config, {})
                    new.nodes[0].inputs = self.fuse_adjacent(self.remap(old.nodes[0].inputs, new, do_sort=False))
                    new.inputs = new.nodes[0].inputs
                    for dst, src in zip(new.nodes, old.nodes):
                        self._copy_weights(dst, src)
                else:
                    config['inputs'] = []
                    new = Node.from_config(config, {})
                    new.inputs = self.fuse_adjacent(self.remap(old.inputs, new, do_sort=False))
                    self._copy_weights(new, old)
                new.infer_shape()
                clones.append(new)
                self.where[old] = (new, 0, new.output_shape[0])
            self.inner.extend(clones)
            stage_names.append([node.name for node in clones])
        self.stages.append(stage_names)


def construct(stage_list: List[Stage], block, constructed_blocks, graph_enter, idn, nid, compute_weight) -> Block:
    new_enter = graph_enter if not constructed_blocks else constructed_blocks[-1].exit_node
    builder = _BlockBuilder(block, new_enter, idn, nid, compute_weight)
    for groups, kind in stage_list:
        if kind == 'merge' and len(groups) > 1:
            builder.add_merged(list(itertools.chain(*groups)))
        else:
            builder.add_groups(groups)
    new_exit = builder.inner.pop()
    return Block(new_enter, new_exit, builder.inner, builder.stages)


# --------------------------------------------------------------------------------------------
# entry points
# --------------------------------------------------------------------------------------------
def graph_dp_summary(graph: Graph, opt_type: str = 'dp_parallel_merge',
                     max_num_groups=8, max_part_size=50, max_group_size=3):
    """Run the search with a free cost model and return its statistics (reference ``optimizer.py:17-35``)."""
    info = {}
    optimize(graph, batch_size=1, cost_model=RandomCostModel(), opt_type=opt_type, warmup=1, number=1, repeat=1,
             max_num_groups=max_num_groups, max_part_size=max_part_size, max_group_size=max_group_size,
             compute_weight=False, debug_dp_info=info, verbose=False)
    return info


def optimize(graph: Graph,
             batch_size=1,
             cost_model: Optional[CostModel] = None,
             opt_type: str = 'dp_parallel_merge',
             warmup=2, number=6, repeat=6,
             max_num_groups=8, max_part_size=100, compute_weight=False, max_group_size=3,
             debug_dp_info=None, verbose=False, native=None) -> Graph:
    """
    Search an execution schedule for ``graph`` and return a NEW graph named ``{name}_{opt_type}``
    that carries it (signature and defaults of the reference, ``optimizer.py:37-43``).

    ``opt_type`` must contain ``parallel`` and/or ``merge`` (``dp_parallel``, ``dp_merge``,
    ``dp_parallel_merge``).  With ``compute_weight`` the convolutions of the new graph receive
    weights (merged ones zero-embedded); without it they have none and the graph can only be timed.

    ``native`` (not in the reference): run the enumeration and the recurrence in the runtime library
    (csrc/dp_search.cc) instead of in Python -- same candidate stages, same order of measurements, same
    schedule.  Default: whenever the library is there, no statistics are asked for and a part has at most
    128 operators.
    """
    if cost_model is None:
        cost_model = IOSCostModel()
    assert 'parallel' in opt_type or 'merge' in opt_type
    on_debug = debug_dp_info is not None
    if on_debug:
        assert isinstance(debug_dp_info, dict)
        for key in ('dp', 'stage_latency'):
            debug_dp_info[key] = {}
        for key in ('#states', '#transitions', '#schedules', 'width', '#operators', 'meta'):
            debug_dp_info[key] = []
    log(f"optimize {opt_type} on {graph.name}", verbose)

    bar_state = None
    if verbose:
        from tqdm import tqdm
        preview = graph_dp_summary(graph, opt_type, max_num_groups=1, max_part_size=max_part_size, max_group_size=1)
        bar_state = tqdm(total=sum(preview['#states']), desc='Progress')

    # prefetch hook: a cost model may ask to see every candidate stage before the first measurement
    prefetch = getattr(cost_model, 'prefetch_stages', None)
    if prefetch is not None and not getattr(cost_model, '_prefetching', False):
        prefetch(graph, dict(batch_size=batch_size, opt_type=opt_type, warmup=warmup, number=number, repeat=repeat,
                             max_num_groups=max_num_groups, max_part_size=max_part_size,
                             max_group_size=max_group_size))

    native_lib = None
    if native is not False and not on_debug and bar_state is None:
        native_lib = _native_library()
        if native and native_lib is None:
            raise RuntimeError('the native search was asked for but libios_runtime.so does not provide it')

    graph_enter = Placeholder(graph.input.name, graph.input.hint_name, graph.input.output_shape)
    graph_enter.output_shape = graph.enter_node.output_shape
    new_blocks: List[Block] = []

    for block in graph.blocks:
        all_nodes = block.inner_nodes + [block.exit_node]
        nid: Dict[Node, int] = {node: i for i, node in enumerate(all_nodes)}
        idn: Dict[int, Node] = dict(enumerate(all_nodes))

        parts = block.parts
        if parts is None:
            parts = [all_nodes[lo:lo + max_part_size] for lo in range(0, len(all_nodes), max_part_size)]

        stage_list: List[Stage] = []
        for part in parts:
            if native_lib is not None and len(part) <= NATIVE_PART_LIMIT:
                stage_list.extend(search_part_native(native_lib, part, block, nid, idn, opt_type, max_group_size,
                                                     max_num_groups, cost_model, batch_size, warmup, number, repeat))
                continue
            dp: Dict[int, float] = {}
            ep: Dict[int, Stage] = {}
            merge_latency: Dict[int, float] = {}
            parallel_latency: Dict[int, float] = {}
            chains = graph_chain_decomposition(build_graph(part, nid))
            if on_debug:
                for key in ('#states', '#transitions', '#schedules', 'width'):
                    debug_dp_info[key].append(0)
                debug_dp_info['#operators'].append(len(part))
                debug_dp_info['meta'].append({0: 1})

            full = _mask(nid[node] for node in part)
            dop(full, block, chains, on_debug, debug_dp_info, idn, nid, dp, ep, opt_type, max_group_size,
                max_num_groups, merge_latency, parallel_latency, cost_model, batch_size, warmup, number, repeat,
                bar_state)
            stage_list.extend(get_stage_list(ep, full))

            if on_debug:
                def names(mask):
                    return [nd.name for nd in state2nset(mask, idn)]
                for mask, value in parallel_latency.items():
                    debug_dp_info['stage_latency'][' '.join(['parallel'] + names(mask))] = value
                for mask, value in merge_latency.items():
                    debug_dp_info['stage_latency'][' '.join(['merge'] + names(mask))] = value
                for state, value in dp.items():
                    chosen = _mask(itertools.chain(*ep[state][0]))
                    debug_dp_info['dp'][' '.join(names(state))] = \
                        f"{value:.3f} ({ep[state][1]} {' '.join(names(chosen))})"
                debug_dp_info['#schedules'][-1] = debug_dp_info['meta'][-1][full]

        new_blocks.append(construct(stage_list, block, new_blocks, graph_enter, idn, nid, compute_weight))

    if bar_state is not None:
        bar_state.close()

    new_graph = Graph(graph.name + "_" + opt_type, graph_enter, new_blocks)
    new_graph.infer_shape()
    return new_graph
