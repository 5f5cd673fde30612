"""
The Python surface: IR wire format, schedules, printing and the DP optimizer.  No GPU: the search
runs on RandomCostModel, and the fixtures pin it to what the reference's optimizer produced from
the same numpy random seed (tests/golden/make_golden.py).
"""
import json

import numpy as np
import pytest

import ios
import ios_oracle as oracle
from helpers import load_ref_schedule, sample_block, seeded, sha, weights_of


def test_sample_block_names_and_print():
    graph = sample_block()
    graph.sequential_schedule()
    assert graph.input.name == '0'
    assert [n.name for n in graph.blocks[0].inner_nodes] == ['1', '2', '3', '4'] and graph.exit_node.name == '5'
    text = str(graph)
    assert text.splitlines() == ['Sequential(', '  [1]Conv2d(0)', '  [2]Conv2d(0)', '  [3]Conv2d(0)', '  [4]Conv2d(1)',
                                 '  [5]Concat(4,2,3)', ')']
    assert graph.blocks[0].stages == [[['1']], [['2']], [['3']], [['4']], [['5']]]
    assert graph.exit_node.output_shape == (1875, 15, 15)


def test_config_round_trip():
    for maker in (ios.models.inception_v3, ios.models.squeezenet, ios.models.randwire_small):
        graph = maker()
        graph.sequential_schedule()
        config = graph.export_config()
        clone = ios.Graph.from_config(json.loads(json.dumps(config)))
        assert json.dumps(clone.export_config()) == json.dumps(json.loads(json.dumps(config)))
        assert clone.flops() == graph.flops() and clone.kernels() == graph.kernels()


def test_model_shapes():
    g = ios.models.inception_v3()
    assert g.exit_node.output_shape == [2048, 1, 1]
    assert len(g.blocks) == 13 and len(list(g.convs())) == 94
    g = ios.models.squeezenet()
    assert g.exit_node.output_shape == [1000, 1, 1] and len(list(g.convs())) == 30
    g = ios.models.randwire_small()
    assert g.exit_node.output_shape == [1280, 1, 1]
    convs = list(g.convs())
    assert len(convs) == 195 and sum(1 for c in convs if c.groups > 1) == 96
    assert [b.exit_node.output_shape for b in g.blocks[1:4]] == [(78, 28, 28), (156, 14, 14), (312, 7, 7)]


def test_model_zoo_exports_equal_the_reference_exports(golden):
    """Graphs that are only hashed (resnet50 cannot execute in the reference either: its bottleneck adds 64 to 256 channels)."""
    for case, maker in (('resnet50', ios.models.resnet50), ('vgg_16', ios.models.vgg_16), ('alexnet', ios.models.alexnet)):
        assert sha(maker().export_config()) == golden.meta(case + '_config')['config_sha256'], case
    g = ios.models.resnet18()
    assert g.exit_node.output_shape == (512, 7, 7) or list(g.exit_node.output_shape) == [512, 7, 7]
    assert g.blocks[0].stages is not None            # the reference hands its ResNets back with the sequential schedule


def test_nasnet_parts_follow_the_cells(golden):
    g = ios.models.nasnet_large()
    block = g.blocks[0]
    assert [[n.name for n in part] for part in block.parts] == golden.meta('nasnet_large')['parts']
    assert sum(len(p) for p in block.parts) == len(block.inner_nodes) + 1
    # the search works part by part: a random cost model is enough to see that every operator is scheduled once
    np.random.seed(1)
    opt = ios.optimize(g, batch_size=1, cost_model=ios.RandomCostModel(), opt_type='dp_parallel_merge', max_group_size=1,
                       max_num_groups=3)
    names = [n for stage in opt.blocks[0].stages for group in stage for n in group]
    assert len(names) == len(set(names)) == len(opt.blocks[0].inner_nodes) + 1


def test_greedy_schedule_covers_every_operator():
    g = ios.models.inception_v3()
    g.greedy_schedule(max_num_stream=4)
    for block in g.blocks:
        names = [n for stage in block.stages for group in stage for n in group]
        assert sorted(names) == sorted(n.name for n in block.inner_nodes + [block.exit_node])
        assert all(len(stage) <= 4 for stage in block.stages)


@pytest.mark.parametrize('model,opt_type', [('squeezenet', 'dp_parallel_merge'), ('inception_v3', 'dp_parallel_merge'),
                                            ('inception_v3', 'dp_parallel')])
def test_optimizer_reproduces_reference_schedule(golden, model, opt_type):
    graph = getattr(ios.models, model)()
    config, weights = seeded(graph, 0)
    np.random.seed(7)
    opt = ios.optimize(graph, batch_size=1, cost_model=ios.RandomCostModel(), opt_type=opt_type, compute_weight=True,
                       max_part_size=50)
    case = f'{model}_{opt_type}_seed7'
    meta = golden.meta(case)
    out_config = opt.export_config()
    assert sha(out_config) == meta['config_sha256'], 'the optimized graph differs from the reference optimizer output'
    assert sum(len(b.stages) for b in opt.blocks) == meta['num_stages']
    assert opt.name == f'{model}_{opt_type}'
    # merged weights included: the optimized graph computes the same function
    y = oracle.run_config(out_config, weights_of(opt), oracle.normal_input(out_config, 1, 0))
    golden.expect(case, y, 2e-5)
    y_seq = oracle.run_config(config, weights, oracle.normal_input(config, 1, 0))
    assert oracle.max_rel_err(y, y_seq) < 2e-5


def test_schedule_invariance_random_schedules():
    """Any schedule the search can emit computes the same function as the sequential one."""
    graph = ios.models.squeezenet()
    config, weights = seeded(graph, 2, law='uniform')
    x = oracle.normal_input(config, 2, 9)
    y_seq = oracle.run_config(config, weights, x)
    for seed, opt_type in ((1, 'dp_parallel'), (2, 'dp_merge'), (3, 'dp_parallel_merge')):
        np.random.seed(seed)
        opt = ios.optimize(graph, batch_size=2, cost_model=ios.RandomCostModel(), opt_type=opt_type,
                           compute_weight=True, max_group_size=2, max_num_groups=4)
        y = oracle.run_config(opt.export_config(), weights_of(opt), x)
        assert oracle.max_rel_err(y, y_seq) < 2e-5


def test_optimize_sample_block_structure():
    graph = sample_block()
    np.random.seed(0)
    info = {}
    opt = ios.optimize(graph, batch_size=1, cost_model=ios.RandomCostModel(), opt_type='dp_parallel',
                       compute_weight=True, debug_dp_info=info)
    names = sorted(n for stage in opt.blocks[0].stages for group in stage for n in group)
    assert names == ['1', '2', '3', '4', '5']
    assert opt.name == 'demo_dp_parallel'
    assert info['#operators'] == [5] and info['#states'][0] > 0 and info['#transitions'][0] > 0
    # without compute_weight the new convolutions carry no weights
    opt2 = ios.optimize(graph, batch_size=1, cost_model=ios.RandomCostModel(), opt_type='dp_merge')
    assert all(c.weight is None for c in opt2.convs())


def test_reference_schedule_fixtures_load():
    for name in ('1', '16', '32', '64', '128', 'k80', 'v100'):
        graph = ios.Graph.from_config(load_ref_schedule(name))
        assert len(graph.blocks) == 13
        for block in graph.blocks:
            scheduled = [n for stage in block.stages for group in stage for n in group]
            assert sorted(scheduled) == sorted(n.name for n in block.inner_nodes + [block.exit_node])


def test_iter_subset_and_counters():
    from ios.utils import iter_subset
    assert list(iter_subset(0b101)) == [0b101, 0b100, 0b001]
    assert list(iter_subset(0b11, include_emtpy_set=True)) == [3, 2, 1, 0]
    g = sample_block()
    assert g.flops() > 0 and g.schedule_operators() == 5


@pytest.mark.parametrize('model,opt_type,kwargs', [
    ('sample_block', 'dp_parallel_merge', {}), ('squeezenet', 'dp_parallel_merge', {}), ('squeezenet', 'dp_merge', {}),
    ('inception_v3', 'dp_parallel_merge', {'max_part_size': 50}), ('inception_v3', 'dp_parallel', {'max_part_size': 50}),
    ('resnet18', 'dp_parallel_merge', {}), ('randwire_small', 'dp_parallel_merge', {'max_group_size': 1, 'max_num_groups': 3}),
])
def test_native_search_equals_the_python_search(model, opt_type, kwargs):
    """Same candidate stages, same order of measurements, same schedule: the exported graphs are identical."""
    results = []
    for native in (False, True):
        graph = sample_block() if model == 'sample_block' else getattr(ios.models, model)()
        np.random.seed(11)
        opt = ios.optimize(graph, batch_size=1, cost_model=ios.RandomCostModel(), opt_type=opt_type, native=native, **kwargs)
        results.append(json.dumps(opt.export_config()))
    assert results[0] == results[1]


def test_native_search_asks_for_all_stages_at_once_when_the_cost_model_can():
    class Batched(ios.cost_model.CostModel):
        calls = 0

        def get_stage_latencies(self, stages, batch_size, warmup, number, repeat):
            Batched.calls += 1
            return [[float(sum(len(group) for group in stage)) + 0.25 * len(stage)] * repeat for stage in stages]

    graph = ios.models.squeezenet()
    opt = ios.optimize(graph, batch_size=1, cost_model=Batched(), opt_type='dp_parallel_merge', native=True)
    assert Batched.calls == len(graph.blocks)             # one request per block (each block is one part)
    names = [n for block in opt.blocks for stage in block.stages for group in stage for n in group]
    assert len(names) == len(set(names))


def test_native_search_rejects_bad_input():
    import ctypes
    from ios.contrib import ios_runtime as rt
    lib = rt.load_ios_library()
    handle = ctypes.c_void_p(None)
    lo, hi, keys = (ctypes.c_ulonglong * 2)(1, 0), (ctypes.c_ulonglong * 2)(0, 0), (ctypes.c_int * 2)(-1, -1)
    offsets, nodes = (ctypes.c_int * 2)(0, 2), (ctypes.c_int * 2)(0, 1)
    # operator 0 lists itself as a successor: not a topological order
    assert lib.ios_dp_create(2, lo, hi, keys, 1, offsets, nodes, 1, 1, 3, 8, ctypes.byref(handle)) == 3
    assert lib.ios_dp_create(200, lo, hi, keys, 1, offsets, nodes, 1, 1, 3, 8, ctypes.byref(handle)) == 6
    lo = (ctypes.c_ulonglong * 2)(2, 0)
    assert lib.ios_dp_create(2, lo, hi, keys, 1, offsets, nodes, 0, 1, 3, 8, ctypes.byref(handle)) == 0
    count = ctypes.c_int(0)
    assert lib.ios_dp_enumerate(handle, ctypes.byref(count)) == 0 and count.value == 3      # {0,1}, then {0} (met while descending), then {1}
    chosen = ctypes.c_int(0)
    assert lib.ios_dp_solve(handle, ctypes.byref(chosen), None, None, None) == 3            # latencies are missing
    lib.ios_dp_set_latency.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_double]
    for index, value in enumerate((2.0, 0.5, 0.75)):
        assert lib.ios_dp_set_latency(handle, index, value) == 0
    best = ctypes.c_double(0.0)
    assert lib.ios_dp_solve(handle, ctypes.byref(chosen), ctypes.byref(best), None, None) == 0
    assert chosen.value == 2 and abs(best.value - 1.25) < 1e-12                            # two stages beat the joint one
    order = (ctypes.c_int * 2)()
    assert lib.ios_dp_chosen(handle, order) == 0 and list(order) == [1, 2]                  # {0} first, then {1}
    lib.ios_dp_destroy(handle)
