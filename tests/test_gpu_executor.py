"""
GPU tests of the executor's variants and of the boundary as the reference binds it: data-flow edges
instead of stage barriers, programmatic edges in captured schedules, plain stores instead of bulk
tensor stores, global max pooling, the four drop-in ``void`` symbols called exactly as the
reference's ctypes front-end calls them, the pipelined host-buffer entry point and engines driven
from several host threads.
"""
import ctypes
import json
import threading

import numpy as np
import pytest

import ios
import ios_oracle as oracle
from ios.contrib import ios_runtime as rt
from helpers import TOL_FP32, TOL_TF32, sample_block, seeded, set_weights, weights_of

pytestmark = pytest.mark.gpu

DEFAULTS = (('precision', 'tf32x3'), ('pdl', '1'), ('executor', 'graph'), ('conv', 'auto'), ('split_k', '0'),
            ('im2col', '1'), ('persistent', '1'), ('stem', '1'), ('bulk_store', '1'), ('stage_barriers', '1'),
            ('pdl_edges', '0'), ('cluster_push', '1'), ('dual_issue', '1'), ('weight_prefetch', '1'))


@pytest.fixture(autouse=True)
def default_options():
    for key, value in DEFAULTS:
        rt.set_option(key, value)
    yield
    for key, value in DEFAULTS:
        rt.set_option(key, value)


def _seeded_dp_graph(model, seed=7, opt_type='dp_parallel_merge'):
    graph = getattr(ios.models, model)()
    config, weights = seeded(graph, 0)
    np.random.seed(seed)
    opt = ios.optimize(graph, batch_size=1, cost_model=ios.RandomCostModel(), opt_type=opt_type, compute_weight=True,
                       max_part_size=50)
    return opt, config


@pytest.mark.parametrize('option', ['stage_barriers', 'pdl_edges'])
@pytest.mark.parametrize('model', ['inception_v3', 'squeezenet'])
def test_executor_variants_reproduce_the_reference_outputs(golden, model, option):
    """Data-flow edges (stage_barriers=0) and programmatic edges (pdl_edges=1) compute the same bits as the default."""
    opt, config = _seeded_dp_graph(model)
    x = oracle.normal_input(config, 1, 0)
    base = rt.graph_inference(opt, 1, x)
    golden.expect(f'{model}_dp_parallel_merge_seed7', base, TOL_TF32)
    rt.set_option(option, '0' if option == 'stage_barriers' else '1')
    rt.set_option('weight_prefetch', '0' if option == 'pdl_edges' else '1')     # (no effect on results either way)
    for executor in ('graph', 'streams'):
        rt.set_option('executor', executor)
        y = rt.graph_inference(opt, 1, x)
        assert np.array_equal(y, base), (option, executor)
    rt.set_option('executor', 'graph')
    engine = rt.Engine(opt, 1)
    try:
        info = engine.describe()
        assert info['stage_barriers'] == (0 if option == 'stage_barriers' else 1)
        assert info['pdl_edges'] == info['pdl_edges_applied'] == (1 if option == 'pdl_edges' else 0)
        for _ in range(3):
            assert np.array_equal(engine.run(x), base)
        assert engine.time(5) > 0
    finally:
        engine.close()


def test_both_variants_together_on_a_wide_graph(golden):
    graph = ios.models.randwire_small()
    graph.greedy_schedule()
    config, weights = seeded(graph, 0)
    x = oracle.normal_input(config, 1, 0)
    base = rt.graph_inference(graph, 1, x)
    golden.expect('randwire_small', base, TOL_TF32)
    rt.set_option('stage_barriers', '0')
    rt.set_option('pdl_edges', '1')
    assert np.array_equal(rt.graph_inference(graph, 1, x), base)
    lat = rt.graph_latency(graph, 1, 1, 2, 2)
    assert all(0 < v < 100 for v in lat)


def test_plain_stores_equal_bulk_tensor_stores(golden):
    graph = ios.models.squeezenet()
    graph.sequential_schedule()
    config, weights = seeded(graph, 0)
    x = oracle.normal_input(config, 3, 5)
    base = rt.graph_inference(graph, 3, x)
    assert oracle.max_rel_err(base, oracle.run_config(config, weights, x)) <= TOL_TF32
    rt.set_option('bulk_store', '0')
    engine = rt.Engine(graph, 3)
    try:
        info = engine.describe()
        assert info['conv_tc_direct_store'] == info['conv_tc'] > 0
        assert np.array_equal(engine.run(x), base)
    finally:
        engine.close()
    # a many-tile layer through the resident kernel, and a split-K layer, stored from registers
    rng = np.random.default_rng(2)
    for shape in ((8, 64, 35, 35, 200), (1, 160, 8, 8, 96)):
        n, cin, h, w, cout = shape
        xs = rng.standard_normal((n, cin, h, w)).astype(np.float32)
        wt = (rng.standard_normal((cout, cin, 3, 3)) / np.sqrt(9 * cin)).astype(np.float32)
        b = rng.standard_normal(cout).astype(np.float32) * 0.1
        ref = oracle.conv2d_numpy(xs, wt, b, (1, 1), (1, 1), 1, 'relu')
        assert oracle.max_rel_err(rt.conv2d(xs, wt, b, padding=(1, 1), act='relu', impl='tensor'), ref) <= TOL_FP32


@pytest.mark.parametrize('precision,tol', [('tf32x3', TOL_FP32), ('tf32', TOL_TF32), ('bf16', 2e-2)])
def test_split_k_exchange_and_issue_variants(precision, tol):
    """Split-K clusters: partial tiles pushed through shared memory (default) or exchanged through the workspace in L2 give
    the same bits; three-pass products issued by two threads or by one agree with the oracle.  Covers full tiles, a
    ragged last tile (17 x 17 = 289 pixels), a tile of 64 valid rows (8 x 8), wide tiles and every cluster size."""
    rt.set_option('precision', precision)
    rng = np.random.default_rng(11)
    shapes = [(1, 768, 17, 17, 192, 1, 0), (1, 2048, 8, 8, 320, 1, 0), (1, 448, 8, 8, 384, 3, 1), (1, 288, 35, 35, 64, 1, 0),
              (2, 160, 17, 17, 192, 3, 1), (1, 1280, 8, 8, 448, 1, 0), (1, 96, 9, 9, 40, 3, 1)]
    for n, cin, h, w, cout, k, pad in shapes:
        xs = rng.standard_normal((n, cin, h, w)).astype(np.float32)
        wt = (rng.standard_normal((cout, cin, k, k)) / np.sqrt(k * k * cin)).astype(np.float32)
        b = rng.standard_normal(cout).astype(np.float32) * 0.1
        ref = oracle.conv2d_numpy(xs, wt, b, (1, 1), (pad, pad), 1, 'relu')
        for split in ('0', '2', '4', '8', '3'):
            rt.set_option('split_k', split)
            outs = {}
            for push in ('1', '0'):
                for dual in ('1', '0'):
                    rt.set_option('cluster_push', push)
                    rt.set_option('dual_issue', dual)
                    y = rt.conv2d(xs, wt, b, padding=(pad, pad), act='relu', impl='tensor')
                    bound = 2 * tol if (precision == 'tf32x3' and k * k * cin > 2000) else tol    # long sums in fp32
                    assert oracle.max_rel_err(y, ref) <= bound, (precision, (n, cin, h, w, cout, k), split, push, dual)
                    outs[(push, dual)] = y
            for dual in ('1', '0'):
                assert np.array_equal(outs[('1', dual)], outs[('0', dual)]), ('exchange changes bits', (n, cin, h, w, cout, k), split, dual)
            # the same call again: the result does not depend on timing
            rt.set_option('cluster_push', '1')
            rt.set_option('dual_issue', '1')
            again = rt.conv2d(xs, wt, b, padding=(pad, pad), act='relu', impl='tensor')
            assert np.array_equal(again, outs[('1', '1')])


@pytest.mark.parametrize('precision,tol', [('tf32x3', TOL_FP32), ('bf16', 2e-2), ('fp32', TOL_FP32)])
def test_global_max_and_global_avg_pooling(precision, tol):
    ios.reset_name()
    v = ios.placeholder(output_shape=(40, 9, 7))
    block = ios.Block(enter_node=v.node)
    c = ios.conv2d(block, [[v]], out_channels=24, kernel=(3, 3), padding=(1, 1), act='tanh')
    gm = ios.pool2d(block, [[c]], pool_type='global_max', kernel=(9, 7))     # the IR infers the window of global_avg only (reference ir.py:531-535)
    ga = ios.pool2d(block, [[c]], pool_type='global_avg')
    ios.identity(block, [[gm], [ga]], is_exit=True)
    graph = ios.Graph('pools', v.node, [block])
    graph.sequential_schedule()
    config, weights = seeded(graph, 3, 'uniform')
    x = oracle.normal_input(config, 5, 1)
    rt.set_option('precision', precision)
    y = rt.graph_inference(graph, 5, x)
    ref = oracle.run_config(config, weights, x)
    assert y.shape == (5, 48, 1, 1)
    assert oracle.max_rel_err(y, ref) <= tol
    assert oracle.max_rel_err(y, oracle.run_config_numpy(config, weights, x)) <= tol


# ---- the four drop-in symbols, bound the way the reference binds them --------------------------------
def _raw_library():
    """A second handle without argtypes / restype, as python/ios/contrib/ios_runtime.py:18-23 of the reference loads it."""
    return ctypes.cdll.LoadLibrary(rt.load_ios_library()._name)


def _c_string(text):
    return ctypes.c_char_p(text.encode())


def test_void_symbols_called_like_the_reference_front_end():
    lib = _raw_library()
    graph = sample_block()
    graph.sequential_schedule()
    config = graph.export_config()
    repeat, number, warmup = 3, 2, 1
    num_stages = sum(len(b.stages) for b in graph.blocks)

    # graph_latency (reference ios_runtime.py:26-50)
    results = (ctypes.c_float * repeat)()
    stage_results = (ctypes.c_float * (repeat * num_stages))()
    lib.graph_latency(_c_string(json.dumps(config)), ctypes.c_int(1), ctypes.c_int(warmup), ctypes.c_int(number),
                      ctypes.c_int(repeat), ctypes.c_int(1), ctypes.cast(results, ctypes.POINTER(ctypes.c_float)),
                      ctypes.cast(stage_results, ctypes.POINTER(ctypes.c_float)))
    lat = [float(v) for v in results]
    per_stage = np.array([float(v) for v in stage_results]).reshape(repeat, num_stages)
    assert all(0 < v < 100 for v in lat) and (per_stage > 0).all()

    # block_latency (:53-77)
    block = graph.blocks[0]
    results = (ctypes.c_float * repeat)()
    stage_results = (ctypes.c_float * (repeat * len(block.stages)))()
    lib.block_latency(_c_string(json.dumps(block.export_config())), ctypes.c_int(1), ctypes.c_int(warmup),
                      ctypes.c_int(number), ctypes.c_int(repeat), ctypes.c_int(0),
                      ctypes.cast(results, ctypes.POINTER(ctypes.c_float)),
                      ctypes.cast(stage_results, ctypes.POINTER(ctypes.c_float)))
    assert all(0 < float(v) < 100 for v in results)

    # stage_latency (:80-111)
    nodes = block.inner_nodes
    stage_text, input_text = rt.stage_config([[nodes[0], nodes[3]], [nodes[1]]])
    results = (ctypes.c_float * repeat)()
    unused = (ctypes.c_float * repeat)()
    lib.stage_latency(_c_string(stage_text), _c_string(input_text), ctypes.c_int(1), ctypes.c_int(warmup),
                      ctypes.c_int(number), ctypes.c_int(repeat), ctypes.c_int(0),
                      ctypes.cast(results, ctypes.POINTER(ctypes.c_float)),
                      ctypes.cast(unused, ctypes.POINTER(ctypes.c_float)))
    assert all(0 < float(v) < 100 for v in results)

    # graph_inference (:114-135)
    convs = list(graph.convs())
    names = (ctypes.c_char_p * len(convs))(*[c.name.encode() for c in convs])
    filters = (ctypes.c_void_p * len(convs))(*[c.weight.ctypes.data for c in convs])
    biases = (ctypes.c_void_p * len(convs))(*[c.bias.ctypes.data for c in convs])
    x = oracle.normal_input(config, 1, 0)
    output = np.empty((1, *graph.blocks[-1].exit_node.output_shape), dtype=np.float32)
    lib.graph_inference(_c_string(json.dumps(config)), ctypes.c_int(1), x.ctypes.data_as(ctypes.c_void_p),
                        ctypes.c_int(len(convs)), names, filters, biases, output.ctypes.data_as(ctypes.c_void_p))
    ref = oracle.run_config(config, weights_of(graph), x)
    assert oracle.max_rel_err(output, ref) <= TOL_TF32

    # an error fills the results with NaN and leaves a message; the process lives on
    results = (ctypes.c_float * repeat)()
    lib.graph_latency(_c_string('{"name": '), ctypes.c_int(1), ctypes.c_int(1), ctypes.c_int(1), ctypes.c_int(repeat),
                      ctypes.c_int(0), ctypes.cast(results, ctypes.POINTER(ctypes.c_float)), None)
    assert all(v != v for v in results)


# ---- host-buffer pipeline and engines on several threads ---------------------------------------------
def test_pipelined_run_equals_run_batch_by_batch():
    import torch
    graph = ios.models.squeezenet()
    graph.greedy_schedule()
    config, weights = seeded(graph, 0)
    batch, count = 4, 5
    engine = rt.Engine(graph, batch)
    try:
        xs = [oracle.normal_input(config, batch, 20 + i) for i in range(count)]
        expect = [engine.run(x) for x in xs]
        assert oracle.max_rel_err(expect[0], oracle.run_config(config, weights, xs[0])) <= TOL_TF32
        # pageable numpy buffers
        got = engine.run_pipelined(xs)
        assert all(np.array_equal(a, b) for a, b in zip(got, expect))
        # page-locked buffers, raw addresses, twice in a row (the staging pairs are reused)
        pin_in = [torch.from_numpy(x).pin_memory() for x in xs]
        pin_out = [torch.empty(engine.output_shape, dtype=torch.float32).pin_memory() for _ in xs]
        for _ in range(2):
            for t in pin_out:
                t.fill_(float('nan'))
            engine.run_pipelined([t.data_ptr() for t in pin_in], [t.data_ptr() for t in pin_out])
            assert all(np.array_equal(t.numpy(), b) for t, b in zip(pin_out, expect))
        assert engine.run_pipelined([]) == []
        assert np.array_equal(engine.run_pipelined(xs[:1])[0], expect[0])
        assert np.array_equal(engine.run(xs[2]), expect[2])
    finally:
        engine.close()


def test_two_engines_driven_from_two_threads():
    """Engines own their streams and lock: two of them on one device run concurrently and stay correct."""
    graphs = []
    for model in ('squeezenet', 'inception_v3'):
        graph = getattr(ios.models, model)()
        graph.greedy_schedule()
        config, weights = seeded(graph, 0)
        x = oracle.normal_input(config, 2, 1)
        graphs.append((graph, x, oracle.run_config(config, weights, x)))
    engines = [rt.Engine(g, 2) for g, _, _ in graphs]
    firsts = [e.run(x) for e, (_, x, _) in zip(engines, graphs)]
    errors = []

    def worker(engine, x, first):
        try:
            for _ in range(20):
                if not np.array_equal(engine.run(x), first):
                    errors.append('result changed under concurrency')
        except Exception as err:      # noqa: BLE001 - reported to the main thread
            errors.append(repr(err))

    threads = [threading.Thread(target=worker, args=(e, x, f)) for e, (_, x, _), f in zip(engines, graphs, firsts)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for e in engines:
        e.close()
    assert not errors, errors
    for first, (_, _, ref) in zip(firsts, graphs):
        assert oracle.max_rel_err(first, ref) <= TOL_TF32


def test_an_engine_does_not_move_the_callers_device():
    graph = sample_block()
    graph.sequential_schedule()
    rt.set_device(0)
    engine = rt.Engine(graph, 1)
    try:
        assert engine.describe()['device'] == 0
        engine.time(2)
        lat = rt.graph_latency(graph, 1, 1, 1, 2)      # still device 0, through the shared context
        assert len(lat) == 2 and all(v > 0 for v in lat)
    finally:
        engine.close()


def test_engine_artefact_round_trip(tmp_path):
    """save -> load rebuilds the engine from packed parameters alone and computes the same bits."""
    opt, config = _seeded_dp_graph('squeezenet')
    x = oracle.normal_input(config, 3, 2)
    for precision in ('tf32x3', 'bf16'):
        rt.set_option('precision', precision)
        engine = rt.Engine(opt, 3)
        path = str(tmp_path / f'squeezenet_{precision}.iosengine')
        try:
            expect = engine.run(x)
            engine.save(path)
        finally:
            engine.close()
        rt.set_option('precision', 'fp32')            # the artefact carries its own options: the current ones do not matter
        loaded = rt.Engine.load(path)
        try:
            assert loaded.input_shape == (3, 3, 224, 224) and loaded.output_shape == (3, 1000, 1, 1)
            assert loaded.describe()['precision'] == precision
            assert np.array_equal(loaded.run(x), expect)
            assert loaded.time(3) > 0
        finally:
            loaded.close()
        # a cut-off file is recognised, not misread
        with open(path, 'rb') as fh:
            data = fh.read()
        with open(path, 'wb') as fh:
            fh.write(data[:len(data) // 2])
        with pytest.raises(RuntimeError, match='truncated|damaged'):
            rt.Engine.load(path)
