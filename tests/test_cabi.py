"""
The C-ABI library without a GPU: it loads, exports every symbol include/ios_runtime.h declares,
rejects malformed input with status codes, and fails loudly (no CPU path) when no device exists.
"""
import ctypes
import json
import os
import re

import pytest

import ios
from ios.contrib import ios_runtime as rt
from helpers import has_gpu, sample_block

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    with open(os.path.join(ROOT, 'include', 'ios_runtime.h')) as fh:
        text = fh.read()
    return re.findall(r'IOS_API\s+[\w\s\*]+?\b(\w+)\s*\(', text)


def test_library_exports_every_declared_symbol():
    lib = rt.load_ios_library()
    names = declared_symbols()
    assert {'graph_latency', 'block_latency', 'stage_latency', 'graph_inference', 'ios_last_error',
            'ios_engine_create', 'ios_conv2d'} <= set(names)
    for name in names:
        assert hasattr(lib, name), f'{name} is declared in include/ios_runtime.h but not exported'


def _latency_call(lib, text, batch=1, repeat=2):
    results = (ctypes.c_float * repeat)()
    stage = (ctypes.c_float * 64)()
    status = lib.ios_graph_latency(text, batch, 1, 1, repeat, 0, results, stage)
    return status, list(results), lib.ios_last_error().decode()


def test_malformed_json_is_reported_not_fatal():
    lib = rt.load_ios_library()
    status, results, message = _latency_call(lib, b'{"name": "x", ')
    assert status == 1 and 'JSON' in message
    assert all(r != r for r in results)          # NaN-filled


def test_structural_errors_are_reported():
    lib = rt.load_ios_library()
    graph = sample_block()
    graph.sequential_schedule()
    config = graph.export_config()

    def status_of(cfg, batch=1):
        return _latency_call(lib, json.dumps(cfg).encode(), batch)

    bad = json.loads(json.dumps(config))
    bad['blocks'][0]['inner_nodes'][0]['type'] = 'fft'
    status, _, message = status_of(bad)
    assert status == 2 and 'fft' in message

    bad = json.loads(json.dumps(config))
    bad['blocks'][0]['stages'][0][0][0] = 'nope'
    status, _, message = status_of(bad)
    assert status == 2 and 'nope' in message

    bad = json.loads(json.dumps(config))
    bad['blocks'][0]['stages'] = [[['4']], [['1']], [['2']], [['3']], [['5']]]     # consumer before producer
    status, _, message = status_of(bad)
    assert status == 2 and 'producer' in message

    bad = json.loads(json.dumps(config))
    bad['blocks'][0]['inner_nodes'][1]['inputs'] = [[['0', 0, 9999]]]
    status, _, message = status_of(bad)
    assert status == 2 and 'channels' in message

    bad = json.loads(json.dumps(config))
    bad['blocks'][0]['stages'] = None
    assert status_of(bad)[0] == 2

    assert status_of(config, batch=0)[0] == 2
    wide = json.loads(json.dumps(config))
    wide['blocks'][0]['stages'] = [[['1']] * 70]
    status, _, message = status_of(wide)
    assert status in (2, 6)


def test_python_wrapper_raises_runtime_error():
    graph = sample_block()          # no schedule yet: stages is None
    with pytest.raises(RuntimeError):
        rt.graph_latency(graph, batch_size=1, repeat=1)


def test_options_round_trip():
    rt.set_option('precision', 'fp32')
    assert rt.get_option('precision') == 'fp32'
    rt.set_option('precision', 'tf32')
    assert rt.get_option('executor') == 'graph'
    with pytest.raises(RuntimeError):
        rt.set_option('precision', 'int3')


def test_no_device_means_loud_failure():
    if has_gpu():
        pytest.skip('a CUDA device is present')
    graph = sample_block()
    graph.sequential_schedule()
    with pytest.raises(RuntimeError, match='CUDA|device'):
        rt.graph_latency(graph, batch_size=1, repeat=1)
    with pytest.raises(RuntimeError):
        rt.Engine(graph, 1)


def test_stage_config_lists_outside_producers():
    graph = sample_block()
    nodes = graph.blocks[0].inner_nodes
    stage_text, input_text = rt.stage_config([[nodes[0], nodes[3]], [nodes[1]]])
    stage = json.loads(stage_text)
    assert [[n['name'] for n in group] for group in stage] == [['1', '4'], ['2']]
    assert json.loads(input_text) == {'0': [375, 15, 15]}


def test_engine_artefact_files_are_validated(tmp_path):
    with pytest.raises(RuntimeError, match='cannot open'):
        rt.Engine.load(str(tmp_path / 'missing.iosengine'))
    junk = tmp_path / 'junk.iosengine'
    junk.write_bytes(b'not an engine artefact at all' * 10)
    with pytest.raises(RuntimeError, match='not an engine artefact'):
        rt.Engine.load(str(junk))
