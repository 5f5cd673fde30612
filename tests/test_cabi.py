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


def _reference_checkout():
    path = os.environ.get('IOS_REFERENCE', os.path.join(os.path.dirname(ROOT), 'reference'))
    return path if os.path.isdir(os.path.join(path, 'python', 'ios')) else None


@pytest.mark.skipif(_reference_checkout() is None, reason='no reference checkout on this machine')
def test_reference_front_end_drives_this_library(tmp_path):
    """
    Route 1 of the integration notes: the reference's own Python package, unmodified, bound to this
    libios_runtime.so.  Its loader looks for the library relative to its own file, so the test hands it
    the search list instead of copying anything.  Without a GPU the call comes back with NaN latencies
    and a message that names the missing device -- proof that the symbol was found and that the graph
    JSON crossed the boundary intact (a marshalling fault would report a JSON error, and the reference's
    own runtime would have ended the interpreter); with a GPU it returns real latencies.
    """
    import subprocess
    import sys
    script = tmp_path / 'route1.py'
    script.write_text(f'''
import sys, types, math
import torch                                      # before the stub: torch probes pydot too
sys.modules.setdefault("pydot", types.ModuleType("pydot"))
sys.path.insert(0, {os.path.join(_reference_checkout(), "python")!r})
import ios
from ios.contrib import ios_runtime
ios_runtime.libname_list = [{rt.load_ios_library()._name!r}]
v = ios.placeholder(output_shape=(375, 15, 15))
block = ios.Block(enter_node=v.node)
v1 = ios.conv2d(block, inputs=[[v]], out_channels=375, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act="relu")
v2 = ios.conv2d(block, inputs=[[v]], out_channels=750, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act="relu")
out = ios.identity(block, inputs=[[v1], [v2]], is_exit=True)
graph = ios.Graph(name="demo", input=v.node, blocks=[block])
graph.init_weights()
graph.sequential_schedule()
lat = ios.ios_runtime.graph_latency(graph, batch_size=1, repeat=3)
print("LATENCY", " ".join("nan" if math.isnan(x) else "ok" if x > 0 else "bad" for x in lat))
''')
    done = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    line = [text for text in done.stdout.splitlines() if text.startswith('LATENCY')][0]
    if has_gpu():
        assert line == 'LATENCY ok ok ok'
    else:
        assert line == 'LATENCY nan nan nan'
        assert 'no CUDA device' in done.stderr or 'device' in done.stderr
