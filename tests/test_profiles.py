"""
The traffic table beside the profile summaries is what bench.py reads for `roofline.traffic`: it must parse,
name the capture it came from, and belong to the kernel sources of this tree (bench.py reports no traffic otherwise).
"""
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location('bench_for_test', os.path.join(ROOT, 'bench.py'))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_traffic_table_belongs_to_these_kernel_sources():
    with open(os.path.join(ROOT, 'profiles', 'conv_tc_traffic.json')) as fh:
        table = json.load(fh)
    entry = table['inception_v3/batch1/tf32x3']
    assert entry['dram_bytes_per_forward'] == entry['dram_bytes_read'] + entry['dram_bytes_write'] > 0
    assert entry['launches'] == 94 and entry['schedule'] == 'sequential'
    assert 'ncu ' in entry['command'] and '--clock-control none' in entry['command'] and 'bench.py' in entry['command']
    assert os.path.exists(os.path.join(ROOT, entry['summary']))
    assert entry['sources_sha16'] == _bench().kernel_sources_sha16(), \
        'the convolution kernels changed after the traffic capture: capture again (command in the table)'


def test_profile_summaries_name_their_commands():
    folder = os.path.join(ROOT, 'profiles')
    summaries = [f for f in os.listdir(folder) if f.endswith('.md')]
    assert summaries
    for name in summaries:
        with open(os.path.join(folder, name)) as fh:
            text = fh.read()
        assert 'ncu ' in text and '--clock-control none' in text, name
        assert '_work/' not in text, name
