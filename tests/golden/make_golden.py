"""
Regenerates the golden fixtures of this folder by running the REFERENCE implementation.

Needs the reference checkout (``--ref``); it is imported, never copied.  For each
case the reference's own package builds the graph, the oracle's seeded generators provide weights
and input (so that the tests can rebuild exactly the same arrays), and the reference's CPU executor
``ios.torch_utils.Net`` (python/ios/torch_utils.py:61-125) produces the output that is stored.

    python tests/golden/make_golden.py [--ref <reference checkout>]

Outputs: golden.npz (output vectors), manifest.json (graph hashes, seeds, shapes) and
ref_schedules/*.json.gz (the reference's seven stored Inception-v3 schedules,
experiments/specialization/schedules/*.json, re-serialised).
"""
import argparse
import gzip
import hashlib
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, 'oracle'))
import ios_oracle as oracle  # noqa: E402


def sha(config):
    return hashlib.sha256(json.dumps(config).encode()).hexdigest()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--ref', default=os.environ.get('IOS_REFERENCE', os.path.join(os.path.dirname(ROOT), 'reference')),
                    help='the reference checkout (default: $IOS_REFERENCE, else a folder named reference beside this repository)')
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(args.ref, 'python', 'ios')):
        raise SystemExit(f'no reference checkout at {args.ref}: pass --ref or set IOS_REFERENCE')
    sys.modules.setdefault('pydot', types.ModuleType('pydot'))   # the visualizer imports it; nothing here draws
    sys.path.insert(0, os.path.join(args.ref, 'python'))
    import ios                                   # the reference package
    from ios import torch_utils
    from ios.models import common, randwire as ref_randwire

    def set_weights(graph, weights):
        def walk(nodes):
            for node in nodes:
                if isinstance(node, ios.ir.Conv):
                    node.weight, node.bias = weights[node.name]
                elif isinstance(node, ios.ir.Sequential):
                    walk(node.nodes)
        walk(graph.nodes())

    def ref_forward(graph, weights, x):
        set_weights(graph, weights)
        net = torch_utils.Net(graph)
        net.write_weights_to_torch()
        net.eval()
        with torch.no_grad():
            return net(torch.from_numpy(x)).numpy()

    arrays, manifest = {}, {}

    def record(case, graph, wseed, xseed, batch=1, law='he', subsample=1):
        config = graph.export_config()
        weights = (oracle.he_normal_weights if law == 'he' else oracle.uniform_weights)(config, wseed)
        x = oracle.normal_input(config, batch, xseed)
        y = ref_forward(graph, weights, x)
        flat = y.reshape(-1)
        arrays[case] = flat[::subsample].astype(np.float32)
        manifest[case] = {'config_sha256': sha(config), 'weight_seed': wseed, 'input_seed': xseed, 'batch': batch,
                          'weight_law': law, 'output_shape': list(y.shape), 'subsample': subsample,
                          'sum': float(flat.astype(np.float64).sum()), 'abs_sum': float(np.abs(flat.astype(np.float64)).sum())}
        print(case, y.shape, manifest[case]['abs_sum'])
        return config

    # -- README sample block (examples/sample.py) --------------------------------------------
    def sample_block():
        common.reset_name()
        v = ios.placeholder(output_shape=(375, 15, 15))
        block = ios.Block(enter_node=v.node)
        v1 = ios.conv2d(block, inputs=[[v]], out_channels=375, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
        v2 = ios.conv2d(block, inputs=[[v]], out_channels=750, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
        v3 = ios.conv2d(block, inputs=[[v]], out_channels=375, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
        v1 = ios.conv2d(block, inputs=[[v1]], out_channels=750, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
        ios.identity(block, inputs=[[v1], [v2], [v3]], is_exit=True)
        return ios.Graph(name="demo", input=v.node, blocks=[block])

    g = sample_block()
    g.sequential_schedule()
    record('sample_block', g, 0, 0, subsample=7)

    g = ios.models.inception_v3()
    g.sequential_schedule()
    record('inception_v3', g, 0, 0)
    record('inception_v3_uniform_b2', g, 1, 1, batch=2, law='uniform')

    g = ios.models.squeezenet()
    g.sequential_schedule()
    record('squeezenet', g, 0, 0)

    # RandWire small regime from the reference's own pieces, on this repository's seeded WS edge lists
    ws_dir = os.path.join(ROOT, 'inter-operator-scheduler_b200', 'ios', 'models', 'randwire_graphs', 'generated')
    common.reset_name()
    pv = ios.placeholder(output_shape=(3, 224, 224))
    v, b0 = ref_randwire.randwire_small_front(pv, 78)
    blocks = [b0]
    for mult, fname in zip((1, 2, 4), ('ws-32-4-0.75-s0.txt', 'ws-32-4-0.75-s1.txt', 'ws-32-4-0.75-s2.txt')):
        v, b = ref_randwire.randwire_stage(v, mult * 78, os.path.join(ws_dir, fname))
        blocks.append(b)
    v, b = ref_randwire.randwire_tail(v)
    blocks.append(b)
    g = ios.Graph('randwire_small', pv.node, blocks)
    g.sequential_schedule()
    record('randwire_small', g, 0, 0)

    # -- the rest of the reference's model zoo: residual adds (element nodes), a block searched in parts --
    from ios.models import nasnet as ref_nasnet, resnet as ref_resnet
    # (resnet50 is exported and hashed only: the reference builds its bottleneck with a last convolution of
    #  `channels` outputs that is added to a shortcut of 4 x `channels`, which its own executor rejects)
    for case, maker in (('resnet18', ref_resnet.resnet18), ('resnet34', ref_resnet.resnet34),
                        ('nasnet_large', ref_nasnet.nasnet_large)):
        g = maker()
        g.sequential_schedule()
        record(case, g, 0, 0)
        block = g.blocks[0]
        if block.parts is not None:
            manifest[case]['parts'] = [[node.name for node in part] for part in block.parts]
    for case, maker in (('resnet50', ref_resnet.resnet50), ('vgg_16', ios.models.vgg_16), ('alexnet', ios.models.alexnet)):
        manifest[case + '_config'] = {'config_sha256': sha(maker().export_config())}

    # -- a small graph that touches every operator type ---------------------------------------
    common.reset_name()
    pv = ios.placeholder(output_shape=(10, 13, 11))
    blk = ios.Block(enter_node=pv.node)
    a = ios.conv2d(blk, [[pv]], out_channels=12, kernel=(3, 3), stride=(1, 1), padding=(1, 1), act='relu')
    b = ios.conv2d(blk, [[pv]], out_channels=12, kernel=(1, 5), stride=(1, 1), padding=(0, 2), act='tanh')
    c = ios.pool2d(blk, [[a, b]], pool_type='avg', kernel=(3, 3), stride=(1, 1), padding=(1, 1))
    d = ios.pool2d(blk, [[a], [b]], pool_type='max', kernel=(3, 3), stride=(1, 1), padding=(1, 1))
    e = common.addition(blk, [[a, b]])
    f = common.multiply(blk, [[a, b]])
    s = common.sigmoid(blk, [[e]])
    r = ios.relu(blk, [[f, c]])
    sep = common.sep_conv(blk, [[r]], out_channels=9, kernel=(3, 3), stride=(2, 2), padding=(1, 1))
    rsep = common.relu_sep_conv(blk, [[s, r]], out_channels=7, kernel=(3, 3), stride=(2, 2), padding=(1, 1))
    grp = ios.conv2d(blk, [[ios.ir.Value(d.node, 2, 22)]], out_channels=6, kernel=(3, 3), stride=(2, 2), padding=(1, 1),
                     groups=2, act='tanh')
    ios.identity(blk, [[sep], [rsep], [grp]], is_exit=True)
    blk2 = ios.Block(enter_node=blk.exit_node)
    top = ios.ir.Value(blk.exit_node, 0, 22)
    g1 = ios.pool2d(blk2, [[top]], pool_type='global_avg')
    g2 = ios.pool2d(blk2, [[top]], pool_type='max', kernel=(2, 2), stride=(2, 2))
    g3 = ios.pool2d(blk2, [[g2]], pool_type='global_avg')
    ios.identity(blk2, [[g1, g3]], is_exit=True)
    g = ios.Graph('all_ops', pv.node, [blk, blk2])
    g.sequential_schedule()
    cfg = record('all_ops_b3', g, 3, 4, batch=3, law='uniform')
    with open(os.path.join(HERE, 'all_ops.json'), 'w') as fh:
        json.dump(cfg, fh)

    # -- the reference optimizer under a seeded random cost model ---------------------------
    for name, maker, opt_type in (('squeezenet', ios.models.squeezenet, 'dp_parallel_merge'),
                                  ('inception_v3', ios.models.inception_v3, 'dp_parallel_merge'),
                                  ('inception_v3', ios.models.inception_v3, 'dp_parallel')):
        g = maker()
        base_cfg = g.export_config()
        weights = oracle.he_normal_weights(base_cfg, 0)
        set_weights(g, weights)
        np.random.seed(7)
        opt = ios.optimize(g, batch_size=1, cost_model=ios.RandomCostModel(), opt_type=opt_type, compute_weight=True,
                           max_part_size=50)
        cfg = opt.export_config()
        x = oracle.normal_input(cfg, 1, 0)
        net = torch_utils.Net(opt)
        net.write_weights_to_torch()
        with torch.no_grad():
            y = net(torch.from_numpy(x)).numpy()
        case = f'{name}_{opt_type}_seed7'
        arrays[case] = y.reshape(-1).astype(np.float32)
        manifest[case] = {'config_sha256': sha(cfg), 'np_random_seed': 7, 'max_part_size': 50,
                          'weight_seed': 0, 'input_seed': 0, 'output_shape': list(y.shape),
                          'num_stages': sum(len(b.stages) for b in opt.blocks)}
        print(case, manifest[case]['num_stages'])

    # -- the reference's stored schedules ----------------------------------------------------
    sched_dir = os.path.join(args.ref, 'experiments', 'specialization', 'schedules')
    os.makedirs(os.path.join(HERE, 'ref_schedules'), exist_ok=True)
    for fname in sorted(os.listdir(sched_dir)):
        with open(os.path.join(sched_dir, fname)) as fh:
            cfg = json.load(fh)
        with gzip.GzipFile(os.path.join(HERE, 'ref_schedules', fname + '.gz'), 'wb', mtime=0) as fh:
            fh.write(json.dumps(cfg, separators=(',', ':')).encode())
        graph = ios.Graph.from_config(cfg)
        cfg2 = graph.export_config()
        weights = oracle.he_normal_weights(cfg2, 0)
        x = oracle.normal_input(cfg2, 1, 0)
        y = ref_forward(graph, weights, x)
        case = 'ref_schedule_' + os.path.splitext(fname)[0]
        arrays[case] = y.reshape(-1).astype(np.float32)
        manifest[case] = {'file': 'ref_schedules/' + fname + '.gz', 'weight_seed': 0, 'input_seed': 0,
                          'output_shape': list(y.shape), 'num_stages': sum(len(b.stages) for b in graph.blocks)}
        print(case, manifest[case]['num_stages'])

    np.savez_compressed(os.path.join(HERE, 'golden.npz'), **arrays)
    with open(os.path.join(HERE, 'manifest.json'), 'w') as fh:
        json.dump(manifest, fh, indent=1, sort_keys=True)


if __name__ == '__main__':
    main()
