"""
Seeded Watts-Strogatz edge-list generator for the RandWire stage graphs.

Writes the text format the RandWire model reader expects: node count, edge count, then one
``u v`` line per undirected edge with ``u < v`` (the model orients every edge from the lower to the
higher index, which makes the graph a DAG).  The construction is the published WS procedure: a ring
lattice where every node is joined to its k/2 neighbours on each side, then each clockwise edge is
rewired with probability p to a uniformly chosen node that is not yet a neighbour.

    python ws.py -n 32 -k 4 -p 0.75 -s 0 -o generated/ws-32-4-0.75-s0.txt
"""
import argparse
import os

import numpy as np


def watts_strogatz_edges(n: int, k: int, p: float, seed: int):
    if k % 2 or not 0 < k < n:
        raise ValueError('k must be even and 0 < k < n')
    rng = np.random.default_rng(seed)
    linked = np.eye(n, dtype=bool)
    for i in range(n):
        for step in range(1, k // 2 + 1):
            j = (i + step) % n
            linked[i, j] = linked[j, i] = True
    for i in range(n):
        for step in range(1, k // 2 + 1):
            if rng.random() >= p:
                continue
            free = np.flatnonzero(~linked[i])
            if free.size == 0:
                continue
            old, new = (i + step) % n, int(rng.choice(free))
            linked[i, old] = linked[old, i] = False
            linked[i, new] = linked[new, i] = True
    return [(i, j) for i in range(n) for j in range(i + 1, n) if linked[i, j]]


def write_edges(path, n, edges):
    with open(path, 'w') as f:
        f.write(f'{n}\n{len(edges)}\n')
        for u, v in edges:
            f.write(f'{u} {v}\n')


if __name__ == '__main__':
    ap = argparse.ArgumentParser(description='Watts-Strogatz graph generator')
    ap.add_argument('-n', '--n_nodes', type=int, default=32)
    ap.add_argument('-k', '--k_neighbors', type=int, required=True)
    ap.add_argument('-p', '--prob', type=float, required=True)
    ap.add_argument('-s', '--seed', type=int, default=0)
    ap.add_argument('-o', '--out_txt', type=str, required=True)
    a = ap.parse_args()
    os.makedirs(os.path.dirname(os.path.abspath(a.out_txt)), exist_ok=True)
    write_edges(a.out_txt, a.n_nodes, watts_strogatz_edges(a.n_nodes, a.k_neighbors, a.prob, a.seed))
