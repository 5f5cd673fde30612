"""
Cost models that guide the schedule search (reference ``python/ios/cost_model.py``).

``IOSCostModel`` measures on the GPU through ``libios_runtime.so``; ``RandomCostModel`` returns
random numbers, which lets the search run with no GPU (tests, random schedule generation).
"""
from typing import List

import numpy as np

from ios.ir import Graph, Block, Node
from ios.contrib.ios_runtime import (graph_latency, stage_latency, block_latency, stage_config, canonical_stage_key,
                                     get_option)


class CostModel:
    def get_stage_latency(self, stage: List[List[Node]], batch_size, warmup, number, repeat,
                          profile_stage=False) -> List[float]:
        raise NotImplementedError

    def get_block_latency(self, block: Block, batch_size, warmup, number, repeat, profile_stage=False) -> List[float]:
        raise NotImplementedError

    def get_graph_latency(self, graph: Graph, batch_size, warmup, number, repeat, profile_stage=False) -> List[float]:
        raise NotImplementedError


class RandomCostModel(CostModel):
    """``repeat`` draws of ``np.random.rand()`` per query (reference ``cost_model.py:22-33``)."""

    @staticmethod
    def _draw(repeat):
        return [float(np.random.rand()) for _ in range(repeat)]

    def get_graph_latency(self, graph, batch_size, warmup, number, repeat, profile_stage=False):
        return self._draw(repeat)

    def get_block_latency(self, block, batch_size, warmup, number, repeat, profile_stage=False):
        return self._draw(repeat)

    def get_stage_latency(self, stage, batch_size, warmup, number, repeat, profile_stage=False):
        return self._draw(repeat)


class IOSCostModel(CostModel):
    """
    Measure by executing on the GPU (reference ``cost_model.py:36-49``).  With ``dedup`` (default) a
    candidate stage whose structure was measured before -- the same operators under other names, as the
    repeated blocks of a network produce them -- is answered from a memo instead of being timed again.
    """

    def __init__(self, dedup=True):
        self.dedup = dedup
        self.memo = {}
        self.measured = 0

    def get_graph_latency(self, graph, batch_size, warmup, number, repeat, profile_stage=False):
        return graph_latency(graph, batch_size, warmup, number, repeat, profile_stage)

    def get_block_latency(self, block, batch_size, warmup, number, repeat, profile_stage=False):
        return block_latency(block, batch_size, warmup, number, repeat, profile_stage)

    def get_stage_latency(self, stage, batch_size, warmup, number, repeat, profile_stage=False):
        if not self.dedup or profile_stage:
            self.measured += 1
            return stage_latency(stage, batch_size, warmup, number, repeat, profile_stage)
        key = (canonical_stage_key(*stage_config(stage)), int(batch_size), warmup, number, repeat,
               get_option('precision'))
        if key not in self.memo:
            self.measured += 1
            self.memo[key] = stage_latency(stage, batch_size, warmup, number, repeat)
        return list(self.memo[key])
