"""
Cost models that guide the schedule search (reference ``python/ios/cost_model.py``).

``IOSCostModel`` measures on the GPU through ``libios_runtime.so``; ``RandomCostModel`` returns
random numbers, which lets the search run with no GPU (tests, random schedule generation).
"""
from typing import List

import numpy as np

from ios.ir import Graph, Block, Node
from ios.contrib.ios_runtime import graph_latency, stage_latency, block_latency


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
    """Measure by executing on the GPU (reference ``cost_model.py:36-49``)."""

    def get_graph_latency(self, graph, batch_size, warmup, number, repeat, profile_stage=False):
        return graph_latency(graph, batch_size, warmup, number, repeat, profile_stage)

    def get_block_latency(self, block, batch_size, warmup, number, repeat, profile_stage=False):
        return block_latency(block, batch_size, warmup, number, repeat, profile_stage)

    def get_stage_latency(self, stage, batch_size, warmup, number, repeat, profile_stage=False):
        return stage_latency(stage, batch_size, warmup, number, repeat, profile_stage)
