"""Stand-ins for the GPU runtime inside worker processes (CPU tests of the worker pool)."""
import hashlib
import os
import time


def fake_latency(stage_json, input_json, batch):
    """
    Deterministic pseudo-latency in (0.01, 1.01) ms derived from the stage's STRUCTURE (operator names do not matter,
    as on a real device: the farm measures structurally equal stages once).
    """
    from ios.contrib.ios_runtime import canonical_stage_key
    return fake_latency_of_structure(canonical_stage_key(stage_json, input_json), batch)


def fake_latency_of_structure(canonical, batch):
    digest = hashlib.sha256((canonical + str(batch)).encode()).digest()
    return 0.01 + int.from_bytes(digest[:4], 'little') / 2 ** 32


class FakeBackend:
    def __init__(self, device):
        self.device = device

    def stage_latency(self, stage_json, input_json, batch, warmup, number, repeat):
        return [fake_latency(stage_json, input_json, batch)] * repeat

    def echo(self, value):
        return (self.device, value)


class DiesOnDeviceOne(FakeBackend):
    """Worker 1 exits abruptly on its first task: the host must move the task elsewhere."""

    def echo(self, value):
        if self.device == 1:
            os._exit(17)
        return (self.device, value)


class HangsOnDeviceOne(FakeBackend):
    """Worker 1 never answers: the host-side time limit must drop it and re-queue the task."""

    def echo(self, value):
        if self.device == 1:
            time.sleep(3600)
        return (self.device, value)


class AlwaysDies(FakeBackend):
    def echo(self, value):
        os._exit(3)


class FailsToStart:
    def __init__(self, device):
        raise RuntimeError('no such device')


class FakeEngineBackend(FakeBackend):
    """
    CPU stand-in for the sharded-inference calls: the "network" maps an image (C, H, W) to its
    per-channel sums times (1 + index of the image inside the whole batch is NOT used: every image is
    treated alike, as the real operators do).  The shared-memory plumbing is the real one.
    """
    fail_first_run_on = None        # device whose first engine_run_shared raises

    def __init__(self, device):
        super().__init__(device)
        self.engines, self.shared, self.runs = {}, {}, 0

    def engine_create(self, key, graph_json, batch, weights):
        import json
        channels = json.loads(graph_json)['input']['output_shape'][0]
        self.engines[key] = (batch, channels)
        return (batch, channels, 1, 1)

    def engine_attach(self, key, in_name, out_name, in_shape, out_shape, begin, end):
        import numpy as np
        from multiprocessing import shared_memory
        shm_in = shared_memory.SharedMemory(name=in_name)
        shm_out = shared_memory.SharedMemory(name=out_name)
        x = np.ndarray(in_shape, dtype=np.float32, buffer=shm_in.buf)[begin:end]
        y = np.ndarray(out_shape, dtype=np.float32, buffer=shm_out.buf)[begin:end]
        self.shared[key] = (shm_in, shm_out, x, y)
        return False                                  # nothing was page-locked

    def engine_run_shared(self, key, repeats=1):
        self.runs += 1
        if self.fail_first_run_on == self.device and self.runs == 1:
            raise RuntimeError('injected failure of the first run')
        _, _, x, y = self.shared[key]
        y[...] = x.sum(axis=(2, 3), keepdims=True)
        return True

    def engine_detach(self, key):
        shm_in, shm_out, x, y = self.shared.pop(key)
        del x, y
        shm_in.close()
        shm_out.close()
        return True


class FakeEngineFailsOnceOnDeviceZero(FakeEngineBackend):
    fail_first_run_on = 0


class SlowOnDeviceOne(FakeBackend):
    """Device 1 reports every stage twice as slow: the farm's calibration must take the factor out again."""

    def stage_latency(self, stage_json, input_json, batch, warmup, number, repeat):
        base = fake_latency(stage_json, input_json, batch)
        return [base * (2.0 if self.device == 1 else 1.0)] * repeat
