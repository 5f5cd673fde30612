"""Stand-ins for the GPU runtime inside worker processes (CPU tests of the worker pool)."""
import hashlib
import os
import time


def fake_latency(stage_json, input_json, batch):
    """Deterministic pseudo-latency in (0.01, 1.01) ms derived from the task's text."""
    digest = hashlib.sha256((stage_json + input_json + str(batch)).encode()).digest()
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
