"""No-op timer with the upstream ``CUDAKernelTimer`` surface (reference:
spconv_triton/tools.py)."""

import contextlib

CPU_ONLY_BUILD = False
nullcontext = contextlib.nullcontext


class CUDAKernelTimer:
    def __init__(self, enable: bool = True):
        self.enable = enable
        self._timer = None

    @contextlib.contextmanager
    def namespace(self, name: str):
        yield

    @contextlib.contextmanager
    def record(self, name: str, stream: int = 0):
        yield

    def get_all_pair_time(self):
        return {}
