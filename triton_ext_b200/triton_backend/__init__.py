"""A Triton backend that runs ``@triton.jit`` K-loop kernels on the library's sm_100a GEMM.

Laid out as Triton expects a backend package (``compiler.py`` + ``driver.py``; triton 3.6.0
backends/__init__.py:57-62), so that a distribution can list it as

    [project.entry-points."triton.backends"]
    b200dot = "triton_ext_b200.triton_backend"

Without an installed entry point, :func:`install` registers it for the running process. Either way the
stock CUDA driver stays Triton's default; :func:`activate` switches a block of code over:

    with triton_backend.activate():
        kernel[grid](a, b, c, M, N, K, ...)     # analysed once, then tx_dot_run on the current stream

A ``JITFunction`` remembers the backend of its first launch on a device, so launch a given kernel object
under one driver only, or decorate it with :func:`jit` instead of ``triton.jit``: that kernel object keeps one
compile cache per driver and can be launched under the stock driver and under this one in turn.

This fills the reference's empty ``backend/`` slot (backend/CMakeLists.txt is empty upstream) from the
Python side; the pass plug-ins it drives are the ones TRITON_PASS_PLUGIN_PATH would load.
"""
from __future__ import annotations

import contextlib

from .ttir import BoundDot, DotKernelMatch, NotCanonical, bind, match_dot_kernel

__all__ = ["install", "activate", "jit", "NotCanonical", "DotKernelMatch", "BoundDot", "bind", "match_dot_kernel"]


def install() -> None:
    """Register the backend in this process (what an installed ``triton.backends`` entry point does)."""
    import triton.backends as tb

    from .compiler import TARGET_NAME, B200DotBackend
    from .driver import B200DotDriver

    if TARGET_NAME not in tb.backends:
        tb.backends[TARGET_NAME] = tb.Backend(compiler=B200DotBackend, driver=B200DotDriver)


@contextlib.contextmanager
def activate():
    """Make the b200dot driver Triton's active driver inside the block; needs an sm_100 device."""
    import os

    from triton.runtime.driver import driver as config

    from .driver import B200DotDriver

    if os.environ.get("TRITON_INTERPRET") == "1":
        raise RuntimeError("TRITON_INTERPRET=1: kernels of this process run in Triton's interpreter, which no backend sees")
    install()
    previous = config._active
    config.set_active(B200DotDriver())
    try:
        yield config.active
    finally:
        config._active = previous


def jit(fn=None, **options):
    """``triton.jit`` for kernels that are launched under more than one driver: the compile cache of the returned
    kernel object (target, backend, binder, compiled kernels per device) is kept per active driver."""
    from collections import defaultdict

    from triton.runtime.driver import driver as config
    from triton.runtime.jit import JITFunction

    class PerDriverJITFunction(JITFunction):
        def run(self, *args, **kwargs):
            caches = self.__dict__.setdefault("_caches_by_driver", {})
            key = type(config.active).__qualname__
            if key not in caches:
                caches[key] = defaultdict(self.create_binder)
            self.device_caches = caches[key]
            return super().run(*args, **kwargs)

    def wrap(f):
        return PerDriverJITFunction(f, **options)

    return wrap(fn) if fn is not None else wrap
