"""B200-native execution backend for triton-shared's lowered kernels.

    import triton, triton_shared_b200
    triton.runtime.driver.set_active(triton_shared_b200.B200Driver())

registers the backend with Triton and makes every subsequent ``kernel[grid](...)``
run on hand-written sm_100a CUDA kernels through the C-ABI library libtsb200.so.
"""
from triton.backends import Backend, backends

from .backend.compiler import BACKEND_NAME, B200Backend, B200Options, compile_ttir_text
from .backend.driver import B200Driver, B200Launcher, B200Utils, DevicePtr, partition_range
from .backend.ttir import UnsupportedTTIR
from .backend import runtime

# Triton discovers backends through entry points; an out-of-tree backend registers itself here.
if BACKEND_NAME not in backends:
    backends[BACKEND_NAME] = Backend(compiler=B200Backend, driver=B200Driver)


def activate(**kwargs) -> B200Driver:
    """Make the B200 driver the active Triton driver and return it."""
    import triton
    drv = B200Driver(**kwargs)
    triton.runtime.driver.set_active(drv)
    return drv


__all__ = ["B200Driver", "B200Backend", "B200Options", "B200Launcher", "B200Utils", "UnsupportedTTIR",
           "activate", "DevicePtr", "compile_ttir_text", "partition_range", "runtime", "BACKEND_NAME"]
