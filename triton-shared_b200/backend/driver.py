"""Triton driver plugin for the B200 execution library.

Counterpart of the reference's ``backend/driver.py``: ``B200Driver`` has the
method set of ``CPUDriver`` (lines 420-464 there), ``B200Utils`` that of
``CPUUtils`` (380-417) and ``B200Launcher`` the call signature of ``CPULauncher``
(361-376, 262-265).  Where the reference compiles a C++ launcher per kernel and
runs the grid as a serial host loop (116-133), this launcher evaluates the
kernel's launch plan for the call's arguments and enqueues CUDA kernels of
libtsb200.so on the current stream.  Launches are asynchronous.

Activation is the same one-line swap as for the reference
(``python/examples/conftest.py:7``):

    import triton, triton_shared_b200
    triton.runtime.driver.set_active(triton_shared_b200.B200Driver())

Multi-GPU: ``B200Driver(program_range=(lo, hi))`` or the context manager
``driver.partition(rank, world)`` restricts every launch to a contiguous range
of the linearised grid; num_programs stays the full grid.
"""
import contextlib
import sys

import numpy as np

from triton.backends.compiler import GPUTarget
from triton.backends.driver import DriverBase

from . import plan as _plan
from . import runtime as rt
from .compiler import BACKEND_NAME


def _ty_to_cpp(ty):
    """Same table as the reference (backend/driver.py:41-64)."""
    if ty[0] == '*':
        return "void*"
    if ty == "constexpr":
        return "PyObject*"
    return {
        "i1": "int32_t", "i8": "int8_t", "i16": "int16_t", "i32": "int32_t", "i64": "int64_t",
        "u1": "uint32_t", "u8": "uint8_t", "u16": "uint16_t", "u32": "uint32_t", "u64": "uint64_t",
        "fp32": "float", "f32": "float", "fp64": "double",
    }[ty]


def partition_range(n_programs: int, rank: int, world: int):
    """Contiguous share of the linearised grid owned by `rank` of `world` (balanced to within one program)."""
    base, rem = divmod(n_programs, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class DevicePtr:
    """A raw device address that Triton treats as a pointer argument of element type `dtype`
    (a torch dtype).  Lets a caller hand a kernel a pointer to *virtual* element 0 of an
    array of which only a shard is resident on this GPU (multi-GPU program ranges)."""

    def __init__(self, address: int, dtype):
        self.address = int(address)
        self.dtype = dtype

    def data_ptr(self) -> int:
        return self.address


class TorchDeviceMemory:
    """Device memory the kernels need beyond inputs and outputs, owned by the host side
    (the C library never allocates).  One instance per process; state is kept per device.

    Scratch is one grow-only buffer per (device, stream): launches on different streams never share
    partial sums, and a buffer that is replaced by a larger one is handed back to torch's caching
    allocator only after the work already queued on its stream (``record_stream``).  Uploaded tile
    tables are keyed by content and are evicted oldest first, after a device synchronisation, so a
    table is never released under a launch that still reads it."""

    MAX_TABLES = 256

    def __init__(self):
        self._state = {}

    def _dev(self):
        import torch
        d = torch.cuda.current_device()
        st = self._state.get(d)
        if st is None:
            st = self._state[d] = {"scratch": {}, "tables": {}, "status": None}
        return st

    def scratch(self, nbytes: int, stream: int = 0) -> int:
        import torch
        st = self._dev()
        buf = st["scratch"].get(stream)
        if buf is None or buf.numel() < nbytes:
            if buf is not None:
                buf.record_stream(torch.cuda.ExternalStream(stream) if stream else torch.cuda.default_stream())
            buf = st["scratch"][stream] = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device="cuda")
        return buf.data_ptr()

    def table(self, key, host: np.ndarray, stream: int = 0) -> int:
        import torch
        st = self._dev()
        t = st["tables"].get(key)
        if t is None:
            if len(st["tables"]) >= self.MAX_TABLES:
                torch.cuda.synchronize()  # nothing in flight reads the tables that go
                for old in list(st["tables"])[: self.MAX_TABLES // 2]:
                    del st["tables"][old]
            t = torch.from_numpy(np.ascontiguousarray(host)).to("cuda")
            st["tables"][key] = t
        return t.data_ptr()

    def status(self) -> int:
        import torch
        st = self._dev()
        if st["status"] is None:
            st["status"] = torch.zeros(4, dtype=torch.int32, device="cuda")
        return st["status"].data_ptr()

    def read_status(self):
        st = self._dev()
        return None if st["status"] is None else st["status"].cpu().tolist()

    def clear_status(self):
        st = self._dev()
        if st["status"] is not None:
            st["status"].zero_()


class LaunchArgs:
    """What a plan needs from one launch: scalars, floats, pointers, device scratch."""

    def __init__(self, memory, values):
        self.scalars, self.floats, self._ptrs = {}, {}, {}
        self._mem = memory
        self.n_args = len(values)
        for k, (ty, v) in enumerate(values):
            if ty[0] == '*':
                self._ptrs[k] = v
            elif ty in ("fp32", "f32", "fp64"):
                self.floats[k] = float(v)
            else:
                self.scalars[k] = int(v)

    def pointer(self, k: int) -> int:
        """Device address of pointer argument k: int, None (null) or an object with data_ptr()
        (the reference's getPointer, backend/driver.py:140-171)."""
        v = self._ptrs[k]
        if v is None:
            return 0
        if isinstance(v, int):
            return v
        dp = getattr(v, "data_ptr", None)
        if dp is None:
            raise TypeError("Pointer argument must be either uint64 or have data_ptr method")
        # a host tensor handed to a GPU launch would fault the device: the launcher stages such
        # tensors through device memory (HostStaging); one that reaches this point unstaged is refused
        if getattr(v, "is_cuda", True) is False and not getattr(self._mem, "host_pointers", False):
            raise ValueError("Pointer argument (at %d) cannot be accessed from the GPU: it is a host tensor" % k)
        p = dp()
        if not isinstance(p, int):
            raise TypeError("data_ptr method of Pointer object must return 64-bit int")
        return p

    def pointer_positions(self):
        return self._ptrs.keys()

    def scratch(self, nbytes: int, stream) -> int:
        return self._mem.scratch(nbytes, int(stream or 0))

    def device_table(self, key, host: np.ndarray, stream) -> int:
        return self._mem.table(key, host, int(stream or 0))

    def status_word(self, stream) -> int:
        return self._mem.status()


class HostStaging:
    """Host (CPU) torch tensors among a launch's pointer arguments, staged through device memory.

    Programs written for the reference keep their tensors on the CPU.  For each such argument the
    whole underlying storage is copied to a device buffer before the launch (so every offset and
    stride the kernel was given stays valid), the kernel gets the device address of the tensor's
    first element, and after the launch the storage is copied back.  The launch is synchronous for
    these calls.  Tensors that share a storage share one device copy."""

    def __init__(self):
        self.copies = {}  # storage address -> (host bytes view, device bytes tensor)

    def device_address(self, t):
        import torch
        st = t.untyped_storage()
        key = st.data_ptr()
        if key not in self.copies:
            host = torch.empty(0, dtype=torch.uint8).set_(st)
            self.copies[key] = (host, host.to("cuda"))
        return self.copies[key][1].data_ptr() + (t.data_ptr() - key)

    def finish(self):
        import torch
        if self.copies:
            torch.cuda.synchronize()
            for host, dev in self.copies.values():
                host.copy_(dev)


class _Staged:
    """A pointer argument replaced by its staged device address."""

    def __init__(self, address):
        self._a = address

    def data_ptr(self):
        return self._a


class B200Launcher(object):
    memory = TorchDeviceMemory()  # provider of scratch/tables/status words (replaceable in tests)

    def __init__(self, src, metadata):
        constants = src.constants if hasattr(src, "constants") else dict()
        arg_names = src.fn.arg_names if hasattr(src, "fn") else list(src.signature.keys())
        cst_key = lambda i: arg_names.index(i) if isinstance(i, str) else i
        self.constants = {cst_key(key): value for key, value in constants.items()}
        self.signature = {cst_key(key): value for key, value in src.signature.items()}
        self.order = sorted(self.signature.keys())

    def __call__(self, gridX, gridY, gridZ, stream, function, kernel_metadata, launch_metadata,
                 launch_enter_hook, launch_exit_hook, *args):
        plan = function
        if not isinstance(plan, _plan.Plan):
            raise rt.TsbError("launch without a launch plan: the kernel was not compiled by the B200 backend")
        if launch_enter_hook is not None:
            launch_enter_hook(launch_metadata)
        values = []
        staging = None
        host_ok = getattr(B200Launcher.memory, "host_pointers", False)
        for idx in self.order:
            ty = self.signature[idx]
            if ty == "constexpr":
                continue
            v = args[idx]
            if ty[0] == '*' and not host_ok and getattr(v, "is_cuda", True) is False and hasattr(v, "untyped_storage"):
                staging = staging or HostStaging()
                v = _Staged(staging.device_address(v))
            values.append((ty, v))
        grid = (int(gridX), int(gridY), int(gridZ))
        total = grid[0] * grid[1] * grid[2]
        if total > 0:
            drv = B200Driver.current
            lo, hi = (0, total) if drv is None else drv.range_for(total)
            if hi > lo:
                largs = LaunchArgs(B200Launcher.memory, values)
                if not plan.launch_native(largs, grid, lo, hi, stream or 0):
                    plan.launch(largs, grid, lo, hi, stream or 0)
        if staging is not None:
            staging.finish()
        if launch_exit_hook is not None:
            launch_exit_hook(launch_metadata)


class B200Utils(object):

    def __new__(cls):
        if not hasattr(cls, "instance"):
            cls.instance = super(B200Utils, cls).__new__(cls)
        return cls.instance

    @staticmethod
    def get_device_properties(device):
        import torch
        if not torch.cuda.is_available():
            return {"max_shared_mem": 232448, "multiprocessor_count": 148, "sm_clock_rate": None,
                    "mem_clock_rate": None, "mem_bus_width": None}
        pr = torch.cuda.get_device_properties(device)
        return {"max_shared_mem": 232448, "multiprocessor_count": pr.multi_processor_count,
                "sm_clock_rate": None, "mem_clock_rate": None, "mem_bus_width": None}

    @staticmethod
    def load_binary(name, kernel_obj, shared, device):
        # same tuple as the reference (backend/driver.py:410-417); `function` is the parsed plan
        rt.lib()  # fail now, loudly, if the CUDA library has not been built
        plan = _plan.plan_from_bytes(kernel_obj)
        # `module` must not be None: Triton re-initialises the kernel handles on every launch
        # while it is (compiler.py `_init_handles`), which would re-parse the plan each time
        return (plan, plan, None, None, sys.maxsize)


class B200Driver(DriverBase):
    current = None  # the driver whose program range launches honour

    def __init__(self, program_range=None):
        super().__init__()
        self.utils = B200Utils()
        self.launcher_cls = B200Launcher
        self.binary_ext = "plan"
        self._range = program_range  # None | (lo, hi) | ("part", rank, world)
        self._cuda = None
        B200Driver.current = self

    # never auto-selected; only through triton.runtime.driver.set_active (reference: driver.py:428-432)
    @staticmethod
    def is_active():
        return False

    def range_for(self, total: int):
        r = self._range
        if r is None:
            return 0, total
        if r[0] == "part":
            return partition_range(total, r[1], r[2])
        return max(0, r[0]), min(total, r[1])

    @contextlib.contextmanager
    def partition(self, rank: int, world: int):
        """Launches inside the block run only rank's contiguous share of each grid."""
        old = self._range
        self._range = ("part", rank, world)
        try:
            yield self
        finally:
            self._range = old

    @contextlib.contextmanager
    def program_range(self, lo: int, hi: int):
        """Launches inside the block run only programs [lo, hi) of each (linearised) grid, e.g. to
        pipeline one large launch as chunks behind their host-to-device copies."""
        old = self._range
        self._range = (int(lo), int(hi))
        try:
            yield self
        finally:
            self._range = old

    def check(self):
        """Raise if a device-side bounded wait of an earlier launch gave up.

        The tcgen05 matmul kernels wait on mbarriers with a time limit; a wait that expires records
        (code, role, tile, k step) in a per-device status word and the kernel returns, leaving its
        output invalid.  Launches are asynchronous, so the launcher cannot see this: call check()
        after the work has been synchronised (it synchronises the device itself) wherever a silent
        failure is not acceptable.  The word is cleared by the call."""
        import torch
        mem = B200Launcher.memory
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        st = mem.read_status()
        if st and st[0] != 0:
            mem.clear_status()
            raise rt.TsbError(f"a device-side wait timed out (code {st[0]}: role {st[1]}, tile {st[2]}, k step {st[3]}); "
                              "the output of that matmul launch is invalid")

    def get_benchmarker(self):
        from triton.testing import do_bench
        return do_bench

    def get_device_capability(self, device=None):
        return (10, 0)

    def _has_cuda(self):
        if self._cuda is None:
            import torch
            self._cuda = bool(torch.cuda.is_available())
            if self._cuda:
                from torch._C import _cuda_getCurrentRawStream
                self._raw_stream = _cuda_getCurrentRawStream
                self._cur_dev = torch.cuda.current_device
        return self._cuda

    def get_current_stream(self, device=None):
        if not self._has_cuda():
            return 0
        return self._raw_stream(self._cur_dev() if device is None else device)

    def get_current_device(self):
        return self._cur_dev() if self._has_cuda() else 0

    def set_current_device(self, device):
        import torch
        if torch.cuda.is_available():
            torch.cuda.set_device(device)

    def get_current_target(self):
        # only B200Backend.supports_target accepts this name: neither Triton's own CUDA
        # code generator nor any CPU path can be selected for kernels launched through this driver
        return GPUTarget(BACKEND_NAME, 100, 32)

    def get_active_torch_device(self):
        import torch
        return torch.device("cuda", self.get_current_device())

    def get_device_interface(self):
        import torch
        return torch.cuda

    def get_empty_cache_for_benchmark(self):
        import torch
        return torch.empty(int(256 * 1024 * 1024 // 4), dtype=torch.int, device="cuda")

    def clear_cache(self, cache):
        cache.zero_()

    def assemble_tensormap_to_arg(self, tensormaps_info, args):
        return args

    def map_python_to_cpp_type(self, ty: str) -> str:
        return _ty_to_cpp(ty)
