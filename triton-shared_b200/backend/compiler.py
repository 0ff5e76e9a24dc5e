"""Triton backend plugin: TTIR -> launch plan for the B200 execution library.

Counterpart of the reference's ``backend/compiler.py`` (``CPUBackend``,
lines 206-275 there).  The reference runs ``ttir -> ttsharedir -> llir -> obj``
through four external tools; here the ``ttir`` stage is the same pass list and a
single ``plan`` stage replaces the rest: it re-derives the structured access
descriptors and op body from the TTIR (see ``structured.py``) and selects a
pre-built sm_100a kernel family (see ``plan.py``).  The "binary" handed to the
driver is the JSON launch plan.  Unsupported TTIR raises at compile time.
"""
import functools
import hashlib
import os
from dataclasses import dataclass
from types import ModuleType
from typing import Any, Dict, Tuple

from triton._C.libtriton import ir, passes
from triton.backends.compiler import BaseBackend, GPUTarget

from . import plan as _plan
from . import structured, ttir

BACKEND_NAME = "triton_shared_b200"


def _dump(name: str, text):
    """TRITON_SHARED_DUMP_PATH: same variable as the reference (backend/compiler.py:30-35)."""
    path = os.getenv("TRITON_SHARED_DUMP_PATH", "")
    if not path:
        return
    os.makedirs(path, exist_ok=True)
    mode = "wb" if isinstance(text, bytes) else "w"
    with open(os.path.join(path, name), mode) as f:
        f.write(text)


def ttir_to_plan(mod, metadata) -> bytes:
    """The `plan` stage: parse, analyse, select a kernel family."""
    text = mod.str_nodebug() if hasattr(mod, "str_nodebug") else str(mod)
    _dump("tt.mlir", text)
    pl, fn = _plan_of(text)
    metadata["name"] = fn.name
    metadata["shared"] = 0
    metadata["family"] = pl.family
    blob = pl.to_bytes()
    _dump("plan.json", blob)
    return blob


def _plan_of(text: str):
    """Parse, analyse, select a family.  Anything the parser or the analysis does not understand is
    reported as UnsupportedTTIR (never as an internal error, and never by falling back)."""
    try:
        fn = ttir.parse_module(text)
        kernel, an = structured.analyze(fn)
    except ttir.UnsupportedTTIR:
        raise
    except (AttributeError, AssertionError, KeyError, IndexError, ValueError, TypeError) as e:
        raise ttir.UnsupportedTTIR(f"TTIR construct outside the structured subset ({type(e).__name__}: {e})") from e
    return _plan.make_plan(kernel, an), fn


def compile_ttir_text(text: str) -> "_plan.Plan":
    """Plan for a TTIR module given as text (used by tests and tools)."""
    return _plan_of(text)[0]


@dataclass(frozen=True)
class B200Options:
    debug: bool = False
    arch: Any = None
    num_warps: int = 4
    num_ctas: int = 1
    num_stages: int = 1
    enable_warp_specialization: bool = False
    enable_fp_fusion: bool = False
    extern_libs: Any = None
    cluster_dims: tuple = (1, 1, 1)
    shared: bool = False
    supported_fp8_dtypes: Tuple[str, ...] = ()
    deprecated_fp8_dot_operand_dtypes: Tuple[str, ...] = ()
    allow_fp8e4nv: bool = False
    allowed_dot_input_precisions: Tuple[str, ...] = ("ieee", )
    default_dot_input_precision: str = "ieee"
    max_num_imprecise_acc_default: int = 0
    sanitize_overflow: bool = True
    launch_cooperative_grid: bool = False
    launch_pdl: bool = False
    backend_name: str = BACKEND_NAME
    instrumentation_mode: str = ""

    def hash(self):
        key = '_'.join([f'{name}-{val}' for name, val in self.__dict__.items()])
        return hashlib.sha256(key.encode("utf-8")).hexdigest()


class B200Backend(BaseBackend):
    binary_ext = 'plan'

    @staticmethod
    def supports_target(target: GPUTarget):
        return target.backend == BACKEND_NAME

    def __init__(self, target: GPUTarget) -> None:
        super().__init__(target)

    def parse_options(self, opts) -> Any:
        args = {'arch': self.target.arch}
        args.update({k: opts[k] for k in B200Options.__dataclass_fields__.keys() if k in opts and opts[k] is not None})
        return B200Options(**args)

    def get_codegen_implementation(self, options):
        return {"min_dot_size": lambda lhsType, rhsType: (1, 1, 1)}

    def pack_metadata(self, metadata):
        # same 7-tuple as the reference (backend/compiler.py:225-237); index 6 is the kernel name
        return (
            metadata.num_warps,
            metadata.num_ctas,
            metadata.shared,
            metadata.cluster_dims[0],
            metadata.cluster_dims[1],
            metadata.cluster_dims[2],
            metadata.name,
        )

    def load_dialects(self, ctx):
        return

    @staticmethod
    def make_ttir(mod, metadata, options):
        # the reference's pass list (backend/compiler.py:244-260)
        pm = ir.pass_manager(mod.context)
        pm.enable_debug()
        passes.common.add_inliner(pm)
        passes.ttir.add_rewrite_tensor_pointer(pm)
        passes.ttir.add_rewrite_tensor_descriptor_to_pointer(pm)
        passes.common.add_canonicalizer(pm)
        passes.ttir.add_combine(pm)
        passes.ttir.add_reorder_broadcast(pm)
        passes.common.add_cse(pm)
        passes.ttir.add_triton_licm(pm)
        passes.common.add_symbol_dce(pm)
        passes.ttir.add_loop_unroll(pm)
        passes.common.add_cse(pm)
        pm.run(mod, 'make_ttir')
        return mod

    def add_stages(self, stages, options, language=None):
        stages["ttir"] = lambda src, metadata: self.make_ttir(src, metadata, options)
        stages["plan"] = lambda src, metadata: ttir_to_plan(src, metadata)

    @functools.lru_cache()
    def hash(self):
        # the plan compiler's sources are part of the cache key
        h = hashlib.sha256(str(self.target).encode())
        here = os.path.dirname(os.path.abspath(__file__))
        for name in ("compiler.py", "plan.py", "structured.py", "ttir.py"):
            with open(os.path.join(here, name), "rb") as f:
                h.update(f.read())
        return h.hexdigest()

    def get_module_map(self) -> Dict[str, ModuleType]:
        return {}
