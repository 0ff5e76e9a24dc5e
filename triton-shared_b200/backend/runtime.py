"""ctypes binding of libtsb200.so, the C-ABI library declared in include/tsb200.h.

The library is the only execution engine of this package: if it cannot be
loaded, every launch fails loudly (there is no CPU or eager fallback).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_PKG, "libtsb200.so")

TSB_MAX_RANK = 3
TSB_MAX_ACCESSES = 24
TSB_MAX_OPS = 96
TSB_NUM_REGS = 16
TSB_MAX_LOOPS = 4
REG_ACC, REG_IMM = -1, -2  # operand forms of tsb_elementwise (TSB_REG_ACC, TSB_REG_IMM)
MEM_INDEX, MEM_MASK = 1, 2  # flags in the imm field of load / store ops: per-lane index / mask operand

DTYPES = {"f32": 0, "f16": 1, "bf16": 2, "i32": 3, "i16": 4, "i8": 5, "i1": 6, "i64": 7, "f64": 8,
          "u32": 9, "u16": 10, "u8": 11}
DTYPE_SIZE = {"f32": 4, "f16": 2, "bf16": 2, "i32": 4, "i16": 2, "i8": 1, "i1": 1, "i64": 8, "f64": 8,
              "u32": 4, "u16": 2, "u8": 1}

OPCODES = {
    "load": 0, "store": 1, "const": 2, "mov": 4,
    "addf": 10, "subf": 11, "mulf": 12, "divf": 13, "maxnumf": 14, "minnumf": 15, "maximumf": 16,
    "minimumf": 17, "remf": 18,
    "exp": 30, "exp2": 31, "log": 32, "log2": 33, "sqrt": 34, "rsqrt": 35, "sin": 36, "cos": 37,
    "tanh": 38, "erf": 39, "absf": 40, "negf": 41, "floor": 42, "ceil": 43,
    "addi": 50, "subi": 51, "muli": 52, "divsi": 53, "remsi": 54, "divui": 55, "remui": 56,
    "minsi": 57, "maxsi": 58, "minui": 59, "maxui": 60, "andi": 61, "ori": 62, "xori": 63,
    "shli": 64, "shrsi": 65, "shrui": 66, "absi": 67,
    "cmpf": 80, "cmpi": 81, "select": 82, "cast": 90, "bitcast": 91, "fma": 92, "reduce": 100, "loop_begin": 101, "loop_end": 102, "argreduce": 103, "scan": 104,
}
CMPF = {"oeq": 1, "ogt": 2, "oge": 3, "olt": 4, "ole": 5, "one": 6, "ord": 7, "ueq": 8, "ugt": 9,
        "uge": 10, "ult": 11, "ule": 12, "une": 13, "uno": 14}
CMPI = {"eq": 32, "ne": 33, "slt": 34, "sle": 35, "sgt": 36, "sge": 37, "ult": 38, "ule": 39,
        "ugt": 40, "uge": 41}


class Wrap(ctypes.Structure):
    """struct tsb_wrap"""
    _fields_ = [
        ("dim", ctypes.c_int32),
        ("pad_", ctypes.c_int32),
        ("offset0", ctypes.c_int64),
        ("offset_pid", ctypes.c_int64 * 3),
        ("stride", ctypes.c_int64),
        ("modulus", ctypes.c_int64),
        ("scale", ctypes.c_int64),
    ]


class Access(ctypes.Structure):
    """struct tsb_access"""
    _fields_ = [
        ("base", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("is_store", ctypes.c_int32),
        ("has_other", ctypes.c_int32),
        ("offset0", ctypes.c_int64),
        ("offset_pid", ctypes.c_int64 * 3),
        ("sizes", ctypes.c_int64 * TSB_MAX_RANK),
        ("strides", ctypes.c_int64 * TSB_MAX_RANK),
        ("masked", ctypes.c_int32 * TSB_MAX_RANK),
        ("pad_", ctypes.c_int32),
        ("mask_start0", ctypes.c_int64 * TSB_MAX_RANK),
        ("mask_start_pid", (ctypes.c_int64 * 3) * TSB_MAX_RANK),
        ("mask_bound", ctypes.c_int64 * TSB_MAX_RANK),
        ("other_bits", ctypes.c_uint64),
        ("n_wrap", ctypes.c_int32),
        ("pad2_", ctypes.c_int32),
        ("wrap", Wrap * 2),
        ("offset_loop", ctypes.c_int64 * 4),
        ("mask_start_loop", (ctypes.c_int64 * 4) * TSB_MAX_RANK),
    ]


class Op(ctypes.Structure):
    """struct tsb_op"""
    _fields_ = [
        ("opcode", ctypes.c_int32),
        ("type", ctypes.c_int32),
        ("dst", ctypes.c_int32),
        ("a", ctypes.c_int32),
        ("b", ctypes.c_int32),
        ("c", ctypes.c_int32),
        ("imm", ctypes.c_uint32),
        ("imm2", ctypes.c_uint32),
    ]


class Scalar(ctypes.Structure):
    """struct tsb_scalar"""
    _fields_ = [("kind", ctypes.c_int32), ("pad_", ctypes.c_int32), ("i", ctypes.c_int64), ("f", ctypes.c_double)]


class TsbError(RuntimeError):
    pass


_lib = None

# every symbol include/tsb200.h declares
SYMBOLS = ["tsb_last_error", "tsb_version", "tsb_sm_count", "tsb_elementwise", "tsb_block_program", "tsb_block_copy",
           "tsb_softmax_rows", "tsb_layernorm_fwd", "tsb_reduce_rows_scratch_bytes", "tsb_reduce_rows",
           "tsb_reduce_rows_static", "tsb_reduce_all", "tsb_gemm", "tsb_gemm_paired", "tsb_plan_create",
           "tsb_plan_destroy", "tsb_plan_family", "tsb_plan_kernel_name", "tsb_launch_scratch_bytes", "tsb_launch"]


def lib():
    """Load libtsb200.so (once). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TsbError(f"{LIB_PATH} is missing: build it with `python {os.path.join(_PKG, 'build.py')}`; "
                       "this backend has no fallback executor")
    L = ctypes.CDLL(LIB_PATH)
    i32, i64, vp, f32 = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float
    L.tsb_last_error.restype = ctypes.c_char_p
    L.tsb_last_error.argtypes = []
    L.tsb_version.restype = ctypes.c_int
    L.tsb_sm_count.restype = ctypes.c_int
    L.tsb_elementwise.restype = ctypes.c_int
    L.tsb_elementwise.argtypes = [ctypes.POINTER(Access), ctypes.c_int, ctypes.POINTER(Op), ctypes.c_int,
                                  ctypes.POINTER(i32), i64, i64, vp]
    L.tsb_block_program.restype = ctypes.c_int
    L.tsb_block_program.argtypes = [ctypes.POINTER(Access), ctypes.c_int, ctypes.POINTER(Op), ctypes.c_int,
                                    ctypes.POINTER(i32), ctypes.c_int, ctypes.POINTER(i32), i64, i64, vp]
    L.tsb_block_copy.restype = ctypes.c_int
    L.tsb_block_copy.argtypes = [ctypes.POINTER(Access), ctypes.POINTER(Access), ctypes.POINTER(i32), i64, i64, vp]
    L.tsb_softmax_rows.restype = ctypes.c_int
    L.tsb_softmax_rows.argtypes = [vp, vp, i32, i64, i64, i64, i64, i64, i64, vp]
    L.tsb_layernorm_fwd.restype = ctypes.c_int
    L.tsb_layernorm_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i32, i64, i64, i64, f32, i64, i64, vp]
    L.tsb_reduce_rows_scratch_bytes.restype = i64
    L.tsb_reduce_rows_scratch_bytes.argtypes = [i64, i64, i64, i64]
    L.tsb_reduce_rows.restype = ctypes.c_int
    L.tsb_reduce_rows.argtypes = [vp, vp, i64, i64, i64, i64, i64, i64, vp, vp]
    L.tsb_reduce_rows_static.restype = ctypes.c_int
    L.tsb_reduce_rows_static.argtypes = [vp, vp, i64, i64, i64, i64, i64, i64, vp]
    L.tsb_reduce_all.restype = ctypes.c_int
    L.tsb_reduce_all.argtypes = [vp, vp, i64, i64, vp]
    L.tsb_gemm.restype = ctypes.c_int
    L.tsb_gemm.argtypes = [vp, vp, vp, i32] + [i64] * 9 + [i32, i32, i32, vp, i64, i64, i64, vp, vp]
    L.tsb_gemm_paired.restype = ctypes.c_int
    L.tsb_gemm_paired.argtypes = [vp, vp, vp, i32] + [i64] * 9 + [i32, i32, i32, vp, i64, vp, vp]
    L.tsb_plan_create.restype = vp
    L.tsb_plan_create.argtypes = [ctypes.c_char_p, i64]
    L.tsb_plan_destroy.restype = None
    L.tsb_plan_destroy.argtypes = [vp]
    L.tsb_plan_family.restype = ctypes.c_char_p
    L.tsb_plan_family.argtypes = [vp]
    L.tsb_plan_kernel_name.restype = ctypes.c_char_p
    L.tsb_plan_kernel_name.argtypes = [vp]
    L.tsb_launch_scratch_bytes.restype = i64
    L.tsb_launch_scratch_bytes.argtypes = [vp, ctypes.POINTER(i32), i64, i64, ctypes.POINTER(Scalar), ctypes.c_int]
    L.tsb_launch.restype = ctypes.c_int
    L.tsb_launch.argtypes = [vp, ctypes.POINTER(i32), i64, i64, vp, ctypes.POINTER(vp), ctypes.POINTER(Scalar), ctypes.c_int,
                             vp, i64, vp]
    _lib = L
    return L


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().tsb_last_error().decode("utf-8", "replace")
        raise TsbError(f"{what} failed ({rc}): {msg}")
