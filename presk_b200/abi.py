"""ctypes mirror of include/presk_cuda.h: the structs, enums and prototypes.

Nothing here computes. The layouts must match the header field for field;
tests/test_abi.py checks sizes and that every declared symbol is exported.
"""
import ctypes as C
import os

MAX_RANK = 8
MAX_INNER = 4
MAX_AXES = MAX_RANK + MAX_INNER
MAX_INPUTS = 8
MAX_STEPS = 64

# psk_dtype
F64, F32, BF16, I64, F16, E8M15, I8, E4M3, U8 = range(9)
DTYPE_NAMES = {F64: "f64", F32: "f32", BF16: "bf16", I64: "i64", F16: "f16", E8M15: "e8m15", I8: "int8", E4M3: "e4m3fn", U8: "uint8"}
DTYPE_BYTES = {F64: 8, F32: 4, BF16: 2, I64: 8, F16: 2, E8M15: 3, I8: 1, E4M3: 1, U8: 1}

# psk_status
OK, E7001, E7005, E7006, E7007, E10001 = 0, 7001, 7005, 7006, 7007, 10001

# psk_op
OP_FUSED, OP_CONTRACT, OP_REDUCE, OP_SOFTMAX, OP_XENT, OP_ARGMAX, OP_EMBED, OP_COPY, OP_IOTA, OP_CONVERT, OP_MAGNITUDE, OP_ATTENTION, OP_RMSNORM, OP_ROPE, OP_CONTRACT_ADD, OP_XENT_VJP, OP_EMBED_VJP = range(17)

# psk_prim
(ADD, SUB, MUL, DIV, MAX, MIN, NEG, EXP, LOG, TANH, SQRT, SIN, COS, ABS, GELU, GELU_DERIV, RELU, HEAVISIDE, SIGN, SIGMOID, POW, REAL, DIV_N, ROUND) = range(24)

ORDER_SEQUENTIAL, ORDER_DEVICE, ORDER_CHUNKED = 0, 1, 2
REDUCE_SUM, REDUCE_MEAN, REDUCE_SUMSQ, REDUCE_SUM_STORED = 0, 1, 2, 3
COMM_U32 = 100
COMM_SUM, COMM_MAX, COMM_MIN = 0, 1, 2
COMM_ID_BYTES = 128
IOTA_POSITIONS, IOTA_CAUSAL, IOTA_ONE_HOT, IOTA_FILL = 0, 1, 2, 3


class Step(C.Structure):
    _fields_ = [("prim", C.c_int32), ("nargs", C.c_int32), ("src", C.c_int32 * 2), ("imm", C.c_int32)]


class Operand(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("is_index", C.c_int32), ("offset", C.c_int64),
        ("stride", C.c_int64 * MAX_AXES), ("scale_stride", C.c_int64 * MAX_AXES), ("numel", C.c_int64),
        ("affine", C.c_int32), ("affine_zero", C.c_int32), ("affine_scale", C.c_float), ("reserved", C.c_int32),
    ]


class Launch(C.Structure):
    _fields_ = [
        ("name", C.c_char_p), ("op", C.c_int32), ("dtype", C.c_int32), ("order", C.c_int32), ("guarded", C.c_int32),
        ("n_inputs", C.c_int32), ("n_outer", C.c_int32), ("n_inner", C.c_int32),
        ("dims", C.c_int64 * MAX_AXES), ("inputs", Operand * MAX_INPUTS), ("out", Operand),
        ("n_steps", C.c_int32), ("steps", Step * MAX_STEPS),
        ("kind", C.c_int32), ("masked", C.c_int32), ("int_accum", C.c_int32), ("order_size", C.c_int32), ("iparam", C.c_int64 * 4), ("fparam", C.c_double * 2),
    ]


class Gemm(C.Structure):
    _fields_ = [
        ("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("b_n_major", C.c_int32), ("guarded", C.c_int32),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64), ("batch", C.c_int64), ("batch_lo", C.c_int64),
        ("a_row", C.c_int64), ("a_lo", C.c_int64), ("a_hi", C.c_int64),
        ("b_row", C.c_int64), ("b_lo", C.c_int64), ("b_hi", C.c_int64),
        ("c_row_lo_count", C.c_int64), ("c_row_lo", C.c_int64), ("c_row_hi", C.c_int64),
        ("c_col_lo_count", C.c_int64), ("c_col_hi", C.c_int64), ("c_lo", C.c_int64), ("c_hi", C.c_int64),
        ("scale", C.c_float), ("scale_on", C.c_int32),
    ]


class Value(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("dims", C.c_int64 * MAX_RANK)]


class ExecVtable(C.Structure):
    _fields_ = [
        ("self", C.c_void_p),
        ("name", C.c_void_p), ("alloc", C.c_void_p), ("free", C.c_void_p), ("upload", C.c_void_p), ("download", C.c_void_p),
        ("run", C.c_void_p), ("sync", C.c_void_p), ("overflow", C.c_void_p), ("last_error", C.c_void_p),
        ("quantize", C.c_void_p), ("init_normal", C.c_void_p),
    ]


# name -> (restype, argtypes): every function include/presk_cuda.h declares
class DataLeaf(C.Structure):
    """psk_data_leaf: a leaf of a .psk.d sample type (`bound` > 0: idx[bound] elements; `n` elements)."""
    _fields_ = [("bound", C.c_uint64), ("n", C.c_uint64)]


PROTOTYPES = {
    "psk_abi_sizeof": (C.c_size_t, [C.c_int]),
    "psk_exec_create": (C.c_void_p, [C.c_int]),
    "psk_exec_destroy": (None, [C.c_void_p]),
    "psk_exec_name": (C.c_char_p, [C.c_void_p]),
    "psk_last_error": (C.c_char_p, [C.c_void_p]),
    "psk_exec_alloc": (C.c_void_p, [C.c_void_p, C.c_size_t]),
    "psk_exec_free": (None, [C.c_void_p, C.c_void_p]),
    "psk_exec_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "psk_exec_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "psk_exec_sync": (C.c_int, [C.c_void_p]),
    "psk_exec_memory": (None, [C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "psk_exec_run": (C.c_int, [C.c_void_p, C.POINTER(Launch), C.POINTER(C.c_void_p)]),
    "psk_exec_overflow": (C.c_int64, [C.c_void_p]),
    "psk_exec_counts": (None, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "psk_exec_set_profiling": (None, [C.c_void_p, C.c_int]),
    "psk_exec_last_ms": (C.c_double, [C.c_void_p]),
    "psk_exec_stream": (C.c_void_p, [C.c_void_p]),
    "psk_exec_profile": (C.c_char_p, [C.c_void_p]),
    "psk_exec_gemm": (C.c_int, [C.c_void_p, C.POINTER(Gemm), C.c_void_p, C.c_void_p, C.c_void_p]),
    "psk_gemm_noalloc": (C.c_int, [C.POINTER(Gemm), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.c_char_p, C.c_size_t]),
    "psk_exec_quantize": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]),
    "psk_exec_init_normal": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_double]),
    "psk_exec_as_vtable": (None, [C.c_void_p, C.POINTER(ExecVtable)]),
    "psk_host_create": (C.c_void_p, [C.POINTER(ExecVtable), C.c_char_p]),
    "psk_host_destroy": (None, [C.c_void_p]),
    "psk_host_error": (C.c_char_p, [C.c_void_p]),
    "psk_host_prepare": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p]),
    "psk_host_set_param": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int32, C.POINTER(C.c_int64), C.c_int32]),
    "psk_host_init_param": (C.c_int, [C.c_void_p, C.c_char_p, C.c_uint64, C.c_double, C.POINTER(C.c_int64), C.c_int32]),
    "psk_host_call": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(Value), C.c_int32, C.c_void_p, C.c_int32, C.c_int64, C.POINTER(C.c_int64)]),
    "psk_exec_wait_selftest": (C.c_int, [C.c_void_p, C.c_int64]),
    "psk_comm_unique_id": (C.c_int, [C.c_void_p]),
    "psk_comm_create": (C.c_void_p, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "psk_comm_destroy": (None, [C.c_void_p]),
    "psk_comm_error": (C.c_char_p, [C.c_void_p]),
    "psk_comm_rank": (C.c_int32, [C.c_void_p]),
    "psk_comm_size": (C.c_int32, [C.c_void_p]),
    "psk_comm_allreduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32]),
    "psk_host_mean_over_ranks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(C.c_double)]),
    "psk_host_envelope_allreduce": (C.c_int, [C.c_void_p, C.c_void_p]),
    "psk_host_grads_allreduce": (C.c_int, [C.c_void_p, C.c_void_p]),
    "psk_host_result": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int32, C.c_int64, C.POINTER(C.c_int64)]),
    "psk_host_set_result": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int32, C.POINTER(C.c_int64), C.c_int32]),
    "psk_host_adamw": (C.c_int, [C.c_void_p, C.c_char_p]),
    "psk_host_adamw_step": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64]),
    "psk_host_adamw_lr": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.POINTER(C.c_double)]),
    "psk_host_call_device": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(Value), C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "psk_host_set_calibrating": (None, [C.c_void_p, C.c_int]),
    "psk_host_envelope": (C.c_char_p, [C.c_void_p]),
    "psk_host_launches": (C.c_int64, [C.c_void_p]),
    "psk_host_launch_log": (C.c_char_p, [C.c_void_p]),
    "psk_host_set_logging": (None, [C.c_void_p, C.c_int]),
    "psk_exec_gap": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int64, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "psk_describe": (C.c_int, [C.c_char_p, C.c_int32, C.POINTER(Launch), C.c_char_p, C.c_size_t, C.POINTER(C.c_char_p), C.c_char_p, C.c_size_t]),
    "psk_data_open": (C.c_int, [C.c_char_p, C.c_char_p, C.POINTER(DataLeaf), C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p, C.c_size_t]),
    "psk_data_count": (C.c_uint64, [C.c_void_p]),
    "psk_data_sample_bytes": (C.c_uint64, [C.c_void_p]),
    "psk_data_read": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(C.c_void_p), C.POINTER(C.c_int32)]),
    "psk_data_error": (C.c_char_p, [C.c_void_p]),
    "psk_data_close": (None, [C.c_void_p]),
}


def bind(lib, names=None):
    """Sets restype/argtypes on `lib` for the declared functions."""
    for name, (res, args) in PROTOTYPES.items():
        if names is not None and name not in names:
            continue
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


def library_path():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib", "libpresk_cuda.so")


def load():
    """Loads libpresk_cuda.so. Raises if it is not built: there is no other path."""
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is not built; run `python -m presk_b200.build` (needs nvcc)")
    return bind(C.CDLL(path))
