"""ctypes binding of libzyxb.so — the C ABI declared in include/zyxb.h.

This is the same stub a maintainer of the reference would write in Rust (`extern "C"` block in
zyx/src/backend/b200.rs); here it is Python so that the parity tests and the bench can drive
the library.  There is no fallback: if the shared library is missing, importing fails loudly.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libzyxb.so")

# ---- enums (include/zyxb.h) ------------------------------------------------------------------
OK = 0
ERR_NAMES = {1: "DyLibNotFound", 2: "Initialization", 3: "Deinitialization", 4: "DeviceEnumeration", 5: "DeviceQuery",
             6: "MemoryAllocation", 7: "MemoryDeallocation", 8: "MemoryCopyH2P", 9: "MemoryCopyP2H", 10: "IncorrectKernelArg",
             11: "KernelCompilation", 12: "KernelLaunch", 13: "KernelSync"}
COMM_OPT_LATENCY = 1
ERR_NAMES_INV = {name: code for code, name in ERR_NAMES.items()}
BF16, F16, F32, F64, U8, U16, U32, U64, I8, I16, I32, I64, BOOL = range(13)
DTYPE_SIZE = {BF16: 2, F16: 2, F32: 4, F64: 8, U8: 1, U16: 2, U32: 4, U64: 8, I8: 1, I16: 2, I32: 4, I64: 8, BOOL: 1}
KIND_ROWREDUCE, KIND_GEMM, KIND_ELTWISE, KIND_OPTIM, KIND_ATTENTION, KIND_ATTENTION_BWD, KIND_CONV, KIND_CONV_WGRAD, KIND_CONV_DGRAD = 1, 2, 3, 4, 5, 6, 7, 8, 9
(RR_SUM, RR_MAX, RR_MIN, RR_MEAN, RR_VAR, RR_STD, RR_SOFTMAX, RR_LN_SOFTMAX, RR_LAYERNORM, RR_CROSS_ENTROPY,
 RR_CROSS_ENTROPY_BWD, RR_SOFTMAX_BWD, RR_LAYERNORM_BWD, RR_COLSUM, RR_MSE, RR_LAYERNORM_DYXHAT) = range(16)
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_BIAS_GELU, EPI_MUL_RELU_GRAD, EPI_MUL_GELU_GRAD, EPI_ADD = range(7)
TRI_NONE, TRI_OUT_LOWER, TRI_A_LOWER, TRI_AT_LOWER = range(4)
(EW_RELU, EW_GELU, EW_ADD, EW_SUB, EW_MUL, EW_SCALE, EW_RELU_BWD, EW_GELU_BWD, EW_MSE_BWD, EW_CAST, EW_TANH, EW_SIGMOID,
 EW_EXP, EW_BIAS_ADD) = range(14)
OPT_SGD, OPT_ADAM, OPT_ADAMW = range(3)


# ---- structs ---------------------------------------------------------------------------------
class Event(C.Structure):
    _fields_ = [("id", C.c_uint64)]


class Config(C.Structure):
    _fields_ = [("n_device_ids", C.c_int32), ("device_ids", C.c_int32 * 16), ("debug", C.c_int32), ("round_nearest", C.c_int32)]


class DevInfo(C.Structure):
    _fields_ = [("compute_flops", C.c_uint64), ("max_global_work_dims", C.c_uint64 * 3), ("max_local_threads", C.c_uint32),
                ("max_local_work_dims", C.c_uint32 * 3), ("preferred_vector_size", C.c_uint32), ("local_mem_size", C.c_uint64),
                ("max_register_bytes", C.c_uint64), ("tensor_cores", C.c_int32), ("warp_size", C.c_uint32),
                ("dtype_capability", C.c_uint32 * 13), ("has_native_exp2", C.c_int32), ("sm_count", C.c_uint32),
                ("total_mem_bytes", C.c_uint64), ("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("name", C.c_char * 128)]


class RowReduceDesc(C.Structure):
    _fields_ = [("op", C.c_int32), ("dtype", C.c_int32), ("rows", C.c_uint64), ("cols", C.c_uint64), ("eps", C.c_float),
                ("correction", C.c_int32), ("has_weight", C.c_int32), ("has_bias", C.c_int32), ("scale", C.c_float),
                ("causal", C.c_int32), ("period", C.c_uint64)]


class GemmDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("m", C.c_uint64), ("n", C.c_uint64), ("k", C.c_uint64), ("batch", C.c_uint64),
                ("trans_a", C.c_int32), ("trans_b", C.c_int32), ("stride_a", C.c_int64), ("stride_b", C.c_int64),
                ("stride_c", C.c_int64), ("epilogue", C.c_int32), ("store_preact", C.c_int32), ("alpha", C.c_float),
                ("lda", C.c_uint64), ("ldb", C.c_uint64), ("ldc", C.c_uint64), ("batch_inner", C.c_uint64),
                ("stride_a_inner", C.c_int64), ("stride_b_inner", C.c_int64), ("stride_c_inner", C.c_int64), ("tri", C.c_int32)]


class EltwiseDesc(C.Structure):
    _fields_ = [("op", C.c_int32), ("dtype", C.c_int32), ("dtype_out", C.c_int32), ("numel", C.c_uint64), ("cols", C.c_uint64),
                ("p0", C.c_float)]


class OptimDesc(C.Structure):
    _fields_ = [("algo", C.c_int32), ("dtype", C.c_int32), ("n_tensors", C.c_int32), ("numel", C.POINTER(C.c_uint64)),
                ("lr", C.c_float), ("weight_decay", C.c_float), ("momentum", C.c_float), ("dampening", C.c_float),
                ("nesterov", C.c_int32), ("maximize", C.c_int32), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("grad_scale", C.c_float), ("standard", C.c_int32)]


class AttentionDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_uint64), ("heads", C.c_uint64), ("seq", C.c_uint64), ("head_dim", C.c_uint64),
                ("ld", C.c_uint64), ("scale", C.c_float), ("causal", C.c_int32)]


class ConvDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("n", C.c_uint64), ("c", C.c_uint64), ("h", C.c_uint64), ("w", C.c_uint64), ("o", C.c_uint64),
                ("kh", C.c_uint64), ("kw", C.c_uint64), ("stride_h", C.c_uint32), ("stride_w", C.c_uint32), ("dil_h", C.c_uint32),
                ("dil_w", C.c_uint32), ("pad_top", C.c_uint32), ("pad_bottom", C.c_uint32), ("pad_left", C.c_uint32),
                ("pad_right", C.c_uint32), ("has_bias", C.c_int32), ("channels_last", C.c_int32), ("flip_filter", C.c_int32)]


class _DescUnion(C.Union):
    _fields_ = [("rowreduce", RowReduceDesc), ("gemm", GemmDesc), ("eltwise", EltwiseDesc), ("optim", OptimDesc),
                ("attention", AttentionDesc), ("conv", ConvDesc)]


class KernelDesc(C.Structure):
    _fields_ = [("kind", C.c_int32), ("u", _DescUnion)]


_EV_P = C.POINTER(Event)
_U32_P = C.POINTER(C.c_uint32)
_CTX = C.c_void_p

# name -> (restype, argtypes): every symbol include/zyxb.h declares
SIGNATURES = {
    "zyxb_init": (C.c_int32, [C.POINTER(Config), C.POINTER(_CTX)]),
    "zyxb_shutdown": (C.c_int32, [_CTX]),
    "zyxb_last_error": (C.c_char_p, [_CTX]),
    "zyxb_device_count": (C.c_int32, [_CTX, C.POINTER(C.c_int32)]),
    "zyxb_device_info": (C.c_int32, [_CTX, C.c_int32, C.POINTER(DevInfo)]),
    "zyxb_free_compute": (C.c_int32, [_CTX, C.c_int32, C.POINTER(C.c_uint64)]),
    "zyxb_free_bytes": (C.c_int32, [_CTX, C.c_int32, C.POINTER(C.c_uint64)]),
    "zyxb_alloc": (C.c_int32, [_CTX, C.c_int32, C.c_uint64, _U32_P, _EV_P]),
    "zyxb_free": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, _EV_P, C.c_int32]),
    "zyxb_h2d": (C.c_int32, [_CTX, C.c_int32, C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint64, _EV_P, C.c_int32, _EV_P]),
    "zyxb_d2h": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.c_uint64, C.c_void_p, C.c_uint64, _EV_P, C.c_int32]),
    "zyxb_d2d": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.c_uint64, C.c_int32, C.c_uint32, C.c_uint64, C.c_uint64, _EV_P,
                             C.c_int32, _EV_P]),
    "zyxb_memset": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.c_uint64, C.c_int32, C.c_uint64]),
    "zyxb_buffer_bytes": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.POINTER(C.c_uint64)]),
    "zyxb_buffer_view": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.c_uint64, C.c_uint64, _U32_P]),
    "zyxb_sync": (C.c_int32, [_CTX, C.c_int32, _EV_P, C.c_int32]),
    "zyxb_release_events": (C.c_int32, [_CTX, C.c_int32, _EV_P, C.c_int32]),
    "zyxb_device_sync": (C.c_int32, [_CTX, C.c_int32]),
    "zyxb_store_variable": (C.c_int32, [_CTX, C.c_int32, C.c_int32, C.c_void_p, _U32_P]),
    "zyxb_get_variable": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.POINTER(C.c_int32), C.c_void_p]),
    "zyxb_host_register": (C.c_int32, [_CTX, C.c_void_p, C.c_uint64]),
    "zyxb_host_unregister": (C.c_int32, [_CTX, C.c_void_p]),
    "zyxb_program_create": (C.c_int32, [_CTX, C.c_int32, C.POINTER(KernelDesc), _U32_P]),
    "zyxb_launch": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, _U32_P, C.c_int32, _EV_P, C.c_int32, _EV_P]),
    "zyxb_program_release": (C.c_int32, [_CTX, C.c_int32, C.c_uint32]),
    "zyxb_program_set_step": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.c_uint64]),
    "zyxb_program_get_step": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.POINTER(C.c_uint64)]),
    "zyxb_capture_begin": (C.c_int32, [_CTX, C.c_int32]),
    "zyxb_capture_end": (C.c_int32, [_CTX, C.c_int32, _U32_P]),
    "zyxb_graph_launch": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, _EV_P, C.c_int32, _EV_P]),
    "zyxb_graph_release": (C.c_int32, [_CTX, C.c_int32, C.c_uint32]),
    "zyxb_colsum_static": (C.c_int32, [_CTX, C.c_int32, C.c_int32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint64]),
    "zyxb_colsum_static_capacity": (C.c_int32, [C.POINTER(C.c_uint64)]),
    "zyxb_launch_count": (C.c_int32, [_CTX, C.c_int32, C.POINTER(C.c_uint64)]),
    "zyxb_device_status": (C.c_int32, [_CTX, C.c_int32, _U32_P]),
    "zyxb_check_guards": (C.c_int32, [_CTX, C.c_int32, _U32_P]),
    "zyxb_selftest_bounded_wait": (C.c_int32, [_CTX, C.c_int32, C.c_uint64, _U32_P]),
    "zyxb_event_record": (C.c_int32, [_CTX, C.c_int32, _EV_P]),
    "zyxb_event_elapsed_ms": (C.c_int32, [_CTX, C.c_int32, Event, Event, C.POINTER(C.c_float)]),
    "zyxb_flush_l2": (C.c_int32, [_CTX, C.c_int32]),
    "zyxb_comm_unique_id": (C.c_int32, [_CTX, C.c_void_p]),
    "zyxb_comm_init": (C.c_int32, [_CTX, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "zyxb_allreduce_sum": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.c_uint64, C.c_uint64, C.c_int32, _EV_P, C.c_int32, _EV_P]),
    "zyxb_reduce_scatter_sum": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.c_uint64, C.c_uint64, C.c_int32, _EV_P, C.c_int32, _EV_P]),
    "zyxb_allgather": (C.c_int32, [_CTX, C.c_int32, C.c_uint32, C.c_uint64, C.c_uint64, C.c_int32, _EV_P, C.c_int32, _EV_P]),
    "zyxb_comm_rank": (C.c_int32, [_CTX, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "zyxb_comm_option": (C.c_int32, [_CTX, C.c_int32, C.c_int32, C.c_int32]),
    "zyxb_comm_destroy": (C.c_int32, [_CTX, C.c_int32]),
}

_lib = None


def load():
    """Load libzyxb.so and attach the prototypes.  Raises if the library has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("zyx_b200: %s is missing — build it with `python -m zyx_b200.build` "
                          "(there is no CPU or PyTorch fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
