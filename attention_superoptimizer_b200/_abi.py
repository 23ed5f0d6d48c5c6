"""ctypes declarations for include/mugraph.h.  Loading fails loudly when the library has not been
built: there is no fallback implementation."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmugraph.so")

MG_OK = 0
STATUS_NAMES = {0: "MG_OK", 1: "MG_ERR_INVALID_ARGUMENT", 2: "MG_ERR_INVALID_GRAPH", 3: "MG_ERR_OUT_OF_MEMORY",
                4: "MG_ERR_CUDA", 5: "MG_ERR_UNSUPPORTED", 6: "MG_ERR_DEVICE_TIMEOUT", 7: "MG_ERR_NO_DEVICE"}


class mg_tensor(ctypes.Structure):
    _fields_ = [("data_type", ctypes.c_int32), ("layout", ctypes.c_int32), ("num_dims", ctypes.c_int32),
                ("dim", ctypes.c_int32 * 4), ("owner_op", ctypes.c_int32), ("owner_ts_idx", ctypes.c_int32),
                ("data_ptr", ctypes.c_void_p), ("fp_ptr", ctypes.c_void_p)]


class mg_plan(ctypes.Structure):
    _fields_ = [("num_ops", ctypes.c_int32), ("op_types", ctypes.POINTER(ctypes.c_int32)),
                ("op_num_srcs", ctypes.POINTER(ctypes.c_int32)), ("op_srcs", ctypes.POINTER(ctypes.c_int32)),
                ("num_inputs", ctypes.c_int32), ("input_map", ctypes.POINTER(ctypes.c_int32)),
                ("forloop_dim", ctypes.POINTER(ctypes.c_int32)),
                ("input_smem_layouts", ctypes.POINTER(ctypes.c_int32)), ("output_map", ctypes.c_int32 * 3),
                ("forloop_range", ctypes.c_int32), ("reduction_dimx", ctypes.c_int32),
                ("grid_dim", ctypes.c_int32 * 3), ("block_dim", ctypes.c_int32 * 3)]


class mgd_op(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int32), ("a", ctypes.c_int32 * 19)]


class mgd_program(ctypes.Structure):
    _fields_ = [("grid", ctypes.c_int32 * 3), ("threads", ctypes.c_int32), ("forloop_range", ctypes.c_int32),
                ("num_ops", ctypes.c_int32), ("num_inputs", ctypes.c_int32), ("num_outputs", ctypes.c_int32),
                ("smem_bytes", ctypes.c_int32), ("reserved", ctypes.c_int32 * 3), ("ops", mgd_op * 24)]


# every symbol the header declares, with (restype, argtypes); None argtypes = left unchecked
_P = ctypes.c_void_p
_I = ctypes.c_int32
_T = ctypes.POINTER(mg_tensor)
SIGNATURES = {
    "mg_runtime_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(_P)]),
    "mg_runtime_destroy": (ctypes.c_int, [_P]),
    "mg_runtime_tables": (ctypes.c_int, [_P, ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P)]),
    "mg_runtime_arena_usage": (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]),
    "mg_runtime_set_max_smem": (ctypes.c_int, [_P, ctypes.c_size_t]),
    "mg_runtime_set_specialisation": (ctypes.c_int, [_P, ctypes.c_int]),
    "mg_runtime_set_launch_policy": (ctypes.c_int, [_P, ctypes.c_int]),
    "mg_runtime_set_option": (ctypes.c_int, [_P, _I, _I]),
    "mg_runtime_get_option": (ctypes.c_int, [_P, _I, ctypes.POINTER(_I)]),
    "mg_stream_inputs_written": (ctypes.c_int, [_P]),
    "mg_selftest_bounded_wait": (ctypes.c_int, [_P, _I, _P]),
    "mg_graph_create": (ctypes.c_int, [_P, ctypes.POINTER(_P)]),
    "mg_graph_destroy": (ctypes.c_int, [_P]),
    "mg_graph_new_input": (ctypes.c_int, [_P, ctypes.POINTER(_I), _I, _I, _I, _T]),
    "mg_graph_customized": (ctypes.c_int, [_P, _T, _I, ctypes.POINTER(mg_plan), _T, _I, ctypes.POINTER(_I)]),
    "mg_graph_matmul": (ctypes.c_int, [_P, _T, _T, _T]),
    "mg_graph_exp": (ctypes.c_int, [_P, _T, _T]),
    "mg_graph_add": (ctypes.c_int, [_P, _T, _T, _T]),
    "mg_graph_mul": (ctypes.c_int, [_P, _T, _T, _T]),
    "mg_graph_div": (ctypes.c_int, [_P, _T, _T, _T]),
    "mg_graph_reduction": (ctypes.c_int, [_P, _T, _I, _I, _T]),
    "mg_graph_num_operators": (ctypes.c_int, [_P, ctypes.POINTER(_I)]),
    "mg_graph_customized_info": (ctypes.c_int, [_P, _I, ctypes.POINTER(_I), ctypes.POINTER(_I), ctypes.POINTER(_I),
                                                ctypes.POINTER(_I)]),
    "mg_graph_customized_program": (ctypes.c_int, [_P, _I, _P, ctypes.c_size_t]),
    "mg_verify_candidates": (ctypes.c_int, [_P, _T, ctypes.POINTER(_P), _T, _I, ctypes.POINTER(_I), _P]),
    "mg_graph_to_json": (ctypes.c_int, [_P, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)]),
    "mg_graph_from_json": (ctypes.c_int, [_P, ctypes.c_char_p, ctypes.POINTER(_P)]),
    "mg_graph_operator_info": (ctypes.c_int, [_P, _I, ctypes.POINTER(_I), _T, _I, ctypes.POINTER(_I)]),
    "mg_graph_customized_set_causal_window": (ctypes.c_int, [_P, _I, _I]),
    "mg_op_fingerprint": (ctypes.c_int, [_P, _I]),
    "mg_graph_fingerprint": (ctypes.c_int, [_P]),
    "mg_graph_fingerprint_compute": (ctypes.c_int, [_P]),
    "mg_graph_fingerprint_enqueue": (ctypes.c_int, [_P, _P]),
    "mg_op_run": (ctypes.c_int, [_P, _I, _P]),
    "mg_op_profile": (ctypes.c_int, [_P, _I, _I, _I, ctypes.POINTER(ctypes.c_float)]),
    "mg_graph_run": (ctypes.c_int, [_P, _P]),
    "mg_graph_fingerprint_batched": (ctypes.c_int, [_P, _I, ctypes.POINTER(_P), _P, _P,
                                                    ctypes.POINTER(ctypes.c_size_t), _P]),
    "mg_graph_run_batched": (ctypes.c_int, [_P, _I, ctypes.POINTER(_P), _P, _P, ctypes.POINTER(ctypes.c_size_t), _P]),
    "mg_compare_fingerprint_rows": (ctypes.c_int, [_P, _P, _P, ctypes.c_int64, ctypes.c_int64, _P, _P, _P]),
    "mg_tensor_has_same_fingerprint": (ctypes.c_int, [_P, _T, _T, ctypes.POINTER(_I)]),
    "mg_tensor_fill_fingerprint_reference": (ctypes.c_int, [_P, _T]),
    "mg_tensor_fill_fingerprint_seeded": (ctypes.c_int, [_P, _T, ctypes.c_uint64, ctypes.c_uint32]),
    "mg_tensor_fill_data_seeded": (ctypes.c_int, [_P, _T, ctypes.c_uint64, ctypes.c_float]),
    "mg_tensor_upload_fingerprint": (ctypes.c_int, [_P, _T, _P]),
    "mg_tensor_download_fingerprint": (ctypes.c_int, [_P, _T, _P]),
    "mg_tensor_upload_data": (ctypes.c_int, [_P, _T, _P]),
    "mg_tensor_download_data": (ctypes.c_int, [_P, _T, _P]),
    "mg_tensor_upload_data_async": (ctypes.c_int, [_P, _T, _P, _P]),
    "mg_tensor_download_data_async": (ctypes.c_int, [_P, _T, _P, _P]),
    "mg_graph_rebind_input": (ctypes.c_int, [_P, _I, _P, _P]),
    "mg_capture_begin": (ctypes.c_int, [_P]),
    "mg_capture_end": (ctypes.c_int, [_P, ctypes.POINTER(_P)]),
    "mg_captured_launch": (ctypes.c_int, [_P, _P]),
    "mg_captured_destroy": (ctypes.c_int, [_P]),
    "mg_device_synchronize": (ctypes.c_int, []),
    "mg_last_error": (ctypes.c_char_p, []),
    "mg_version": (ctypes.c_char_p, []),
    "mg_launch_count": (ctypes.c_uint64, []),
}

_lib = None


class MuGraphError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("%s: %s" % (STATUS_NAMES.get(status, status), message))
        self.status = status


def load():
    """Load libmugraph.so (built in-tree by attention_superoptimizer_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libmugraph.so is missing at %s - run `python -m attention_superoptimizer_b200.build`; "
                              "there is no CPU fallback" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status):
    if status != MG_OK:
        raise MuGraphError(status, load().mg_last_error().decode())
