"""ctypes binding of liber_kv.so (the C ABI of include/er_kv.h).

The library is the product: there is no Python or CPU fallback.  Importing this module on a machine
where the shared library has not been built raises immediately with the build command.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "liber_kv.so")


class ERKVCacheParams(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("maxSeqLen", "currentLen", "writePos", "numKVHeads", "headDim", "precision")]


class ERGQAParams(C.Structure):
    _fields_ = [("seqLen", C.c_uint32), ("headDim", C.c_uint32), ("numHeads", C.c_uint32), ("numKVHeads", C.c_uint32),
                ("groupSize", C.c_uint32), ("scale", C.c_float), ("causal", C.c_uint32), ("kvBlockSize", C.c_uint32),
                ("qBlockSize", C.c_uint32), ("kvSeqLen", C.c_uint32), ("qOffset", C.c_uint32)]


class ERWindowedGQAParams(C.Structure):
    _fields_ = [("numHeads", C.c_uint32), ("numKVHeads", C.c_uint32), ("headDim", C.c_uint32), ("kvStart", C.c_uint32),
                ("kvCount", C.c_uint32), ("kvCapacity", C.c_uint32), ("attentionScale", C.c_float)]


class ERRoPEParams(C.Structure):
    _fields_ = [("seqLen", C.c_uint32), ("numHeads", C.c_uint32), ("headDim", C.c_uint32), ("startPos", C.c_uint32),
                ("theta", C.c_float), ("scalingFactor", C.c_float), ("partialRotaryFactor", C.c_float)]


class er_kv_config(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("max_seq_len", "num_layers", "num_kv_heads", "head_dim", "precision",
                                          "key_type", "value_type", "norm_format", "max_batch", "layout",
                                          "page_size", "num_pages", "prefill_kernel", "decode_kernel")] + [
        ("key_residual_scale", C.c_float), ("value_residual_scale", C.c_float)]


class er_kv_buffers(C.Structure):
    _fields_ = [("keys", C.c_void_p), ("values", C.c_void_p), ("key_norms", C.c_void_p), ("value_norms", C.c_void_p),
                ("key_bytes", C.c_uint64), ("value_bytes", C.c_uint64), ("key_row_bytes", C.c_uint32),
                ("value_row_bytes", C.c_uint32)]


class er_step_params(C.Structure):
    _fields_ = [("rope_theta", C.c_float), ("rope_scaling", C.c_float), ("softmax_scale", C.c_float),
                ("apply_rope", C.c_uint32), ("q_norm_weight", C.c_void_p), ("k_norm_weight", C.c_void_p),
                ("rms_eps", C.c_float), ("norm_weight_layer_stride", C.c_uint32), ("sliding_window", C.c_uint32), ("reserved", C.c_uint32)]


# status codes (include/er_kv.h)
ER_OK = 0
ER_ERR_ALLOCATION_FAILED, ER_ERR_INVALID_LAYER, ER_ERR_PRECISION_MISMATCH, ER_ERR_UNSUPPORTED_STORAGE = -1, -2, -3, -4
ER_ERR_COMPRESSED_RETRIEVE_REQUIRES_DECODED_API, ER_ERR_COMPRESSED_BUFFER_ACCESS_REQUIRES_TURBOQUANT_API = -5, -6
ER_ERR_SHAPE, ER_ERR_CUDA, ER_ERR_INVALID_ARGUMENT, ER_ERR_OUT_OF_PAGES, ER_ERR_UNSUPPORTED, ER_ERR_DEVICE_TIMEOUT = (
    -7, -8, -9, -10, -11, -12)

# every symbol include/er_kv.h declares: name -> (restype, argtypes)
_vp, _u32, _i32, _sz = C.c_void_p, C.c_uint32, C.c_int32, C.c_size_t
_stp = C.POINTER(er_step_params)
SYMBOLS = {
    "er_status_string": (C.c_char_p, [_i32]),
    "er_last_error_string": (C.c_char_p, []),
    "er_device_count": (_i32, []),
    "er_kv_create": (_i32, [C.POINTER(er_kv_config), C.POINTER(_vp)]),
    "er_kv_destroy": (None, [_vp]),
    "er_kv_get_config": (_i32, [_vp, C.POINTER(er_kv_config)]),
    "er_kv_current_length": (_i32, [_vp]),
    "er_kv_total_written": (C.c_int64, [_vp, _u32, _u32]),
    "er_kv_append_f32": (_i32, [_vp, _u32, _u32, _vp, _vp, _sz]),
    "er_kv_append_f16": (_i32, [_vp, _u32, _u32, _vp, _vp, _sz]),
    "er_kv_retrieve": (_i32, [_vp, _u32, _u32, _u32, _vp, _vp, _sz, C.POINTER(_u32)]),
    "er_kv_retrieve_decoded_turboquant": (_i32, [_vp, _u32, _u32, _vp, _vp, _sz, C.POINTER(_u32)]),
    "er_kv_retrieve_decoded_q8_0": (_i32, [_vp, _u32, _u32, _vp, _vp, _sz, C.POINTER(_u32)]),
    "er_kv_retrieve_q8_0_rows": (_i32, [_vp, _u32, _u32, _vp, _vp, _sz, C.POINTER(_u32)]),
    "er_kv_retrieve_turboquant_rows": (_i32, [_vp, _u32, _u32, C.c_int, _vp, _vp, _vp, _vp, _sz, C.POINTER(_u32)]),
    "er_kv_device_buffers": (_i32, [_vp, _u32, C.POINTER(er_kv_buffers)]),
    "er_kv_cache_params": (_i32, [_vp, _u32, _u32, C.POINTER(ERKVCacheParams)]),
    "er_kv_reset": (_i32, [_vp]),
    "er_kv_advance_write_position": (_i32, [_vp, _u32, _u32, _u32]),
    "er_kv_set_position": (_i32, [_vp, _u32, _u32]),
    "er_kv_set_block_table": (_i32, [_vp, _u32, _vp, _u32]),
    "er_kv_get_block_table": (_i32, [_vp, _u32, _vp, _u32, C.POINTER(_u32)]),
    "er_rope_neox_f32": (_i32, [_vp, _vp, C.POINTER(ERRoPEParams), _vp]),
    "er_rope_neox_f32_to_f16": (_i32, [_vp, _vp, C.POINTER(ERRoPEParams), _vp]),
    "er_quantize_q8_0_rows": (_i32, [_vp, _u32, _u32, _u32, _vp, _vp]),
    "er_turboquant_quantize_rows": (_i32, [_vp, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "er_turboquant_quantize_rows_outliers": (_i32, [_vp, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "er_gqa_attention_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, C.POINTER(ERGQAParams), _vp]),
    "er_gqa_attention_f16kv": (_i32, [_vp, _vp, _vp, _vp, C.POINTER(ERGQAParams), _vp]),
    "er_gqa_attention_f16kv_static": (_i32, [_vp, _vp, _vp, _vp, C.POINTER(ERGQAParams), _vp]),
    "er_gqa_attention_f16kv_windowed": (_i32, [_vp, _vp, _vp, _vp, C.POINTER(ERWindowedGQAParams), _vp]),
    "er_kv_append_rope_kv": (_i32, [_vp, _u32, _u32, _vp, _vp, _stp, _vp]),
    "er_kv_attention_decode": (_i32, [_vp, _u32, _u32, _vp, _vp, _u32, _u32, _stp, _vp]),
    "er_kv_attention_prefill": (_i32, [_vp, _u32, _u32, _vp, _vp, _u32, _u32, _u32, _stp, _vp]),
    "er_kv_decode_step": (_i32, [_vp, _u32, _u32, _vp, _vp, _vp, _vp, _u32, _stp, _vp]),
    "er_kv_decode_step_host": (_i32, [_vp, _u32, _u32, _vp, _vp, _vp, _vp, _u32, _stp, _vp]),
    "er_kv_advance": (_i32, [_vp, _u32, _u32, _u32, _vp]),
    "er_kv_write_rows": (_i32, [_vp, _u32, _u32, _u32, _u32, _vp, _vp, _stp, _vp]),
    "er_kv_set_output_sharding": (_i32, [_vp, _u32, _u32, C.POINTER(_vp), _u32]),
    "er_relayout_head_shards": (_i32, [_vp, _vp, _u32, _u32, _u32, _vp]),
    "er_peer_buffer_create": (_i32, [_sz, C.POINTER(_vp), _vp]),
    "er_peer_buffer_open": (_i32, [_vp, C.POINTER(_vp)]),
    "er_peer_buffer_close": (_i32, [_vp]),
    "er_peer_buffer_destroy": (_i32, [_vp]),
    "er_kernel_launch_count": (C.c_uint64, []),
    "er_kv_device_status": (_i32, [_vp]),
    "er_kv_clear_device_status": (_i32, [_vp]),
    "er_kv_debug_wait_probe": (_i32, [_vp, _u32, C.c_int]),
    "er_workspace_status": (_i32, []),
    "er_gqa_attention_f16kv_static_status": (_i32, []),
    "er_kv_set_trace": (_i32, [_vp, _vp, _u32]),
    "er_kv_attention_decode_pair": (_i32, [_vp, _vp, _u32, _u32, _vp, _vp, _u32, _u32, _vp, _vp]),
    "er_kv_attention_prefill_pair": (_i32, [_vp, _vp, _u32, _u32, _vp, _vp, _u32, _u32, _u32, _vp, _vp]),
    "er_kv_page_bytes": (C.c_int64, [_vp]),
    "er_kv_export_pages": (_i32, [_vp, _vp, _u32, _vp, _sz, _vp]),
    "er_kv_import_pages": (_i32, [_vp, _vp, _u32, _vp, _sz, _vp]),
    "er_host_alloc": (_i32, [C.POINTER(_vp), _sz]),
    "er_host_free": (_i32, [_vp]),
}

_LIB = None


class EdgeRunnerCUDAError(RuntimeError):
    """Status returned by the C ABI; `.code` is the ER_ERR_* value, `.name` its KVCacheError case name."""

    def __init__(self, code, detail=""):
        self.code = code
        self.name = lib().er_status_string(code).decode() if _LIB is not None else str(code)
        super().__init__("%s (%d)%s" % (self.name, code, ": " + detail if detail else ""))


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "edgerunner_b200: %s is missing. Build it with `python -m edgerunner_b200.build` "
            "(needs nvcc); there is no fallback implementation." % LIB_PATH)
    L = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(L, name)      # AttributeError here = the library does not export what the header declares
        fn.restype = res
        fn.argtypes = args
    _LIB = L
    return L


def check(code):
    if code < 0:
        raise EdgeRunnerCUDAError(code, lib().er_last_error_string().decode())
    return code


def ptr(x):
    """Device/host pointer of a torch tensor, numpy array, ctypes object or int."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    return C.cast(x, C.c_void_p).value


def stream_ptr(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream
