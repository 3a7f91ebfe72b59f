"""Host-side mirror of the reference's KVCache (Sources/EdgeRunnerMetal/KVCache.swift:12-1138) over the
CUDA backend.  Method names, argument meaning and error cases follow the Swift class; storage lives on the
GPU behind the C ABI (include/er_kv.h), so the `MTLBuffer` accessors become raw device pointers.

Device-side operators take torch CUDA tensors (or raw device pointers) and a torch stream.
"""
import ctypes as C
import enum

import numpy as np

from . import _lib
from ._lib import (EdgeRunnerCUDAError, ERKVCacheParams, check, er_kv_buffers, er_kv_config, er_step_params, lib, ptr,
                   stream_ptr)

ALL_SEQUENCES = 0xFFFFFFFF


def _sync_current_stream(stream):
    """Host-visible completion of copies enqueued on `stream` (None: the whole device)."""
    import torch
    if stream is None or isinstance(stream, int):
        torch.cuda.synchronize()
    else:
        stream.synchronize()


class Precision(enum.IntEnum):
    """KVCache.Precision raw values (KVCache.swift:39-49)."""
    float32 = 0
    float16 = 1
    float8 = 2
    q8_0 = 3
    turboquantV2 = 4
    turboQuantBalanced = 5
    turboQuantAggressive = 6


class TurboQuantFixedType(enum.IntEnum):
    """TurboQuantFixedType (TurboQuant.swift:172-190); value = bits per coordinate."""
    turbo2 = 2
    turbo3 = 3
    turbo4 = 4


class OutlierSelection(enum.IntEnum):
    """TurboQuantOutlierSelection (TurboQuant.swift:1185-1238); default_ = the contract's rule for the tensor."""
    default_ = 0
    magnitude = 1
    quantizationBenefit = 2


class Layout(enum.IntEnum):
    token_major = 0   # the reference's [slot][kvHead][dim] ring
    head_major = 1    # [seq][kvHead][slot][dim]
    paged = 2         # [page][kvHead][slotInPage][dim] + block tables


class NormFormat(enum.IntEnum):
    float32 = 0
    float16 = 1


def step_params(rope_theta=10000.0, rope_scaling=1.0, softmax_scale=0.0, apply_rope=True, q_norm_weight=None,
                k_norm_weight=None, rms_eps=1e-6, norm_weight_layer_stride=0, sliding_window=0):
    """q_norm_weight / k_norm_weight: device float tensors (or raw pointers) of headDim weights per layer; the caller keeps
    them alive while the parameters are in use.  sliding_window > 0: every query row attends to the newest rows only."""
    p = er_step_params()
    p.rope_theta, p.rope_scaling, p.softmax_scale, p.apply_rope = rope_theta, rope_scaling, softmax_scale, int(apply_rope)
    p.q_norm_weight, p.k_norm_weight = ptr(q_norm_weight), ptr(k_norm_weight)
    p.rms_eps, p.norm_weight_layer_stride = rms_eps, norm_weight_layer_stride
    p.sliding_window = sliding_window
    return p


class KVCache:
    def __init__(self, max_seq_len, num_layers, num_kv_heads, head_dim, precision, *, key_type=None, value_type=None,
                 norm_format=NormFormat.float32, max_batch=1, layout=Layout.head_major, page_size=0, num_pages=0,
                 prefill_kernel=0, decode_kernel=0, key_residual_scale=0.0, value_residual_scale=0.0):
        """key_type / value_type: TurboQuantFixedType for turboquantV2 caches (default turbo3, the reference's contract);
        OutlierSelection for turboQuantBalanced / turboQuantAggressive caches (default: keys by magnitude, values by
        quantisation benefit), whose residual scales default to the contract's 0."""
        preset = int(precision) in (int(Precision.turboQuantBalanced), int(Precision.turboQuantAggressive))
        if key_type is None:
            key_type = 0 if preset else TurboQuantFixedType.turbo3
        if value_type is None:
            value_type = 0 if preset else TurboQuantFixedType.turbo3
        cfg = er_kv_config()
        cfg.key_residual_scale, cfg.value_residual_scale = float(key_residual_scale), float(value_residual_scale)
        cfg.max_seq_len, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim = max_seq_len, num_layers, num_kv_heads, head_dim
        cfg.precision, cfg.key_type, cfg.value_type = int(precision), int(key_type), int(value_type)
        cfg.norm_format, cfg.max_batch, cfg.layout = int(norm_format), max_batch, int(layout)
        cfg.page_size, cfg.num_pages = page_size, num_pages
        cfg.prefill_kernel = int(prefill_kernel)     # 0 = automatic, 1 = always the mma.sync kernel (A/B measurements)
        cfg.decode_kernel = int(decode_kernel)       # float16 caches: 0 = automatic, 1 = persistent kernel, 2 = slim kernel; 3 = SIMT kernel for balanced / aggressive caches
        self._h = C.c_void_p()
        self._destroy = lib().er_kv_destroy      # held by the object: close() may run while the interpreter shuts down
        check(lib().er_kv_create(C.byref(cfg), C.byref(self._h)))
        got = er_kv_config()
        check(lib().er_kv_get_config(self._h, C.byref(got)))
        self.max_seq_len, self.num_layers, self.num_kv_heads, self.head_dim = max_seq_len, num_layers, num_kv_heads, head_dim
        self.precision = Precision(precision)
        self.key_type, self.value_type = int(key_type), int(value_type)
        self.max_batch, self.layout = got.max_batch, Layout(got.layout)
        self.norm_format = NormFormat(got.norm_format)
        self.page_size, self.num_pages = page_size, num_pages

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._destroy(self._h)
            self._h.value = None

    __del__ = close

    # ---- getters (KVCache.swift:90-190) ----
    @property
    def handle(self):
        return self._h

    @property
    def is_turboquant(self):
        return self.precision in (Precision.turboquantV2, Precision.turboQuantBalanced, Precision.turboQuantAggressive)

    @property
    def outlier_preset(self):
        """(regular bits, high-precision bits, high-precision channels) of a balanced / aggressive cache, else None."""
        return {Precision.turboQuantBalanced: (3, 5, 32), Precision.turboQuantAggressive: (2, 3, 32)}.get(self.precision)

    @property
    def elements_per_token(self):
        return self.num_kv_heads * self.head_dim

    @property
    def dense_bytes_per_token(self):
        per = {Precision.float32: 4, Precision.float16: 2}.get(self.precision)
        return None if per is None else self.elements_per_token * per

    @property
    def current_length(self):
        return check(lib().er_kv_current_length(self._h))

    def total_written(self, layer, seq=0):
        return check(lib().er_kv_total_written(self._h, layer, seq))

    # ---- host append / retrieve (KVCache.swift:410-629) ----
    def append(self, layer, keys, values, seq=0):
        k = np.ascontiguousarray(keys, dtype=np.float32).ravel()
        v = np.ascontiguousarray(values, dtype=np.float32).ravel()
        if k.size != v.size:
            raise EdgeRunnerCUDAError(_lib.ER_ERR_SHAPE, "keys/values differ in size")
        check(lib().er_kv_append_f32(self._h, layer, seq, k.ctypes.data, v.ctypes.data, k.size))

    def append_f16(self, layer, keys, values, seq=0):
        k = np.ascontiguousarray(keys, dtype=np.float16).ravel()
        v = np.ascontiguousarray(values, dtype=np.float16).ravel()
        check(lib().er_kv_append_f16(self._h, layer, seq, k.ctypes.data, v.ctypes.data, k.size))

    def retrieve(self, layer, as_type, seq=0):
        dt = np.dtype(as_type)
        cap = self.max_seq_len * self.elements_per_token
        k, v = np.zeros(cap, dtype=dt), np.zeros(cap, dtype=dt)
        n = C.c_uint32(0)
        check(lib().er_kv_retrieve(self._h, layer, seq, dt.itemsize, k.ctypes.data, v.ctypes.data, cap, C.byref(n)))
        m = n.value * self.elements_per_token
        return k[:m], v[:m]

    def retrieve_decoded_turboquant(self, layer, seq=0):
        cap = self.max_seq_len * self.elements_per_token
        k, v = np.zeros(cap, dtype=np.float32), np.zeros(cap, dtype=np.float32)
        n = C.c_uint32(0)
        check(lib().er_kv_retrieve_decoded_turboquant(self._h, layer, seq, k.ctypes.data, v.ctypes.data, cap, C.byref(n)))
        m = n.value * self.elements_per_token
        return k[:m], v[:m]

    def retrieve_decoded_q8_0(self, layer, seq=0):
        """KVCache.retrieveDecodedQ8_0 (KVCache.swift:882-908): (keys, values) as flat float32 arrays."""
        cap = self.max_seq_len * self.elements_per_token
        k, v = np.zeros(cap, dtype=np.float32), np.zeros(cap, dtype=np.float32)
        n = C.c_uint32(0)
        check(lib().er_kv_retrieve_decoded_q8_0(self._h, layer, seq, k.ctypes.data, v.ctypes.data, cap, C.byref(n)))
        m = n.value * self.elements_per_token
        return k[:m], v[:m]

    def retrieve_q8_0_rows(self, layer, seq=0):
        """Stored rows in the reference's block format: (k, v) uint8 [tokens, kv heads, 136]."""
        cap = self.max_seq_len * self.num_kv_heads * 136
        k, v = np.zeros(cap, dtype=np.uint8), np.zeros(cap, dtype=np.uint8)
        n = C.c_uint32(0)
        check(lib().er_kv_retrieve_q8_0_rows(self._h, layer, seq, k.ctypes.data, v.ctypes.data, cap, C.byref(n)))
        m = n.value * self.num_kv_heads * 136
        return k[:m].reshape(n.value, self.num_kv_heads, 136), v[:m].reshape(n.value, self.num_kv_heads, 136)

    def retrieve_turboquant_runtime_rows(self, layer, seq=0):
        """((k_codes, k_signs, k_mask, k_meta), (v_...)) in the reference's split-buffer row format."""
        out = []
        cap = self.max_seq_len * self.num_kv_heads
        for is_value, bits in ((0, self.key_type), (1, self.value_type)):
            words = (128 * bits + 31) // 32
            if self.outlier_preset is not None:
                rb, hb, n_high = self.outlier_preset
                words = (128 * rb + n_high * (hb - rb) + 31) // 32
            codes = np.zeros((cap, words), dtype=np.uint32)
            signs = np.zeros((cap, 4), dtype=np.uint32)
            mask = np.zeros((cap, 4), dtype=np.uint32)
            meta = np.zeros((cap, 2), dtype=np.float32)
            n = C.c_uint32(0)
            check(lib().er_kv_retrieve_turboquant_rows(self._h, layer, seq, is_value, codes.ctypes.data, signs.ctypes.data,
                                                       mask.ctypes.data, meta.ctypes.data, cap, C.byref(n)))
            out.append((codes[:n.value], signs[:n.value], mask[:n.value], meta[:n.value]))
        return tuple(out)

    # ---- buffers / params / position control (KVCache.swift:631-729) ----
    def device_buffers(self, layer):
        b = er_kv_buffers()
        check(lib().er_kv_device_buffers(self._h, layer, C.byref(b)))
        return b

    def metal_buffers(self, layer):
        """Dense-path accessor: raises compressedBufferAccessRequiresTurboQuantAPI on TurboQuant storage
        (KVCache.swift:631-634, 836-848)."""
        b = self.device_buffers(layer)
        if self.is_turboquant:
            raise EdgeRunnerCUDAError(_lib.ER_ERR_COMPRESSED_BUFFER_ACCESS_REQUIRES_TURBOQUANT_API)
        return b.keys, b.values

    def turboquant_buffers(self, layer):
        b = self.device_buffers(layer)
        if not self.is_turboquant:
            raise EdgeRunnerCUDAError(_lib.ER_ERR_PRECISION_MISMATCH)
        return b

    def cache_params(self, layer, seq=0):
        p = ERKVCacheParams()
        check(lib().er_kv_cache_params(self._h, layer, seq, C.byref(p)))
        return p

    def reset(self):
        check(lib().er_kv_reset(self._h))

    def advance_write_position(self, layer, count, seq=ALL_SEQUENCES):
        check(lib().er_kv_advance_write_position(self._h, layer, seq, count))

    def set_position(self, position, seq=ALL_SEQUENCES):
        check(lib().er_kv_set_position(self._h, seq, position))

    def set_block_table(self, seq, pages):
        arr = np.ascontiguousarray(pages, dtype=np.int32)
        check(lib().er_kv_set_block_table(self._h, seq, arr.ctypes.data, arr.size))

    def get_block_table(self, seq):
        arr = np.zeros(max(1, (self.max_seq_len + max(self.page_size, 1) - 1) // max(self.page_size, 1)), dtype=np.int32)
        n = C.c_uint32(0)
        check(lib().er_kv_get_block_table(self._h, seq, arr.ctypes.data, arr.size, C.byref(n)))
        return arr[:n.value].tolist()

    # ---- device operators ----
    def append_rope_kv(self, k, v, params, layer_begin=0, layer_end=None, stream=None):
        le = self.num_layers if layer_end is None else layer_end
        check(lib().er_kv_append_rope_kv(self._h, layer_begin, le, ptr(k), ptr(v), C.byref(params), stream_ptr(stream)))

    def attention_decode(self, q, out, num_heads, params, pending=0, layer_begin=0, layer_end=None, stream=None):
        le = self.num_layers if layer_end is None else layer_end
        check(lib().er_kv_attention_decode(self._h, layer_begin, le, ptr(q), ptr(out), num_heads, pending, C.byref(params),
                                           stream_ptr(stream)))

    def attention_prefill(self, layer, seq, q, out, num_heads, seq_len, params, q_offset=None, stream=None):
        """Causal attention of `seq_len` query rows over the cache rows of (layer, seq); q_offset None = the queries are
        the newest rows."""
        off = 0xFFFFFFFF if q_offset is None else q_offset
        check(lib().er_kv_attention_prefill(self._h, layer, seq, ptr(q), ptr(out), num_heads, seq_len, off, C.byref(params),
                                            stream_ptr(stream)))

    def attention_decode_with_values_of(self, value_cache, q, out, num_heads, params, pending=0, layer_begin=0, layer_end=None,
                                        stream=None):
        """Decode attention with THIS cache's K rows and `value_cache`'s V rows (layers whose keys and values use different
        row formats; er_kv_attention_decode_pair)."""
        le = self.num_layers if layer_end is None else layer_end
        check(lib().er_kv_attention_decode_pair(self._h, value_cache._h, layer_begin, le, ptr(q), ptr(out), num_heads, pending,
                                                C.byref(params), stream_ptr(stream)))

    def attention_prefill_with_values_of(self, value_cache, layer, seq, q, out, num_heads, seq_len, params, q_offset=None, stream=None):
        off = 0xFFFFFFFF if q_offset is None else q_offset
        check(lib().er_kv_attention_prefill_pair(self._h, value_cache._h, layer, seq, ptr(q), ptr(out), num_heads, seq_len, off,
                                                 C.byref(params), stream_ptr(stream)))

    def decode_step(self, q, k, v, out, num_heads, params, layer_begin=0, layer_end=None, stream=None):
        le = self.num_layers if layer_end is None else layer_end
        check(lib().er_kv_decode_step(self._h, layer_begin, le, ptr(q), ptr(k), ptr(v), ptr(out), num_heads,
                                      C.byref(params), stream_ptr(stream)))

    def decode_step_host(self, q, k, v, out, num_heads, params, layer_begin=0, layer_end=None, stream=None):
        """q/k/v/out: host buffers (numpy arrays or pinned torch CPU tensors)."""
        le = self.num_layers if layer_end is None else layer_end
        check(lib().er_kv_decode_step_host(self._h, layer_begin, le, ptr(q), ptr(k), ptr(v), ptr(out), num_heads,
                                           C.byref(params), stream_ptr(stream)))

    def advance(self, count=1, layer_begin=0, layer_end=None, stream=None):
        le = self.num_layers if layer_end is None else layer_end
        check(lib().er_kv_advance(self._h, layer_begin, le, count, stream_ptr(stream)))

    def write_rows(self, layer, seq, start, count, k, v, params, stream=None):
        check(lib().er_kv_write_rows(self._h, layer, seq, start, count, ptr(k), ptr(v), C.byref(params), stream_ptr(stream)))

    def page_bytes(self):
        """Bytes of one page over all layers, side arrays included (er_kv_page_bytes)."""
        return check(lib().er_kv_page_bytes(self._h))

    def export_pages(self, page_ids, buffer=None, stream=None):
        """Pack the pages into `buffer` (torch CUDA / pinned tensor, numpy array or raw address; default: a new numpy
        uint8 array, copied synchronously) and return it."""
        ids = np.ascontiguousarray(page_ids, dtype=np.int32)
        need = int(self.page_bytes()) * len(ids)
        own = buffer is None
        if own:
            buffer = np.empty(need, dtype=np.uint8)
        size = need if isinstance(buffer, int) else int(buffer.nbytes if hasattr(buffer, "nbytes") else buffer.numel() * buffer.element_size())
        check(lib().er_kv_export_pages(self._h, ids.ctypes.data, len(ids), ptr(buffer), size, stream_ptr(stream)))
        if own or stream is None:
            _sync_current_stream(stream)
        return buffer

    def import_pages(self, page_ids, buffer, stream=None):
        ids = np.ascontiguousarray(page_ids, dtype=np.int32)
        size = int(self.page_bytes()) * len(ids) if isinstance(buffer, int) else int(
            buffer.nbytes if hasattr(buffer, "nbytes") else buffer.numel() * buffer.element_size())
        check(lib().er_kv_import_pages(self._h, ids.ctypes.data, len(ids), ptr(buffer), size, stream_ptr(stream)))
        if stream is None:
            _sync_current_stream(stream)

    def set_trace(self, buffer, capacity_ctas):
        """Install (or, with None, remove) a device int64 buffer [capacity_ctas, 8] for per-CTA phase timestamps."""
        return check(lib().er_kv_set_trace(self._h, ptr(buffer), capacity_ctas))

    def device_status(self):
        """0, or the negative status a kernel of this cache left behind (ER_ERR_DEVICE_TIMEOUT, ER_ERR_OUT_OF_PAGES)."""
        return lib().er_kv_device_status(self._h)

    def set_output_sharding(self, heads_total, head_offset, peer_outputs=()):
        """kv-head sharding (er_kv_set_output_sharding): decode launches write their rows at head offset `head_offset` of
        [layers, batch, heads_total, 128] buffers -- the call's `out` and the raw peer addresses in `peer_outputs`."""
        arr = (C.c_void_p * max(len(peer_outputs), 1))(*[int(p) for p in peer_outputs])
        check(lib().er_kv_set_output_sharding(self._h, heads_total, head_offset, arr, len(peer_outputs)))

    def clear_device_status(self):
        check(lib().er_kv_clear_device_status(self._h))

    def debug_wait_probe(self, wait_limit_us=0, withhold_tiles=False):
        """Test hook of the bounded-wait path (er_kv_debug_wait_probe); (0, False) restores normal operation."""
        check(lib().er_kv_debug_wait_probe(self._h, wait_limit_us, int(bool(withhold_tiles))))
