"""ctypes front end of the CPU oracle (oracle/er_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
CPU-baseline legs of bench.py.  The shipped package never imports this module.

`build()` compiles the C restatement next to its source; `lib()` loads it.
All array arguments are numpy arrays; outputs are freshly allocated numpy arrays.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liber_oracle.so")
_LIB = None

DIM = 128
PREC_F32, PREC_F16, PREC_TURBO_V2 = 0, 1, 4
ERR = {
    0: "ok", -1: "allocationFailed", -2: "invalidLayer", -3: "precisionMismatch", -4: "unsupportedStorage",
    -5: "compressedRetrieveRequiresDecodedAPI", -6: "compressedBufferAccessRequiresTurboQuantAPI", -7: "shape",
}


def build(force=False):
    src = os.path.join(_HERE, "er_oracle.c")
    hdr = os.path.join(_HERE, "er_tq_tables.h")
    if (not force and os.path.exists(_SO)
            and os.path.getmtime(_SO) >= max(os.path.getmtime(src), os.path.getmtime(hdr))):
        return _SO
    env = dict(os.environ)
    env.pop("CC", None)
    subprocess.check_call(["make", "-C", _HERE, "-B", "liber_oracle.so"], env=env,
                          stdout=subprocess.DEVNULL)
    return _SO


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_SO):
        build()
    L = C.CDLL(_SO)
    f32p, u16p, u32p, u8p, i32p = (C.POINTER(C.c_float), C.POINTER(C.c_uint16), C.POINTER(C.c_uint32),
                                   C.POINTER(C.c_uint8), C.POINTER(C.c_int))
    L.ero_f32_to_f16.restype = C.c_uint16
    L.ero_f32_to_f16.argtypes = [C.c_float]
    L.ero_f16_to_f32.restype = C.c_float
    L.ero_f16_to_f32.argtypes = [C.c_uint16]
    rope_args = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_float]
    L.ero_rope_interleaved_f32.argtypes = [f32p, f32p] + rope_args
    L.ero_rope_neox_f32.argtypes = [f32p, f32p] + rope_args
    L.ero_rope_neox_f32_to_f16.argtypes = [f32p, u16p] + rope_args
    L.ero_convert_f32_to_f16.argtypes = [f32p, u16p, C.c_size_t]
    L.ero_convert_f16_to_f32.argtypes = [u16p, f32p, C.c_size_t]
    L.ero_gqa_f32.argtypes = [f32p, f32p, f32p, f32p] + [C.c_int] * 8
    L.ero_gqa_f32_masked.argtypes = [f32p, f32p, f32p, f32p] + [C.c_int] * 8 + [f32p]
    L.ero_gqa_f16kv.argtypes = [f32p, u16p, u16p, f32p] + [C.c_int] * 8
    L.ero_splitk_merge.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, f32p]
    L.ero_gqa_f16kv_windowed.argtypes = [f32p, u16p, u16p, f32p] + [C.c_int] * 6 + [C.c_float]
    L.ero_tq_sign.restype = C.c_float
    L.ero_tq_sign.argtypes = [C.c_int, C.c_int]
    L.ero_tq_centroid.restype = C.c_float
    L.ero_tq_centroid.argtypes = [C.c_int, C.c_int]
    L.ero_tq_threshold.restype = C.c_float
    L.ero_tq_threshold.argtypes = [C.c_int, C.c_int]
    L.ero_tq_code_words_per_row.argtypes = [C.c_int]
    L.ero_tq_bytes_per_row.argtypes = [C.c_int]
    L.ero_tq_layout_words.argtypes = [C.c_int, C.c_int, C.c_int, i32p, i32p, i32p]
    L.ero_tq_fwht.argtypes = [f32p]
    L.ero_tq_forward_scale.restype = C.c_float
    L.ero_tq_forward.argtypes = [f32p, C.c_int, f32p]
    L.ero_tq_inverse.argtypes = [f32p, f32p]
    L.ero_tq_code_for.argtypes = [C.c_float, C.c_int]
    L.ero_tq_pack_codes.argtypes = [u8p, C.c_int, C.c_int, u32p]
    L.ero_tq_unpack_codes.argtypes = [u32p, C.c_int, C.c_int, u8p]
    L.ero_tq_pack_codes_split.argtypes = [u8p, u8p, C.c_int, C.c_int, C.c_int, u32p]
    L.ero_tq_unpack_codes_split.argtypes = [u32p, C.c_int, u8p, C.c_int, C.c_int, C.c_int, u8p]
    L.ero_tq_encode.argtypes = [f32p, C.c_int, C.c_int, u32p, u32p, u32p, f32p, f32p, f32p]
    L.ero_tq_decode.argtypes = [u32p, C.c_int, C.c_float, C.c_int, f32p]
    L.ero_tq_topk_mask.argtypes = [f32p, C.c_int, C.c_int, C.c_int, C.c_int, u8p]
    L.ero_tq_preset_code_words.argtypes = [C.c_int] * 3
    L.ero_tq_encode_preset.argtypes = [f32p] + [C.c_int] * 5 + [u32p, u32p, u32p, f32p, f32p]
    L.ero_tq_decode_preset.argtypes = [u32p, u32p, u32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, C.c_int, f32p]
    L.ero_tq_score.restype = C.c_float
    L.ero_tq_score.argtypes = [f32p, C.c_int, u32p, C.c_int, C.c_float, C.c_float, f32p]
    L.ero_tq_attention_decode.argtypes = [f32p, u32p, f32p, C.c_int, u32p, f32p, C.c_int, f32p,
                                          C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]
    L.ero_tq_attention_decode_preset.argtypes = [f32p, u32p, u32p, u32p, f32p, u32p, u32p, u32p, f32p, C.c_int, C.c_int, C.c_int,
                                                 C.c_float, C.c_float, f32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]
    L.ero_kv_create.restype = C.c_void_p
    L.ero_kv_create.argtypes = [C.c_int] * 7
    L.ero_kv_destroy.argtypes = [C.c_void_p]
    L.ero_kv_current_length.argtypes = [C.c_void_p]
    L.ero_kv_append_f32.argtypes = [C.c_void_p, C.c_int, f32p, f32p]
    L.ero_kv_append_f16.argtypes = [C.c_void_p, C.c_int, u16p, u16p]
    L.ero_kv_ordered_slots.argtypes = [C.c_void_p, C.c_int, i32p]
    L.ero_kv_retrieve.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    L.ero_kv_retrieve_decoded_turboquant.argtypes = [C.c_void_p, C.c_int, f32p, f32p]
    L.ero_kv_turbo_buffer.restype = C.c_void_p
    L.ero_kv_turbo_buffer.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
    L.ero_kv_dense_buffer.restype = C.c_void_p
    L.ero_kv_dense_buffer.argtypes = [C.c_void_p, C.c_int, C.c_int]
    L.ero_kv_params.argtypes = [C.c_void_p, C.c_int, u32p]
    L.ero_kv_reset.argtypes = [C.c_void_p]
    L.ero_kv_advance_write_position.argtypes = [C.c_void_p, C.c_int, C.c_int]
    L.ero_kv_set_position.argtypes = [C.c_void_p, C.c_int]
    L.ero_decode_step_f16.argtypes = [f32p, f32p, f32p, u16p, u16p, f32p, f32p] + [C.c_int] * 4 + [
        C.c_float, C.c_float, C.c_int]
    L.ero_decode_step_turboquant.argtypes = [f32p, f32p, f32p, u32p, f32p, C.c_int, u32p, f32p, C.c_int, f32p,
                                             C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int]
    L.ero_head_rms_norm.argtypes = [f32p, f32p, C.c_float, C.c_int, f32p]
    L.ero_q8_encode_row.argtypes = [f32p, C.c_int, u8p]
    L.ero_q8_decode_row.argtypes = [u8p, C.c_int, f32p]
    L.ero_gqa_q8kv.argtypes = [f32p, u8p, u8p, f32p] + [C.c_int] * 8
    L.ero_decode_step_q8.argtypes = [f32p, f32p, f32p, u8p, u8p, f32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int]
    _LIB = L
    return L


F32, U16, U32, U8 = C.c_float, C.c_uint16, C.c_uint32, C.c_uint8


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads():
    return int(lib().ero_max_threads())


# ----------------------------------------------------------------------------- conversions / RoPE

def f32_to_f16_bits(a):
    a = _f32(a)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().ero_convert_f32_to_f16(_p(a, F32), _p(out, U16), a.size)
    return out


def f16_bits_to_f32(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().ero_convert_f16_to_f32(_p(a, U16), _p(out, F32), a.size)
    return out


def rope_neox(x, start_pos, theta, scaling=1.0, partial=1.0, interleaved=False):
    """x: [seq, heads, head_dim] float32."""
    x = _f32(x)
    s, h, d = x.shape
    out = np.empty_like(x)
    fn = lib().ero_rope_interleaved_f32 if interleaved else lib().ero_rope_neox_f32
    fn(_p(x, F32), _p(out, F32), s, h, d, start_pos, theta, scaling, partial)
    return out


def rope_neox_to_f16(x, start_pos, theta, scaling=1.0, partial=1.0):
    x = _f32(x)
    s, h, d = x.shape
    out = np.empty(x.shape, dtype=np.uint16)
    lib().ero_rope_neox_f32_to_f16(_p(x, F32), _p(out, U16), s, h, d, start_pos, theta, scaling, partial)
    return out


# ----------------------------------------------------------------------------- dense attention

def gqa_f32(q, k, v, causal=True, q_offset=0, threads=1, additive_mask=None):
    """q: [S,H,D]; k, v: [T,Hkv,D] float32 -> [S,H,D] (cpuGQA); additive_mask: [S,T] added to the scaled scores."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    s, h, d = q.shape
    t, hkv, _ = k.shape
    out = np.empty_like(q)
    if additive_mask is None:
        lib().ero_gqa_f32(_p(q, F32), _p(k, F32), _p(v, F32), _p(out, F32), s, d, h, hkv, int(causal), t, q_offset, threads)
    else:
        m = _f32(additive_mask)
        assert m.size == s * t
        lib().ero_gqa_f32_masked(_p(q, F32), _p(k, F32), _p(v, F32), _p(out, F32), s, d, h, hkv, int(causal), t, q_offset,
                                 threads, _p(m, F32))
    return out


def gqa_f16kv(q, k16, v16, causal=True, q_offset=0, threads=1):
    """q: [S,H,D] float32; k16, v16: [T,Hkv,D] uint16 fp16 bit patterns."""
    q = _f32(q)
    k16 = np.ascontiguousarray(k16, dtype=np.uint16)
    v16 = np.ascontiguousarray(v16, dtype=np.uint16)
    s, h, d = q.shape
    t, hkv, _ = k16.shape
    out = np.empty_like(q)
    lib().ero_gqa_f16kv(_p(q, F32), _p(k16, U16), _p(v16, U16), _p(out, F32), s, d, h, hkv, int(causal), t,
                        q_offset, threads)
    return out


def gqa_f16kv_windowed(q, k16, v16, kv_start, kv_count, scale=None):
    """q: [H,D] float32; k16, v16: [capacity,Hkv,D] fp16 bit patterns; rows (kv_start + i) % capacity, i < kv_count."""
    q = _f32(q)
    k16 = np.ascontiguousarray(k16, dtype=np.uint16)
    v16 = np.ascontiguousarray(v16, dtype=np.uint16)
    h, d = q.shape
    cap, hkv, _ = k16.shape
    out = np.empty_like(q)
    lib().ero_gqa_f16kv_windowed(_p(q, F32), _p(k16, U16), _p(v16, U16), _p(out, F32), h, hkv, d, kv_start, kv_count, cap,
                                 float(1.0 / np.sqrt(d)) if scale is None else float(scale))
    return out


def splitk_merge(part_max, part_sum, part_acc):
    part_max, part_sum, part_acc = _f32(part_max), _f32(part_sum), _f32(part_acc)
    n, d = part_acc.shape
    out = np.empty(d, dtype=np.float32)
    lib().ero_splitk_merge(_p(part_max, F32), _p(part_sum, F32), _p(part_acc, F32), n, d, _p(out, F32))
    return out


# ----------------------------------------------------------------------------- TurboQuant

def tq_forward(x):
    x = _f32(x).ravel()
    out = np.empty(DIM, dtype=np.float32)
    lib().ero_tq_forward(_p(x, F32), x.size, _p(out, F32))
    return out


def tq_inverse(x):
    x = _f32(x).ravel()
    assert x.size == DIM
    out = np.empty(DIM, dtype=np.float32)
    lib().ero_tq_inverse(_p(x, F32), _p(out, F32))
    return out


def tq_pack_codes(codes, bits):
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    words = np.zeros((codes.size * bits + 31) // 32, dtype=np.uint32)
    lib().ero_tq_pack_codes(_p(codes, U8), codes.size, bits, _p(words, U32))
    return words


def tq_unpack_codes(words, bits, count=DIM):
    words = np.ascontiguousarray(words, dtype=np.uint32)
    codes = np.empty(count, dtype=np.uint8)
    lib().ero_tq_unpack_codes(_p(words, U32), count, bits, _p(codes, U8))
    return codes


def tq_encode(x, bits):
    """One row -> dict(codes u32[w], signs u32[4], mask u32[4], row_norm, residual_norm, rotated f32[128])."""
    x = _f32(x).ravel()
    w = lib().ero_tq_code_words_per_row(bits)
    codes = np.zeros(w, dtype=np.uint32)
    signs = np.zeros(4, dtype=np.uint32)
    mask = np.zeros(4, dtype=np.uint32)
    rn, resn = F32(0), F32(0)
    rot = np.zeros(DIM, dtype=np.float32)
    lib().ero_tq_encode(_p(x, F32), x.size, bits, _p(codes, U32), _p(signs, U32), _p(mask, U32), C.byref(rn),
                        C.byref(resn), _p(rot, F32))
    return dict(codes=codes, signs=signs, mask=mask, row_norm=np.float32(rn.value),
                residual_norm=np.float32(resn.value), rotated=rot)


def tq_encode_rows(x, bits):
    """x: [rows, 128] -> (codes [rows, w] u32, norms [rows] f32)."""
    x = _f32(x)
    rows = x.shape[0]
    w = lib().ero_tq_code_words_per_row(bits)
    codes = np.zeros((rows, w), dtype=np.uint32)
    norms = np.zeros(rows, dtype=np.float32)
    signs = np.zeros(4, dtype=np.uint32)
    mask = np.zeros(4, dtype=np.uint32)
    rn, resn = F32(0), F32(0)
    L = lib()
    for r in range(rows):
        L.ero_tq_encode(_p(x[r], F32), x.shape[1], bits, _p(codes[r], U32), _p(signs, U32), _p(mask, U32),
                        C.byref(rn), C.byref(resn), None)
        norms[r] = rn.value
    return codes, norms


# TurboQuantPreset.descriptor of the presets with high-precision channels (TurboQuant.swift:78-84, 117-124):
# (regularBits, highPrecisionBits, highPrecisionChannelCount)
PRESETS = {"balanced": (3, 5, 32), "aggressive": (2, 3, 32)}


def tq_topk_mask(values, count, regular_bits, high_bits, use_benefit=False):
    v = _f32(values)
    mask = np.zeros(DIM, dtype=np.uint8)
    lib().ero_tq_topk_mask(_p(v, F32), count, regular_bits, high_bits, int(use_benefit), _p(mask, U8))
    return mask.astype(bool)


def tq_encode_preset(x, preset, use_benefit=False):
    """One row through TurboQuantReferenceEncoder.encode with a balanced / aggressive preset ->
    (code words, residual sign words [4], outlier mask words [4], rowNorm, residualNorm)."""
    rb, hb, n = PRESETS[preset]
    x = _f32(x).ravel()
    words = lib().ero_tq_preset_code_words(rb, hb, n)
    codes, signs, mask = np.zeros(words, np.uint32), np.zeros(4, np.uint32), np.zeros(4, np.uint32)
    rn, resn = C.c_float(0), C.c_float(0)
    lib().ero_tq_encode_preset(_p(x, F32), x.size, rb, hb, n, int(use_benefit), _p(codes, U32), _p(signs, U32), _p(mask, U32),
                               C.byref(rn), C.byref(resn))
    return codes, signs, mask, np.float32(rn.value), np.float32(resn.value)


def tq_encode_rows_preset(x, preset, use_benefit=False):
    """x: [n, 128] -> (codes [n, words], signs [n, 4], mask [n, 4], meta [n, 2] = (rowNorm, residualNorm))."""
    x = _f32(x).reshape(-1, DIM)
    rows = [tq_encode_preset(r, preset, use_benefit) for r in x]
    return (np.stack([r[0] for r in rows]), np.stack([r[1] for r in rows]), np.stack([r[2] for r in rows]),
            np.array([[r[3], r[4]] for r in rows], dtype=np.float32))


def tq_decode_preset(codes, signs, mask, preset, row_norm, residual_norm, residual_weight=1.0, count=DIM):
    rb, hb, n = PRESETS[preset]
    out = np.zeros(count, dtype=np.float32)
    codes, signs, mask = (np.ascontiguousarray(a, dtype=np.uint32) for a in (codes, signs, mask))
    lib().ero_tq_decode_preset(_p(codes, U32), _p(signs, U32), _p(mask, U32), rb, hb, n, float(row_norm), float(residual_norm),
                               float(residual_weight), count, _p(out, F32))
    return out


def tq_decode(codes, bits, row_norm, count=DIM):
    codes = np.ascontiguousarray(codes, dtype=np.uint32)
    out = np.empty(count, dtype=np.float32)
    lib().ero_tq_decode(_p(codes, U32), bits, float(row_norm), count, _p(out, F32))
    return out


def tq_score(q, codes, bits, row_norm, scale):
    q = _f32(q).ravel()
    codes = np.ascontiguousarray(codes, dtype=np.uint32)
    mse = F32(0)
    s = lib().ero_tq_score(_p(q, F32), q.size, _p(codes, U32), bits, float(row_norm), float(scale), C.byref(mse))
    return np.float32(s), np.float32(mse.value)


def tq_attention_decode(q, k_codes, k_norm, k_bits, v_codes, v_norm, v_bits, num_kv_heads, kv_len,
                        scale=None, threads=1):
    """q: [H,128]; codes: [T*Hkv, w] (row = token*Hkv + kvHead); norms: [T*Hkv] float32."""
    q = _f32(q)
    h = q.shape[0]
    k_codes = np.ascontiguousarray(k_codes, dtype=np.uint32)
    v_codes = np.ascontiguousarray(v_codes, dtype=np.uint32)
    k_norm, v_norm = _f32(k_norm), _f32(v_norm)
    out = np.empty_like(q)
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(DIM))
    lib().ero_tq_attention_decode(_p(q, F32), _p(k_codes, U32), _p(k_norm, F32), k_bits, _p(v_codes, U32),
                                  _p(v_norm, F32), v_bits, _p(out, F32), h, num_kv_heads, kv_len, float(scale),
                                  threads)
    return out


def tq_attention_decode_preset(q, k_rows, v_rows, preset, num_kv_heads, kv_len, key_residual_scale=0.0,
                               value_residual_scale=0.0, scale=None, threads=1):
    """q: [H,128]; k_rows / v_rows: (codes [T*Hkv, w], signs [T*Hkv, 4], mask [T*Hkv, 4], meta [T*Hkv, 2]) as
    tq_encode_rows_preset returns them (row = token*Hkv + kvHead)."""
    q = _f32(q)
    rb, hb, hc = PRESETS[preset]
    kc, ks, km, kmeta = (np.ascontiguousarray(a) for a in k_rows)
    vc, vs, vm, vmeta = (np.ascontiguousarray(a) for a in v_rows)
    out = np.empty_like(q)
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(DIM))
    lib().ero_tq_attention_decode_preset(_p(q, F32), _p(kc.astype(np.uint32, copy=False), U32), _p(ks.astype(np.uint32, copy=False), U32),
                                         _p(km.astype(np.uint32, copy=False), U32), _p(_f32(kmeta), F32),
                                         _p(vc.astype(np.uint32, copy=False), U32), _p(vs.astype(np.uint32, copy=False), U32),
                                         _p(vm.astype(np.uint32, copy=False), U32), _p(_f32(vmeta), F32), rb, hb, hc,
                                         C.c_float(key_residual_scale), C.c_float(value_residual_scale), _p(out, F32),
                                         q.shape[0], num_kv_heads, kv_len, C.c_float(scale), threads)
    return out


def head_rms_norm(x, weight, eps):
    """Per-head RMS norm of fused_qk_norm_rope_neox: x [..., 128], weight [128]."""
    x, weight = _f32(x), _f32(weight)
    out = np.empty_like(x)
    lib().ero_head_rms_norm(_p(x, F32), _p(weight, F32), float(eps), x.size // DIM, _p(out, F32))
    return out


# ----------------------------------------------------------------------------- q8_0 KV rows

def q8_encode_rows(x):
    """x: [..., 128] float32 -> uint8 [..., 136] (four 34-byte blocks per row: fp16 scale, 32 int8)."""
    x = _f32(x)
    d = x.shape[-1]
    rows = x.reshape(-1, d)
    out = np.empty((rows.shape[0], d // 32 * 34), dtype=np.uint8)
    U8 = C.POINTER(C.c_uint8)
    for r in range(rows.shape[0]):
        lib().ero_q8_encode_row(_p(rows[r], F32), d, out[r].ctypes.data_as(U8))
    return out.reshape(x.shape[:-1] + (d // 32 * 34,))


def q8_decode_rows(blocks, head_dim=DIM):
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    rows = blocks.reshape(-1, head_dim // 32 * 34)
    out = np.empty((rows.shape[0], head_dim), dtype=np.float32)
    U8 = C.POINTER(C.c_uint8)
    for r in range(rows.shape[0]):
        lib().ero_q8_decode_row(rows[r].ctypes.data_as(U8), head_dim, _p(out[r], F32))
    return out.reshape(blocks.shape[:-1] + (head_dim,))


def gqa_q8kv(q, k8, v8, causal=True, kv_seq_len=None, q_offset=0, threads=1):
    """q: [S, H, 128]; k8/v8: [T, Hkv, 136] uint8 rows."""
    q = _f32(q)
    k8 = np.ascontiguousarray(k8, dtype=np.uint8)
    v8 = np.ascontiguousarray(v8, dtype=np.uint8)
    s, h, d = q.shape
    t, hkv = k8.shape[0], k8.shape[1]
    out = np.empty_like(q)
    U8 = C.POINTER(C.c_uint8)
    lib().ero_gqa_q8kv(_p(q, F32), k8.ctypes.data_as(U8), v8.ctypes.data_as(U8), _p(out, F32), s, d, h, hkv, 1 if causal else 0,
                       t if kv_seq_len is None else kv_seq_len, q_offset, threads)
    return out


def decode_step_q8(q, k, v, k_cache, v_cache, pos, theta, scaling=1.0, threads=1):
    """q: [H,128]; k, v: [Hkv,128]; caches: uint8 [T, Hkv, 136], row `pos` is written in place."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty_like(q)
    U8 = C.POINTER(C.c_uint8)
    assert k_cache.flags.c_contiguous and v_cache.flags.c_contiguous and k_cache.dtype == np.uint8
    lib().ero_decode_step_q8(_p(q, F32), _p(k, F32), _p(v, F32), k_cache.ctypes.data_as(U8), v_cache.ctypes.data_as(U8), _p(out, F32),
                             int(pos), q.shape[0], k.shape[0], float(theta), float(scaling), threads)
    return out


# ----------------------------------------------------------------------------- KV ring cache

class OracleError(Exception):
    def __init__(self, code):
        super().__init__(ERR.get(code, str(code)))
        self.code = code


class OracleKVCache:
    """KVCache (KVCache.swift:12-1138) host semantics for float32 / float16 / turboquantV2."""

    def __init__(self, max_seq_len, num_layers, num_kv_heads, head_dim, precision, key_bits=3, value_bits=3):
        self.max_seq_len, self.num_layers = max_seq_len, num_layers
        self.num_kv_heads, self.head_dim, self.precision = num_kv_heads, head_dim, precision
        self.key_bits, self.value_bits = key_bits, value_bits
        self._h = lib().ero_kv_create(max_seq_len, num_layers, num_kv_heads, head_dim, precision, key_bits, value_bits)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ero_kv_destroy(self._h)
            self._h = None

    @property
    def current_length(self):
        return lib().ero_kv_current_length(self._h)

    def append(self, layer, keys, values):
        keys, values = _f32(keys).ravel(), _f32(values).ravel()
        assert keys.size == self.num_kv_heads * self.head_dim == values.size
        rc = lib().ero_kv_append_f32(self._h, layer, _p(keys, F32), _p(values, F32))
        if rc:
            raise OracleError(rc)

    def append_f16(self, layer, keys, values):
        keys = np.ascontiguousarray(keys, dtype=np.uint16).ravel()
        values = np.ascontiguousarray(values, dtype=np.uint16).ravel()
        rc = lib().ero_kv_append_f16(self._h, layer, _p(keys, U16), _p(values, U16))
        if rc:
            raise OracleError(rc)

    def retrieve(self, layer, dtype):
        dtype = np.dtype(dtype)
        n_max = self.max_seq_len * self.num_kv_heads * self.head_dim
        k = np.zeros(n_max, dtype=dtype)
        v = np.zeros(n_max, dtype=dtype)
        rc = lib().ero_kv_retrieve(self._h, layer, dtype.itemsize, k.ctypes.data, v.ctypes.data)
        if rc < 0:
            raise OracleError(rc)
        n = rc * self.num_kv_heads * self.head_dim
        return k[:n], v[:n]

    def retrieve_decoded_turboquant(self, layer):
        n_max = self.max_seq_len * self.num_kv_heads * self.head_dim
        k = np.zeros(n_max, dtype=np.float32)
        v = np.zeros(n_max, dtype=np.float32)
        rc = lib().ero_kv_retrieve_decoded_turboquant(self._h, layer, _p(k, F32), _p(v, F32))
        if rc < 0:
            raise OracleError(rc)
        n = rc * self.num_kv_heads * self.head_dim
        return k[:n], v[:n]

    def turbo_rows(self, layer, is_value):
        """(codes [rows,w] u32, meta [rows,2] f32) views copied out of the split buffers."""
        bits = self.value_bits if is_value else self.key_bits
        w = lib().ero_tq_code_words_per_row(bits)
        rows = self.max_seq_len * self.num_kv_heads
        cp = lib().ero_kv_turbo_buffer(self._h, layer, int(is_value), 0)
        mp = lib().ero_kv_turbo_buffer(self._h, layer, int(is_value), 3)
        codes = np.ctypeslib.as_array(C.cast(cp, C.POINTER(U32)), shape=(rows, w)).copy()
        meta = np.ctypeslib.as_array(C.cast(mp, C.POINTER(F32)), shape=(rows, 2)).copy()
        return codes, meta

    def cache_params(self, layer):
        out = np.zeros(6, dtype=np.uint32)
        rc = lib().ero_kv_params(self._h, layer, _p(out, U32))
        if rc:
            raise OracleError(rc)
        return dict(zip(("maxSeqLen", "currentLen", "writePos", "numKVHeads", "headDim", "precision"),
                        (int(x) for x in out)))

    def reset(self):
        lib().ero_kv_reset(self._h)

    def advance_write_position(self, layer, count):
        lib().ero_kv_advance_write_position(self._h, layer, count)

    def set_position(self, position):
        lib().ero_kv_set_position(self._h, position)


# ----------------------------------------------------------------------------- whole decode step

def decode_step_f16(q, k, v, k_cache, v_cache, pos, theta, scaling=1.0, threads=1):
    """One layer.  q [H,D], k/v [Hkv,D] float32; caches [T,Hkv,D] uint16, updated in place at slot pos.
    Returns (out [H,D], q_rot [H,D])."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    h, d = q.shape
    hkv = k.shape[0]
    assert k_cache.dtype == np.uint16 and k_cache.flags.c_contiguous and v_cache.flags.c_contiguous
    out = np.empty_like(q)
    q_rot = np.empty_like(q)
    lib().ero_decode_step_f16(_p(q, F32), _p(k, F32), _p(v, F32), _p(k_cache, U16), _p(v_cache, U16), _p(out, F32),
                              _p(q_rot, F32), pos, h, hkv, d, theta, scaling, threads)
    return out, q_rot


def decode_step_turboquant(q, k, v, k_codes, k_norm, k_bits, v_codes, v_norm, v_bits, pos, theta, scaling=1.0,
                           norm_fp16=False, threads=1):
    """q [H,128], k/v [Hkv,128]; codes [T*Hkv, w] u32 and norms [T*Hkv] f32 updated in place at row pos*Hkv+h."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    h = q.shape[0]
    hkv = k.shape[0]
    out = np.empty_like(q)
    lib().ero_decode_step_turboquant(_p(q, F32), _p(k, F32), _p(v, F32), _p(k_codes, U32), _p(k_norm, F32), k_bits,
                                     _p(v_codes, U32), _p(v_norm, F32), v_bits, _p(out, F32), pos, h, hkv, theta,
                                     scaling, int(norm_fp16), threads)
    return out
