"""Pin the CPU oracle against every literal the reference's own tests hold for the path
(tests/golden/reference_literals.json), plus analytically derived known answers."""
import json
import math
import os

import numpy as np
import pytest

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_literals.json")))


def test_kv_append_single_step(oracle):
    g = GOLD["kv_append_single_step"]
    c = oracle.OracleKVCache(g["max_seq_len"], g["num_layers"], g["num_kv_heads"], g["head_dim"], oracle.PREC_F32)
    c.append(0, g["keys"], g["values"])
    assert c.current_length == g["current_length"]
    k, v = c.retrieve(0, np.float32)
    assert k.tolist() == g["keys"] and v.tolist() == g["values"]


def test_kv_append_multiple_steps(oracle):
    g = GOLD["kv_append_multiple_steps"]
    c = oracle.OracleKVCache(g["max_seq_len"], 1, g["num_kv_heads"], g["head_dim"], oracle.PREC_F32)
    for k, v in g["appends"]:
        c.append(0, k, v)
    assert c.current_length == g["current_length"]
    k, v = c.retrieve(0, np.float32)
    assert k.tolist() == g["keys"] and v.tolist() == g["values"]


def test_kv_wrap_around(oracle):
    g = GOLD["kv_wrap_around"]
    c = oracle.OracleKVCache(g["max_seq_len"], 1, g["num_kv_heads"], g["head_dim"], oracle.PREC_F32)
    for i in range(4):
        c.append(0, [i, i + 0.5], [i * 10, i * 10 + 5])
    c.append(0, *g["final_append"])
    assert c.current_length == g["current_length"]
    k, _ = c.retrieve(0, np.float32)
    for idx, val in g["keys_expect"].items():
        assert k[int(idx)] == val
    p = c.cache_params(0)
    assert p["writePos"] == 1 and p["currentLen"] == 4 and p["maxSeqLen"] == 4


def test_kv_multi_layer_and_reset(oracle):
    g = GOLD["kv_multi_layer"]
    c = oracle.OracleKVCache(g["max_seq_len"], g["num_layers"], g["num_kv_heads"], g["head_dim"], oracle.PREC_F32)
    for layer, (k, v) in enumerate(g["appends"]):
        c.append(layer, k, v)
    assert c.retrieve(0, np.float32)[0].tolist() == g["keys0"]
    assert c.retrieve(1, np.float32)[0].tolist() == g["keys1"]
    c.reset()
    assert c.current_length == 0


def test_kv_float16_and_type_errors(oracle):
    g = GOLD["kv_float16"]
    c = oracle.OracleKVCache(g["max_seq_len"], 1, g["num_kv_heads"], g["head_dim"], oracle.PREC_F16)
    k16 = np.array(g["keys"], dtype=np.float16).view(np.uint16)
    v16 = np.array(g["values"], dtype=np.float16).view(np.uint16)
    c.append_f16(0, k16, v16)
    assert c.current_length == 1
    k, v = c.retrieve(0, np.uint16)
    assert k.view(np.float16).tolist() == g["keys"] and v.view(np.float16).tolist() == g["values"]
    # KVCacheTests.swift:177-197: Float16 cache retrieved as Float -> precisionMismatch
    with pytest.raises(oracle.OracleError) as e:
        c.retrieve(0, np.float32)
    assert e.value.code == -3
    # KVCacheTests.swift:199-219: invalid layer
    with pytest.raises(oracle.OracleError) as e:
        c.retrieve(1, np.uint16)
    assert e.value.code == -2


def test_turboquant_layout_words(oracle):
    L = oracle.lib()
    import ctypes as C
    for name, p in GOLD["turboquant_layout_words"]["presets"].items():
        cw, bw, sw = C.c_int(), C.c_int(), C.c_int()
        L.ero_tq_layout_words(p["regular_bits"], p["high_bits"], p["high_count"], C.byref(cw), C.byref(bw), C.byref(sw))
        assert cw.value == p["code_words"], name
        if "base_words" in p:
            assert bw.value == p["base_words"], name
        if "sideband_words" in p:
            assert sw.value == p["sideband_words"], name
    assert L.ero_tq_code_words_per_row(3) == 12 and L.ero_tq_code_words_per_row(4) == 16
    # bytesPerRow ordering asserted at TurboQuantReferenceTests.swift:139-140
    assert L.ero_tq_bytes_per_row(3) < L.ero_tq_bytes_per_row(4)
    assert L.ero_tq_bytes_per_row(3) == 88 and L.ero_tq_bytes_per_row(4) == 104


def test_hadamard_round_trip(oracle):
    g = GOLD["hadamard_round_trip"]
    x = np.array([float(i % 11) - 5.0 for i in range(128)], dtype=np.float32)
    rec = oracle.tq_inverse(oracle.tq_forward(x))
    assert np.max(np.abs(rec - x)) < g["tolerance"]


def test_split_plane_pack_round_trip(oracle):
    g = GOLD["split_plane_pack"]
    mask = np.array([i % 4 == 0 for i in range(128)], dtype=np.uint8)
    codes = np.array([(i // 4) % 8 if mask[i] else i % 4 for i in range(128)], dtype=np.uint8)
    import ctypes as C
    words = np.zeros(32, dtype=np.uint32)
    L = oracle.lib()
    n = L.ero_tq_pack_codes_split(codes.ctypes.data_as(C.POINTER(C.c_uint8)), mask.ctypes.data_as(C.POINTER(C.c_uint8)),
                                  128, g["regular_bits"], g["high_bits"], words.ctypes.data_as(C.POINTER(C.c_uint32)))
    assert n == g["packed_words"]
    back = np.zeros(128, dtype=np.uint8)
    L.ero_tq_unpack_codes_split(words.ctypes.data_as(C.POINTER(C.c_uint32)), n, mask.ctypes.data_as(C.POINTER(C.c_uint8)),
                                128, g["regular_bits"], g["high_bits"], back.ctypes.data_as(C.POINTER(C.c_uint8)))
    assert back.tolist() == codes.tolist()


def test_rope_known_values(oracle):
    g = GOLD["rope_known_values"]
    x = np.array(g["input"], dtype=np.float32).reshape(g["seq_len"], g["num_heads"], g["head_dim"])
    out = oracle.rope_neox(x, g["start_pos"], g["theta"], interleaved=True).ravel()
    assert abs(out[0]) < g["tolerance"] and abs(out[1]) < g["tolerance"]
    assert abs(out[2] - math.cos(1.0)) < g["tolerance"] and abs(out[3] - math.sin(1.0)) < g["tolerance"]
    # head_dim 2 has a single pair, so the NeoX pairing (d, d+1) coincides with the interleaved one
    out2 = oracle.rope_neox(x, g["start_pos"], g["theta"]).ravel()
    assert np.array_equal(out, out2)


def test_codebooks_monotonic(oracle):
    # TurboQuantReferenceTests.swift:33-39
    L = oracle.lib()
    for bits in (2, 3, 4):
        cent = [L.ero_tq_centroid(bits, i) for i in range(1 << bits)]
        thr = [L.ero_tq_threshold(bits, i) for i in range((1 << bits) - 1)]
        assert cent == sorted(cent) and thr == sorted(thr)


# ----------------------------------------------------------------------- analytically derived known answers

def test_forward_scale_bits(oracle):
    # 1/sqrt(Float(128)) in Float (TurboQuant.swift:877) and the shader literal 0.08838834764831845f
    # (TurboQuant.metal:357) are the same float, bits 0x3DB504F3.
    s = np.float32(oracle.lib().ero_tq_forward_scale())
    assert s.view(np.uint32) == 0x3DB504F3
    assert np.float32(0.08838834764831845).view(np.uint32) == 0x3DB504F3


def test_encode_unit_vector_known_answer(oracle):
    """x = a*e_j: normalized = e_j, rotated[d] = s1[j]*H[d][j]*s2[d]/sqrt(128) with H[d][j] = (-1)^popcount(d&j),
    i.e. +-0.0883883.  4-bit: 0.079142 <= 0.0883883 < 0.103361 -> code 13 (+) / 2 (-);
    3-bit: 0.0435885 <= 0.0883883 < 0.0917745 -> code 5 (+) / 2 (-) ; every centroid has the same magnitude so the stored norm is
    a / (|c| * sqrt(128))."""
    L = oracle.lib()
    for j in (0, 5, 77):
        x = np.zeros(128, dtype=np.float32)
        x[j] = 3.0
        sgn = np.array([L.ero_tq_sign(1, j) * L.ero_tq_sign(2, d) * (-1.0) ** bin(d & j).count("1") for d in range(128)])
        for bits, pos_code, neg_code in ((4, 13, 2), (3, 5, 2)):
            enc = oracle.tq_encode(x, bits)
            codes = oracle.tq_unpack_codes(enc["codes"], bits)
            want = np.where(sgn > 0, pos_code, neg_code)
            assert codes.tolist() == want.tolist()
            c = abs(L.ero_tq_centroid(bits, pos_code))
            assert abs(enc["row_norm"] - 3.0 / (c * math.sqrt(128.0))) < 1e-4
            assert enc["residual_norm"] == 0 and not enc["signs"].any() and not enc["mask"].any()
            dec = oracle.tq_decode(enc["codes"], bits, enc["row_norm"])
            assert abs(dec[j] - 3.0) < 1e-4 and np.max(np.abs(np.delete(dec, j))) < 1e-4


def test_encode_zero_row(oracle):
    # TurboQuant.swift:1018-1028: rowNorm == 0 -> all-zero row
    enc = oracle.tq_encode(np.zeros(128, dtype=np.float32), 4)
    assert not enc["codes"].any() and enc["row_norm"] == 0


def test_bit_packing_layout(oracle):
    # code i occupies bits [3i, 3i+3) of the little-endian word stream (TurboQuant.swift:1554-1573)
    codes = np.arange(128, dtype=np.uint8) % 8
    words = oracle.tq_pack_codes(codes, 3)
    assert words.size == 12
    big = 0
    for i, c in enumerate(codes.tolist()):
        big |= c << (3 * i)
    assert [int(w) for w in words] == [(big >> (32 * w)) & 0xFFFFFFFF for w in range(12)]
    assert oracle.tq_unpack_codes(words, 3).tolist() == codes.tolist()
    words4 = oracle.tq_pack_codes(np.arange(128, dtype=np.uint8) % 16, 4)
    assert int(words4[0]) == 0x76543210 and words4.size == 16


def test_threshold_rule_edges(oracle):
    # equality goes to the upper bin; NaN falls through to the last code (TurboQuant.swift:692-697)
    L = oracle.lib()
    assert L.ero_tq_code_for(0.0, 4) == 8 and L.ero_tq_code_for(-0.0, 4) == 8
    assert L.ero_tq_code_for(np.float32(-0.145560), 4) == 1
    assert L.ero_tq_code_for(float("nan"), 3) == 7
    assert L.ero_tq_code_for(1e9, 3) == 7 and L.ero_tq_code_for(-1e9, 3) == 0


def test_half_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 100, 70000)])
    x = np.concatenate([x, np.array([0, -0.0, 65504, 65519.99, 65520, np.inf, -np.inf, 2.0 ** -24, 2.0 ** -25,
                                     2.0 ** -25 * 1.0001, 6.1e-5], dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = oracle.f32_to_f16_bits(x)
    assert np.array_equal(got, want)
    allh = np.arange(65536, dtype=np.uint16)
    f = oracle.f16_bits_to_f32(allh)
    ref = allh.view(np.float16).astype(np.float32)
    ok = np.isnan(ref) | (f == ref)
    assert ok.all()


def test_gqa_matches_numpy_softmax(oracle):
    g = GOLD["gqa_f16kv_tolerance"]
    rng = np.random.default_rng(3)
    S, D, H, Hkv = g["seq_len"], g["head_dim"], g["num_heads"], g["num_kv_heads"]
    q = rng.uniform(-0.25, 0.25, (S, H, D)).astype(np.float32)
    k = rng.uniform(-0.25, 0.25, (S, Hkv, D)).astype(np.float32)
    v = rng.uniform(-0.25, 0.25, (S, Hkv, D)).astype(np.float32)
    out = oracle.gqa_f32(q, k, v, causal=True)
    ref = np.zeros_like(out, dtype=np.float64)
    for h in range(H):
        kv = h // (H // Hkv)
        s = (q[:, h].astype(np.float64) @ k[:, kv].astype(np.float64).T) / math.sqrt(D)
        s = np.where(np.tril(np.ones((S, S), dtype=bool)), s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        ref[:, h] = p @ v[:, kv].astype(np.float64)
    assert np.max(np.abs(out - ref)) < 1e-5
    out16 = oracle.gqa_f16kv(q, k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16))
    assert np.max(np.abs(out16 - out)) < g["abs_tolerance"]


def test_turbo_attention_consistency(oracle):
    """score path (approximateScoreTerms) and decoded-value path (approximateDecode) agree with the fused
    rotated-space attention restatement."""
    rng = np.random.default_rng(5)
    H, Hkv, T = 4, 2, 37
    q = rng.standard_normal((H, 128)).astype(np.float32)
    k = rng.standard_normal((T * Hkv, 128)).astype(np.float32)
    v = rng.standard_normal((T * Hkv, 128)).astype(np.float32)
    kc, kn = oracle.tq_encode_rows(k, 4)
    vc, vn = oracle.tq_encode_rows(v, 3)
    out = oracle.tq_attention_decode(q, kc, kn, 4, vc, vn, 3, Hkv, T)
    scale = np.float32(1.0 / math.sqrt(128.0))
    for h in range(H):
        kv = h // (H // Hkv)
        s = np.array([oracle.tq_score(q[h], kc[t * Hkv + kv], 4, kn[t * Hkv + kv], scale)[0] for t in range(T)])
        p = np.exp(s - s.max())
        p /= p.sum()
        dec = np.stack([oracle.tq_decode(vc[t * Hkv + kv], 3, vn[t * Hkv + kv]) for t in range(T)])
        assert np.max(np.abs(p @ dec - out[h])) < 1e-4
    # quantisation error of the whole thing stays in the range the reference tolerates (0.25-0.30 abs)
    dense = oracle.gqa_f32(q[None], k.reshape(T, Hkv, 128), v.reshape(T, Hkv, 128), causal=False)[0]
    assert np.max(np.abs(dense - out)) < 0.3


def test_turbo_cache_roundtrip(oracle):
    # KVCacheTests.swift:221-240 (finite decode) with the fixed presets; signal from :267-272
    c = oracle.OracleKVCache(8, 1, 2, 128, oracle.PREC_TURBO_V2, key_bits=4, value_bits=3)
    sig = lambda s: np.array([(math.sin(x * 0.17) + math.cos(x * 0.07) * 0.5) * s for x in range(128)], dtype=np.float32)
    keys = np.concatenate([sig(1.0), sig(0.7)])
    values = np.concatenate([sig(0.5), sig(1.2)])
    c.append(0, keys, values)
    dk, dv = c.retrieve_decoded_turboquant(0)
    assert dk.size == keys.size and np.isfinite(dk).all() and np.isfinite(dv).all()
    # Lloyd-Max distortion of a Gaussian source: ~0.0095 (4-bit) / ~0.0345 (3-bit) of the variance
    assert np.linalg.norm(dk - keys) / np.linalg.norm(keys) < 0.13
    assert np.linalg.norm(dv - values) / np.linalg.norm(values) < 0.24
    with pytest.raises(oracle.OracleError) as e:
        c.retrieve(0, np.float32)
    assert e.value.code == -5


def test_splitk_merge_equals_single_pass(oracle):
    rng = np.random.default_rng(7)
    T, D = 50, 128
    s = rng.standard_normal(T).astype(np.float32) * 3
    v = rng.standard_normal((T, D)).astype(np.float32)
    p = np.exp(s - s.max())
    ref = (p / p.sum()) @ v
    parts = [(0, 13), (13, 14), (14, 50)]
    pm = [s[a:b].max() for a, b in parts]
    ps = [np.exp(s[a:b] - m).sum() for (a, b), m in zip(parts, pm)]
    pa = [np.exp(s[a:b] - m) @ v[a:b] for (a, b), m in zip(parts, pm)]
    out = oracle.splitk_merge(pm, ps, np.stack(pa))
    assert np.max(np.abs(out - ref)) < 1e-5


# ------------------------------------------------------------------------------------------------ q8_0 rows

def test_q8_0_block_known_answers(oracle):
    """encodeQ8Row / decodeQ8Row (KVCache.swift:1007-1057) on inputs whose answers follow from the rule itself: the test
    pattern of the reference's own block test (DequantQ8_0Tests.swift:52-54: values i * 0.1 - 1.6), zeros, and a tie."""
    x = np.zeros(128, np.float32)
    x[:32] = np.arange(32, dtype=np.float32) * np.float32(0.1) - np.float32(1.6)
    blocks = oracle.q8_encode_rows(x)
    scale = np.float32(1.6) / np.float32(127.0)
    assert blocks[:2].view(np.float16)[0] == np.float16(scale)
    want = np.clip(np.sign(x[:32] / scale) * np.floor(np.abs(x[:32] / scale) + np.float32(0.5)), -128, 127).astype(np.int8)
    assert np.array_equal(blocks[2:34].view(np.int8), want)
    assert want[0] == -127 and want[16] == 0 and want[31] == 119
    assert not blocks[34:].any()                         # all-zero blocks: scale 0, codes 0
    dec = oracle.q8_decode_rows(blocks)
    assert np.array_equal(dec[:32], np.float32(np.float16(scale)) * want.astype(np.float32))
    # round half away from zero on an exact tie: max 127 -> scale 1, 0.5 -> 1, -0.5 -> -1, 2.5 -> 3
    y = np.zeros(128, np.float32)
    y[:4] = [127.0, 0.5, -0.5, 2.5]
    q = oracle.q8_encode_rows(y)[2:6].view(np.int8)
    assert list(q) == [127, 1, -1, 3]


def test_q8_0_attention_matches_dequantised_float_attention(oracle):
    rng = np.random.Generator(np.random.PCG64(77))
    T, H, Hkv = 37, 4, 2
    k = rng.standard_normal((T, Hkv, 128), dtype=np.float32)
    v = rng.standard_normal((T, Hkv, 128), dtype=np.float32)
    q = rng.standard_normal((3, H, 128), dtype=np.float32)
    k8, v8 = oracle.q8_encode_rows(k), oracle.q8_encode_rows(v)
    got = oracle.gqa_q8kv(q, k8, v8, causal=True, q_offset=T - 3)
    want = oracle.gqa_f32(q, oracle.q8_decode_rows(k8), oracle.q8_decode_rows(v8), causal=True, q_offset=T - 3)
    assert np.array_equal(got, want)
    assert np.max(np.abs(oracle.q8_decode_rows(k8) - k)) < 0.02      # |x| <= ~4.5, step = max/127


def _windowed_inputs(num_heads, num_kv_heads, head_dim, capacity, mods):
    """The generated inputs of the reference's windowed-attention tests (Gemma4DecodeKernelTests.swift:344-346, 389-391)."""
    (qm, qo, qd), (km, ko, kd), (vm, vo, vd) = mods
    q = np.array([((i % qm) - qo) / qd for i in range(num_heads * head_dim)], np.float32).reshape(num_heads, head_dim)
    k = np.array([((i % km) - ko) / kd for i in range(capacity * num_kv_heads * head_dim)], np.float32)
    v = np.array([((i % vm) - vo) / vd for i in range(capacity * num_kv_heads * head_dim)], np.float32)
    shape = (capacity, num_kv_heads, head_dim)
    return q, k.astype(np.float16).view(np.uint16).reshape(shape), v.astype(np.float16).view(np.uint16).reshape(shape)


@pytest.mark.parametrize("head_dim,capacity,kv_start,kv_count,scale,mods", [
    (256, 8, 5, 6, None, ((13, 6, 17.0), (11, 5, 19.0), (7, 3, 11.0))),    # windowedF16KVGQA: wraps the 8-slot ring
    (512, 8, 5, 6, None, ((13, 6, 17.0), (11, 5, 19.0), (7, 3, 11.0))),
    (256, 4, 0, 4, 1.0, ((17, 8, 11.0), (13, 6, 13.0), (7, 3, 7.0))),      # windowedF16KVGQAUnscaledAttention
    (128, 8, 5, 6, None, ((13, 6, 17.0), (11, 5, 19.0), (7, 3, 11.0))),    # the head size this backend's kernels are built for
])
def test_windowed_gqa_equals_attention_over_the_gathered_ring_rows(oracle, head_dim, capacity, kv_start, kv_count, scale, mods):
    """gemma4_decode_gqa_f16kv_windowed on the reference tests' shapes and generated inputs: the ring range is a row
    gather, so the result must equal the plain fp16-KV attention restatement over the gathered rows (within the fp32
    noise of the two summation orders); the test's own CPU routine is the same two-pass form."""
    q, k16, v16 = _windowed_inputs(8, 2, head_dim, capacity, mods)
    got = oracle.gqa_f16kv_windowed(q, k16, v16, kv_start, kv_count, scale)
    rows = [(kv_start + i) % capacity for i in range(kv_count)]
    s = 1.0 / math.sqrt(head_dim) if scale is None else scale
    # gqa_f16kv scales by 1/sqrt(D): fold the requested scale into q
    want = oracle.gqa_f16kv((q * (s * math.sqrt(head_dim)))[None], k16[rows], v16[rows], causal=False)[0]
    assert np.abs(got - want).max() < 2e-6
    kf, vf = k16.view(np.float16).astype(np.float64)[rows], v16.view(np.float16).astype(np.float64)[rows]
    for head in (0, 3, 7):
        sc = kf[:, head // 4] @ q[head].astype(np.float64) * s
        w = np.exp(sc - sc.max())
        assert np.abs(got[head] - (w / w.sum()) @ vf[:, head // 4]).max() < 2e-6


def test_windowed_gqa_empty_range_is_zero(oracle):
    q, k16, v16 = _windowed_inputs(8, 2, 128, 8, ((13, 6, 17.0), (11, 5, 19.0), (7, 3, 11.0)))
    assert not oracle.gqa_f16kv_windowed(q, k16, v16, 3, 0).any()


# ---- presets with high-precision channels and a QJL residual (balanced, aggressive) ----

def _make_signal():
    """makeSignal of the reference's encoder tests (TurboQuantReferenceTests.swift:331-336)."""
    i = np.arange(128, dtype=np.float32)
    return (np.sin(i * np.float32(0.17)) + np.cos(i * np.float32(0.07)) * np.float32(0.5)).astype(np.float32)


def test_outlier_preset_layout_literals(oracle):
    # layoutMatchesExpectedRowSize (TurboQuantReferenceTests.swift:112-143): aggressive 8 + 1 words, balanced 12 + 2
    assert oracle.lib().ero_tq_preset_code_words(2, 3, 32) == 9
    assert oracle.lib().ero_tq_preset_code_words(3, 5, 32) == 14


@pytest.mark.parametrize("preset", ["aggressive", "balanced"])
def test_outlier_preset_encoder_properties(oracle, preset):
    """aggressiveEncodingIsDeterministic / approximateDecodeProducesFiniteValues (TurboQuantReferenceTests.swift:41-85): the
    properties the reference asserts on makeSignal(), plus the structure of the row (32 selected channels, the selected
    ones are the largest by the selection rule, split-plane round trip of the codes)."""
    x = _make_signal()
    rb, hb, cnt = oracle.PRESETS[preset]
    for benefit in (False, True):
        a = oracle.tq_encode_preset(x, preset, benefit)
        b = oracle.tq_encode_preset(x, preset, benefit)
        assert all(np.array_equal(u, v) for u, v in zip(a, b))
        codes, signs, mask, row_norm, res_norm = a
        assert codes.size > 0 and signs.size == 4 and mask.size == 4
        bits = np.unpackbits(mask.view(np.uint8), bitorder="little")
        assert bits.sum() == cnt
        acc = np.float32(0)
        for t in x:                                      # rowNorm: Float sum of squares accumulated left to right
            acc = np.float32(acc + np.float32(t * t))
        assert row_norm == np.sqrt(acc)                  # the residual path stores the plain norm, not the corrected one
        assert 0 < res_norm < 1
        dec = oracle.tq_decode_preset(codes, signs, mask, preset, row_norm, res_norm)
        assert dec.shape == x.shape and np.isfinite(dec).all()
        assert float(np.mean((x - dec) ** 2)) < 10          # the reference's bound; the encoder actually reaches ~0.03
        # the mask is exactly the top-32 of the selection score over the rotated, normalised row
        rot = oracle.tq_forward(x / row_norm)
        want = oracle.tq_topk_mask(rot, cnt, rb, hb, benefit)
        assert np.array_equal(bits.astype(bool), want)
        if not benefit:
            mag = np.abs(rot)
            assert mag[want].min() >= mag[~want].max()
    # an all-zero row encodes to an all-zero row (TurboQuant.swift:1018-1028)
    z = oracle.tq_encode_preset(np.zeros(128, np.float32), preset)
    assert not z[0].any() and not z[1].any() and not z[2].any() and z[3] == 0 and z[4] == 0


def test_topk_ties_keep_channel_order(oracle):
    v = np.zeros(128, np.float32)
    v[[5, 9, 70, 100]] = [0.5, -0.5, 0.5, 0.25]          # three equal magnitudes, then a smaller one
    m = oracle.tq_topk_mask(v, 2, 2, 3)
    assert np.nonzero(m)[0].tolist() == [5, 9]             # equal scores: the lower channel wins
    m = oracle.tq_topk_mask(v, 4, 2, 3)
    assert np.nonzero(m)[0].tolist() == [5, 9, 70, 100]
