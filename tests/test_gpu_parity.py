"""GPU parity tests: every check drives the CUDA kernels through the C ABI (edgerunner_b200 -> liber_kv.so) and
compares with the CPU oracle on the same seeded inputs.

Bars: bit-exact for cache contents, packed TurboQuant codes, norms stored as float32 and block-table gathers;
2e-3 max relative error for attention outputs (fp32 accumulate), the bound named by the benchmark contract and
by the reference's own fp16-KV test (Tests/EdgeRunnerMetalTests/GQATests.swift:431-433).
"""
import ctypes as C
import json
import math
import os

import numpy as np
import pytest

from helpers import THETA_QWEN3, attention_err, max_rel_err, normal_f16, outlier_channels, rng_for

pytestmark = pytest.mark.gpu
TOL = 2e-3
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_literals.json")))


@pytest.fixture(scope="module")
def er():
    import edgerunner_b200 as er
    assert er.lib().er_device_count() > 0
    return er


@pytest.fixture(scope="module")
def torch():
    import torch
    return torch


def dev(torch, a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


# --------------------------------------------------------------------------------------------- KVCache host surface

def test_kvcache_literals_through_abi(er):
    g = GOLD["kv_append_single_step"]
    c = er.KVCache(g["max_seq_len"], g["num_layers"], g["num_kv_heads"], g["head_dim"], er.Precision.float32)
    c.append(0, g["keys"], g["values"])
    assert c.current_length == 1
    k, v = c.retrieve(0, np.float32)
    assert k.tolist() == g["keys"] and v.tolist() == g["values"]

    g = GOLD["kv_wrap_around"]
    for layout in (er.Layout.token_major, er.Layout.head_major):
        c = er.KVCache(g["max_seq_len"], 1, g["num_kv_heads"], g["head_dim"], er.Precision.float32, layout=layout)
        for i in range(4):
            c.append(0, [i, i + 0.5], [i * 10, i * 10 + 5])
        c.append(0, *g["final_append"])
        assert c.current_length == 4
        k, v = c.retrieve(0, np.float32)
        for idx, val in g["keys_expect"].items():
            assert k[int(idx)] == val
        assert v.tolist() == [10, 15, 20, 25, 30, 35, 990, 995]
        p = c.cache_params(0)
        assert (p.maxSeqLen, p.currentLen, p.writePos, p.numKVHeads, p.headDim, p.precision) == (4, 4, 1, 1, 2, 0)

    g = GOLD["kv_multi_layer"]
    c = er.KVCache(g["max_seq_len"], g["num_layers"], g["num_kv_heads"], g["head_dim"], er.Precision.float32)
    for layer, (k, v) in enumerate(g["appends"]):
        c.append(layer, k, v)
    assert c.retrieve(0, np.float32)[0].tolist() == g["keys0"] and c.retrieve(1, np.float32)[0].tolist() == g["keys1"]
    c.reset()
    assert c.current_length == 0

    g = GOLD["kv_float16"]
    c = er.KVCache(g["max_seq_len"], 1, g["num_kv_heads"], g["head_dim"], er.Precision.float16)
    c.append_f16(0, g["keys"], g["values"])
    k, v = c.retrieve(0, np.float16)
    assert k.tolist() == g["keys"] and v.tolist() == g["values"]


def test_kvcache_error_cases(er):
    c = er.KVCache(8, 1, 1, 4, er.Precision.float16)
    c.append_f16(0, [1, 2, 3, 4], [5, 6, 7, 8])
    with pytest.raises(er.EdgeRunnerCUDAError) as e:       # KVCacheTests.swift:177-197
        c.retrieve(0, np.float32)
    assert e.value.name == "precisionMismatch"
    with pytest.raises(er.EdgeRunnerCUDAError) as e:       # KVCacheTests.swift:199-219
        c.device_buffers(1)
    assert e.value.name == "invalidLayer"
    with pytest.raises(er.EdgeRunnerCUDAError) as e:       # Float rows into a float16 cache (KVCache.swift:450-452)
        c.append(0, [1, 2, 3, 4], [5, 6, 7, 8])
    assert e.value.name == "precisionMismatch"
    with pytest.raises(er.EdgeRunnerCUDAError) as e:       # precondition(keys.count == layerElements) -> status, not a trap
        c.append_f16(0, [1, 2, 3], [5, 6, 7])
    assert e.value.name == "shape"
    t = er.KVCache(8, 1, 1, 128, er.Precision.turboquantV2)
    with pytest.raises(er.EdgeRunnerCUDAError) as e:       # KVCacheTests.swift:242-265
        t.metal_buffers(0)
    assert e.value.name == "compressedBufferAccessRequiresTurboQuantAPI"
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        t.retrieve(0, np.float32)
    assert e.value.name == "compressedRetrieveRequiresDecodedAPI"
    assert t.turboquant_buffers(0).key_row_bytes == 48
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        er.KVCache(8, 1, 1, 128, er.Precision.float8)
    assert e.value.name == "unsupportedStorage"
    b = er.KVCache(8, 1, 1, 128, er.Precision.turboQuantBalanced)      # presets with high-precision channels: TurboQuant accessors too
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        b.metal_buffers(0)
    assert e.value.name == "compressedBufferAccessRequiresTurboQuantAPI"
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        b.retrieve(0, np.float32)
    assert e.value.name == "compressedRetrieveRequiresDecodedAPI"


def test_set_position_and_advance(er):
    c = er.KVCache(16, 3, 1, 2, er.Precision.float32, max_batch=2)
    c.set_position(5)
    assert c.current_length == 5 and c.cache_params(2, 1).writePos == 5
    c.advance_write_position(1, 13, seq=0)
    assert c.total_written(1, 0) == 18 and c.total_written(1, 1) == 5
    p = c.cache_params(1, 0)
    assert (p.currentLen, p.writePos) == (16, 2)
    c.reset()
    assert c.current_length == 0


# --------------------------------------------------------------------------------------------- RoPE

def test_rope_known_values_and_oracle(er, oracle):
    g = GOLD["rope_known_values"]
    rk = er.RoPEKernel()
    out = rk.execute_neox(np.array(g["input"], dtype=np.float32), g["seq_len"], g["num_heads"], g["head_dim"],
                          start_pos=0, theta=g["theta"]).ravel()
    assert abs(out[0]) < 1e-5 and abs(out[1]) < 1e-5
    assert abs(out[2] - math.cos(1.0)) < 1e-5 and abs(out[3] - math.sin(1.0)) < 1e-5

    rng = rng_for(11)
    x = rng.standard_normal((7, 5, 128), dtype=np.float32)
    for theta, start, scaling, partial in ((1e6, 4090, 1.0, 1.0), (1e4, 0, 2.0, 0.25), (5e5, 131000, 1.0, 1.0)):
        want = oracle.rope_neox(x, start, theta, scaling, partial)
        got = rk.execute_neox(x, 7, 5, 128, start, theta, scaling, partial)
        assert np.array_equal(got.reshape(want.shape), want), (theta, start)
        want16 = oracle.rope_neox_to_f16(x, start, theta, scaling, partial)
        got16 = rk.execute_neox(x, 7, 5, 128, start, theta, scaling, partial, to_f16=True)
        assert np.array_equal(got16.view(np.uint16).reshape(want16.shape), want16)
    x = rng.standard_normal((3, 2, 64), dtype=np.float32)       # another head_dim
    assert np.array_equal(rk.execute_neox(x, 3, 2, 64, 17, 1e4).reshape(x.shape), oracle.rope_neox(x, 17, 1e4))


# --------------------------------------------------------------------------------------------- TurboQuant quantiser

def _signal(phase):
    # TurboQuantAttentionTests.swift:1472-1477
    x = np.arange(128, dtype=np.float32)
    return (np.sin(x * np.float32(0.15) + np.float32(phase)) + np.float32(0.35) * np.cos(x * np.float32(0.05) - np.float32(phase))).astype(np.float32)


def _quantizer_inputs():
    rng = rng_for(21)
    rows = [rng.standard_normal((600, 128), dtype=np.float32)]
    rows.append(normal_f16(rng, (300, 128)) * outlier_channels(rng, 128, 0.05))
    rows.append(np.stack([_signal(0.1 * i) for i in range(64)]))
    special = np.zeros((8, 128), dtype=np.float32)
    special[1, 5] = 3.0
    special[2] = 1e-20
    special[3] = 1e18
    special[4, :] = -2.5
    special[5, ::2] = 1.0
    special[6] = np.float32(np.nan)
    special[7, 0] = np.float32(np.inf)
    rows.append(special)
    return np.concatenate(rows).astype(np.float32)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_quantize_rows_bit_exact(er, oracle, bits):
    x = _quantizer_inputs()
    codes, signs, mask, meta = er.TurboQuantKernel().execute_quantize_rows(x, bits)
    want_codes, want_norm = oracle.tq_encode_rows(x, bits)
    assert np.array_equal(codes, want_codes)                       # codes ==   (TurboQuantAttentionTests.swift:760)
    assert not signs.any() and not mask.any()                      # mask / signs ==
    finite = np.isfinite(want_norm)
    assert np.array_equal(meta[finite, 0].view(np.uint32), want_norm[finite].view(np.uint32))   # rowNorm (< 1e-5 there)
    assert np.array_equal(np.isnan(meta[:, 0]), np.isnan(want_norm))
    assert not meta[:, 1].any()                                    # residualNorm == 0


@pytest.mark.parametrize("preset", ["balanced", "aggressive"])
@pytest.mark.parametrize("benefit", [False, True])
def test_quantize_rows_outlier_presets_bit_exact(er, oracle, preset, benefit):
    """turboquant_quantize_rows for the presets with 32 high-precision channels and a QJL residual (Shaders/TurboQuant.metal:
    562-709) against the CPU encoder (TurboQuantReferenceEncoder.encode, TurboQuant.swift:1003-1100): packed split-plane
    codes, outlier mask, residual signs and both norms bit for bit, with the keys' (.magnitude) and the values'
    (.quantizationBenefit) selection rule.  Finite rows (random, outlier channels, closed-form signals, ties, zero rows)."""
    x = _quantizer_inputs()[:-2]                                   # the NaN / inf rows have no defined selection order
    ties = np.zeros((4, 128), dtype=np.float32)
    ties[0, [5, 9, 70, 100]] = [0.5, -0.5, 0.5, 0.25]
    ties[1, :] = 1.0                                               # every score equal: channels 0..31 are selected
    ties[2, ::3] = -2.0
    ties[3, 64:] = np.linspace(1, 2, 64, dtype=np.float32)
    x = np.concatenate([x, ties])
    codes, signs, mask, meta = er.TurboQuantKernel().execute_quantize_rows_preset(x, preset, benefit)
    wc, ws, wm, wmeta = oracle.tq_encode_rows_preset(x, preset, benefit)
    assert np.array_equal(mask, wm)
    assert np.array_equal(codes, wc)
    assert np.array_equal(signs, ws)
    assert np.array_equal(meta.view(np.uint32), wmeta.view(np.uint32))       # (rowNorm, residualNorm)
    assert (np.unpackbits(mask[x.any(axis=1)].view(np.uint8), axis=1).sum(axis=1) == 32).all()


def test_quantize_rows_stride_and_base(er, oracle, torch):
    rng = rng_for(22)
    x = rng.standard_normal((37, 160), dtype=np.float32)           # source_row_stride 160 > 128
    base = 5
    codes = torch.zeros((64, 16), dtype=torch.int32, device="cuda")
    meta = torch.zeros((64, 2), dtype=torch.float32, device="cuda")
    signs = torch.ones((64, 4), dtype=torch.int32, device="cuda")
    mask = torch.ones((64, 4), dtype=torch.int32, device="cuda")
    er.TurboQuantKernel().encode_quantize_rows(dev(torch, x), 37, 160, base, 4, codes, signs, mask, meta)
    torch.cuda.synchronize()
    want_codes, want_norm = oracle.tq_encode_rows(x[:, :128], 4)
    got = codes.cpu().numpy().view(np.uint32)
    assert np.array_equal(got[base:base + 37], want_codes) and not got[:base].any() and not got[base + 37:].any()
    assert np.array_equal(meta.cpu().numpy()[base:base + 37, 0], want_norm)
    assert not signs.cpu().numpy()[base:base + 37].any() and signs.cpu().numpy()[:base].all()


# --------------------------------------------------------------------------------------------- dense decode

def _oracle_dense_cache(oracle, K, V, theta):
    """K, V: [T, Hkv, D] float32 -> fp16 caches [T, Hkv, D] with K NeoX-rotated at its row position."""
    T = K.shape[0]
    kc = np.empty(K.shape, dtype=np.uint16)
    for t in range(T):
        kc[t] = oracle.rope_neox_to_f16(K[t:t + 1], t, theta)[0]
    return kc, oracle.f32_to_f16_bits(V)


KERNELS = [("persistent", 1), ("slim", 2)]       # er_kv_config.decode_kernel: both fp16 decode kernels run every dense case


def _run_dense_config(er, oracle, torch, layout, L, B, Hq, Hkv, ctx, steps, seed, theta=THETA_QWEN3, page_size=0,
                      ragged=False, max_seq_len=None, decode_kernel=0):
    D = 128
    rng = rng_for(seed)
    lens = [ctx] * B if not ragged else [int(x) for x in rng.integers(max(1, ctx // 8), ctx + 1, size=B)]
    max_len = max(lens) + steps
    T = max_seq_len or ((max_len + 15) // 16 * 16)
    kw = {}
    alloc = None
    if layout == er.Layout.paged:
        pages_per_seq = (T + page_size - 1) // page_size
        num_pages = pages_per_seq * B + 3
        kw = dict(page_size=page_size, num_pages=num_pages)
        alloc = er.BlockTableAllocator(num_pages, page_size, free_order=rng.permutation(num_pages))
    cache = er.KVCache(T, L, Hkv, D, er.Precision.float16, max_batch=B, layout=layout, decode_kernel=decode_kernel, **kw)
    if alloc:
        for b in range(B):
            cache.set_block_table(b, alloc.ensure(b, lens[b] + steps))
            assert cache.get_block_table(b) == alloc.block_table(b)
    sp = er.step_params(rope_theta=theta)
    okc = [[None] * B for _ in range(L)]
    ovc = [[None] * B for _ in range(L)]
    for l in range(L):
        for b in range(B):
            K = normal_f16(rng, (lens[b], Hkv, D))
            V = normal_f16(rng, (lens[b], Hkv, D))
            cache.write_rows(l, b, 0, lens[b], dev(torch, K), dev(torch, V), sp)
            kc, vc = _oracle_dense_cache(oracle, K, V, theta)
            okc[l][b] = np.concatenate([kc, np.zeros((steps, Hkv, D), np.uint16)])
            ovc[l][b] = np.concatenate([vc, np.zeros((steps, Hkv, D), np.uint16)])
    torch.cuda.synchronize()
    worst = 0.0
    for s in range(steps):
        q = normal_f16(rng, (L, B, Hq, D))
        k = normal_f16(rng, (L, B, Hkv, D))
        v = normal_f16(rng, (L, B, Hkv, D))
        out = torch.full((L, B, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
        torch.cuda.synchronize()
        assert cache.device_status() == 0
        got = out.cpu().numpy()
        for l in range(L):
            for b in range(B):
                want, _ = oracle.decode_step_f16(q[l, b], k[l, b], v[l, b], okc[l][b], ovc[l][b], lens[b] + s, theta, threads=8)
                worst = max(worst, max_rel_err(got[l, b], want))
                assert attention_err(got[l, b], want) < TOL
    assert worst < TOL, worst
    # cache contents, read back in logical order through the ABI, are bit-identical to the oracle's
    for l in range(L):
        for b in range(B):
            n = lens[b] + steps
            assert cache.total_written(l, b) == n
            gk, gv = cache.retrieve(l, np.float16, seq=b)
            assert np.array_equal(gk.view(np.uint16), okc[l][b][:n].ravel())
            assert np.array_equal(gv.view(np.uint16), ovc[l][b][:n].ravel())
    return worst


@pytest.mark.parametrize("kernel,dk", KERNELS)
def test_config0_single_layer_decode(er, oracle, torch, kernel, dk):
    """Configuration 0: Qwen3-0.6B-shaped layer, 16 q heads / 8 kv heads / head_dim 128, fp16 cache pre-filled with
    512 tokens, append 1 token, RoPE theta 1e6 at positions 0..512, output fp32 [16,128]."""
    for layout in (er.Layout.head_major, er.Layout.token_major):
        worst = _run_dense_config(er, oracle, torch, layout, L=1, B=1, Hq=16, Hkv=8, ctx=512, steps=1, seed=0, decode_kernel=dk)
        print("config0 %s %s kernel max rel err %.3e" % (layout.name, kernel, worst))


def test_config0_against_committed_golden(er, oracle, torch):
    """Same configuration against the committed fixture (tests/golden/config0_expected.npz, generated by
    tests/golden/make_config0.py from the oracle)."""
    path = os.path.join(os.path.dirname(__file__), "golden", "config0_expected.npz")
    gold = np.load(path)
    from golden.make_config0 import config0_inputs
    Q, K, V = config0_inputs()
    cache = er.KVCache(1024, 1, 8, 128, er.Precision.float16)
    sp = er.step_params(rope_theta=THETA_QWEN3)
    cache.write_rows(0, 0, 0, 512, dev(torch, K[:512]), dev(torch, V[:512]), sp)
    out = torch.empty((16, 128), dtype=torch.float32, device="cuda")
    cache.decode_step(dev(torch, Q), dev(torch, K[512]), dev(torch, V[512]), out, 16, sp)
    torch.cuda.synchronize()
    assert max_rel_err(out.cpu().numpy(), gold["out"]) < TOL
    gk, gv = cache.retrieve(0, np.float16)
    assert np.array_equal(gk.view(np.uint16).reshape(513, 8, 128)[[0, 1, 255, 511, 512]], gold["k_rows"])
    assert np.array_equal(gv.view(np.uint16).reshape(513, 8, 128)[[0, 1, 255, 511, 512]], gold["v_rows"])


@pytest.mark.parametrize("kernel,dk", KERNELS)
def test_multilayer_steps_all_layouts(er, oracle, torch, kernel, dk):
    """Configuration-1-shaped (several independent layers, consecutive decode steps) at a size the oracle finishes
    quickly, in every storage layout; odd context so tiles end ragged."""
    for layout, ps in ((er.Layout.head_major, 0), (er.Layout.token_major, 0), (er.Layout.paged, 16), (er.Layout.paged, 64)):
        _run_dense_config(er, oracle, torch, layout, L=3, B=1, Hq=16, Hkv=8, ctx=777, steps=3, seed=3, page_size=ps, decode_kernel=dk)


@pytest.mark.parametrize("kernel,dk", KERNELS)
def test_batched_ragged_paged_llama_shape(er, oracle, torch, kernel, dk):
    """Configuration-3-shaped: 32 q heads / 8 kv heads (group 4), 16-token pages, block tables a seeded random
    permutation of a shared pool, ragged context lengths."""
    _run_dense_config(er, oracle, torch, er.Layout.paged, L=2, B=5, Hq=32, Hkv=8, ctx=1500, steps=2, seed=2,
                      theta=5e5, page_size=16, ragged=True, decode_kernel=dk)


@pytest.mark.parametrize("layout,page_size", [("head_major", 0), ("token_major", 0), ("paged", 32)])
def test_group8_and_group4_tensor_core_policy(er, oracle, torch, layout, page_size):
    """GQA groups 4 and 8 on fp16 rows run both contractions on the tensor cores: ragged batches, several steps, every
    layout, contexts from a single row to several tiles."""
    lay = getattr(er.Layout, layout)
    for dk in (1, 0):      # group 8 exists in the persistent kernel only; 0 = automatic choice (slim for group 4 here)
        _run_dense_config(er, oracle, torch, lay, L=2, B=3, Hq=32, Hkv=4, ctx=900, steps=3, seed=40, page_size=page_size, ragged=True, decode_kernel=dk)
        _run_dense_config(er, oracle, torch, lay, L=1, B=2, Hq=16, Hkv=2, ctx=1, steps=19, seed=41, page_size=page_size, decode_kernel=dk)
        _run_dense_config(er, oracle, torch, lay, L=1, B=2, Hq=16, Hkv=4, ctx=3, steps=20, seed=42, page_size=page_size, decode_kernel=dk)


@pytest.mark.parametrize("layout,page_size", [("head_major", 0), ("token_major", 0), ("paged", 16)])
def test_group2_tensor_core_policy_on_long_rings(er, oracle, torch, layout, page_size):
    """GQA group 2 takes the tensor-core policy in the persistent kernel when the ring holds 16384 tokens or more (the scalar
    policy below that): ragged batches, several steps, every layout, contexts from a single row to several tiles."""
    lay = getattr(er.Layout, layout)
    _run_dense_config(er, oracle, torch, lay, L=2, B=3, Hq=16, Hkv=8, ctx=1100, steps=3, seed=50, page_size=page_size, ragged=True,
                      max_seq_len=16384, decode_kernel=1)
    _run_dense_config(er, oracle, torch, lay, L=1, B=2, Hq=4, Hkv=2, ctx=1, steps=19, seed=51, page_size=page_size, max_seq_len=16400,
                      decode_kernel=1)


@pytest.mark.parametrize("kernel,dk", KERNELS)
def test_group1_and_tiny_contexts(er, oracle, torch, kernel, dk):
    _run_dense_config(er, oracle, torch, er.Layout.head_major, L=1, B=3, Hq=4, Hkv=4, ctx=40, steps=2, seed=5, ragged=True, decode_kernel=dk)
    _run_dense_config(er, oracle, torch, er.Layout.token_major, L=2, B=2, Hq=8, Hkv=2, ctx=1, steps=18, seed=6, decode_kernel=dk)


@pytest.mark.parametrize("kernel,dk", KERNELS)
def test_ring_wrap_decode(er, oracle, torch, kernel, dk):
    """More decode steps than ring slots: new rows overwrite the oldest slots and attention covers the whole ring
    (reads ignore the wrap: softmax is order-independent and K carries its absolute RoPE position)."""
    D, Hq, Hkv, T = 128, 4, 2, 32
    rng = rng_for(9)
    cache = er.KVCache(T, 1, Hkv, D, er.Precision.float16, decode_kernel=dk)
    sp = er.step_params(rope_theta=1e4)
    kc = np.zeros((T, Hkv, D), np.uint16)
    vc = np.zeros((T, Hkv, D), np.uint16)
    for s in range(T + 9):
        q, k, v = normal_f16(rng, (Hq, D)), normal_f16(rng, (Hkv, D)), normal_f16(rng, (Hkv, D))
        out = torch.empty((Hq, D), dtype=torch.float32, device="cuda")
        cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
        torch.cuda.synchronize()
        slot = s % T
        q_rot = oracle.rope_neox(q[None], s, 1e4)[0]
        kc[slot] = oracle.rope_neox_to_f16(k[None], s, 1e4)[0]
        vc[slot] = oracle.f32_to_f16_bits(v)
        n = min(s + 1, T)
        want = oracle.gqa_f16kv(q_rot[None], kc[:n], vc[:n], causal=False)[0]
        assert max_rel_err(out.cpu().numpy(), want) < TOL
    p = cache.cache_params(0)
    assert (p.currentLen, p.writePos) == (T, 9)
    gk, _ = cache.retrieve(0, np.float16)          # logical order: oldest first
    order = [(9 + i) % T for i in range(T)]
    assert np.array_equal(gk.view(np.uint16).reshape(T, Hkv, D), kc[order])


def test_append_then_attention_split_calls(er, oracle, torch):
    """er_kv_append_rope_kv + er_kv_attention_decode(pending=1) + er_kv_advance == er_kv_decode_step."""
    rng = rng_for(12)
    L, B, Hq, Hkv, D, ctx = 2, 2, 8, 4, 128, 300
    for dk in (1, 2):
        caches = [er.KVCache(512, L, Hkv, D, er.Precision.float16, max_batch=B, decode_kernel=dk) for _ in range(2)]
        sp = er.step_params(rope_theta=1e6)
        for l in range(L):
            for b in range(B):
                K, V = normal_f16(rng, (ctx, Hkv, D)), normal_f16(rng, (ctx, Hkv, D))
                for c in caches:
                    c.write_rows(l, b, 0, ctx, dev(torch, K), dev(torch, V), sp)
        q, k, v = (dev(torch, normal_f16(rng, (L, B, h, D))) for h in (Hq, Hkv, Hkv))
        o1 = torch.empty((L, B, Hq, D), dtype=torch.float32, device="cuda")
        o2 = torch.empty_like(o1)
        caches[0].decode_step(q, k, v, o1, Hq, sp)
        caches[1].append_rope_kv(k, v, sp)
        caches[1].attention_decode(q, o2, Hq, sp, pending=1)
        caches[1].advance(1)
        torch.cuda.synchronize()
        assert torch.equal(o1, o2), dk
        assert caches[0].total_written(1, 1) == caches[1].total_written(1, 1) == ctx + 1


def test_decode_step_host_buffers(er, oracle, torch):
    rng = rng_for(13)
    L, B, Hq, Hkv, D, ctx = 2, 1, 16, 8, 128, 200
    c1 = er.KVCache(256, L, Hkv, D, er.Precision.float16)
    c2 = er.KVCache(256, L, Hkv, D, er.Precision.float16)
    sp = er.step_params(rope_theta=1e6)
    for l in range(L):
        K, V = normal_f16(rng, (ctx, Hkv, D)), normal_f16(rng, (ctx, Hkv, D))
        for c in (c1, c2):
            c.write_rows(l, 0, 0, ctx, dev(torch, K), dev(torch, V), sp)
    q, k, v = (normal_f16(rng, (L, B, h, D)) for h in (Hq, Hkv, Hkv))
    out_d = torch.empty((L, B, Hq, D), dtype=torch.float32, device="cuda")
    c1.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out_d, Hq, sp)
    hq, hk, hv = (torch.as_tensor(a).pin_memory() for a in (q, k, v))
    hout = torch.empty((L, B, Hq, D), dtype=torch.float32).pin_memory()
    c2.decode_step_host(hq, hk, hv, hout, Hq, sp)
    torch.cuda.synchronize()
    assert torch.equal(out_d.cpu(), hout)


@pytest.mark.parametrize("Hq,Hkv", [(16, 8), (32, 8), (8, 8)])
def test_decode_step_host_rows_pulled_by_the_kernel(er, torch, Hq, Hkv):
    """Host-buffer steps on the persistent fp16 kernel: with every buffer pinned the launch pulls its q / k / v rows out of
    host memory itself (no gather launch, no stream synchronisation; the last CTA reports to a host word).  Several steps
    re-use the SAME pinned buffers with new contents (a stale cached line would show), ragged batch, pages; outputs and
    cache rows must equal the device-buffer step's bit for bit.  A pageable output buffer takes the copy path instead."""
    rng = rng_for(113)
    L, B, D, ps = 3, 5, 128, 16
    lens = [700, 33, 1, 260, 415]
    T = 768
    pages = (T // ps) * B
    caches = []
    for _ in range(4):
        c = er.KVCache(T, L, Hkv, D, er.Precision.float16, max_batch=B, layout=er.Layout.paged, page_size=ps, num_pages=pages, decode_kernel=1)
        alloc = er.BlockTableAllocator(pages, ps, free_order=rng_for(5).permutation(pages))
        for b in range(B):
            c.set_block_table(b, alloc.ensure(b, T))
        caches.append(c)
    sp = er.step_params(rope_theta=1e6)
    for l in range(L):
        for b in range(B):
            K, V = normal_f16(rng, (lens[b], Hkv, D)), normal_f16(rng, (lens[b], Hkv, D))
            for c in caches:
                c.write_rows(l, b, 0, lens[b], dev(torch, K), dev(torch, V), sp)
    hq = torch.empty((L, B, Hq, D), dtype=torch.float32).pin_memory()
    hk = torch.empty((L, B, Hkv, D), dtype=torch.float32).pin_memory()
    hv = torch.empty((L, B, Hkv, D), dtype=torch.float32).pin_memory()
    hout = torch.empty((L, B, Hq, D), dtype=torch.float32).pin_memory()
    pageable_out = np.empty((L, B, Hq, D), dtype=np.float32)
    out_d = torch.empty((L, B, Hq, D), dtype=torch.float32, device="cuda")
    out_dev = torch.empty((L, B, Hq, D), dtype=torch.float32, device="cuda")
    launches = er.lib().er_kernel_launch_count
    for step in range(4):
        q, k, v = (normal_f16(rng, (L, B, h, D)) for h in (Hq, Hkv, Hkv))
        hq.copy_(torch.as_tensor(q)); hk.copy_(torch.as_tensor(k)); hv.copy_(torch.as_tensor(v))
        caches[0].decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out_d, Hq, sp)
        n0 = launches()
        hout.fill_(float("nan"))
        caches[1].decode_step_host(hq, hk, hv, hout, Hq, sp)      # returns with the rows in hout: no synchronize here
        got = hout.clone()
        assert launches() - n0 == 1                               # the decode launch alone
        caches[2].decode_step_host(hq, hk, hv, pageable_out, Hq, sp)
        n1 = launches()
        out_dev.fill_(float("nan"))
        caches[3].decode_step_host(hq, hk, hv, out_dev, Hq, sp)    # device output: enqueued only, rows pulled by the kernel
        assert launches() - n1 == 1
        torch.cuda.synchronize()
        assert torch.equal(out_d.cpu(), got), step
        assert np.array_equal(out_d.cpu().numpy(), pageable_out), step
        assert torch.equal(out_d, out_dev), step
    for c in caches[1:]:
        assert c.device_status() == 0
        for l in range(L):
            for b in range(B):
                assert c.total_written(l, b) == lens[b] + 4
                k0, v0 = caches[0].retrieve(l, np.float16, seq=b)
                k1, v1 = c.retrieve(l, np.float16, seq=b)
                assert np.array_equal(k0.view(np.uint16), k1.view(np.uint16)) and np.array_equal(v0.view(np.uint16), v1.view(np.uint16))


def test_gqa_kernel_operator_matches_cpu_gqa(er, oracle):
    """GQAKernel on raw fp16 K/V buffers (pipelineF16KV), prefill semantics: the reference's own test shape
    (GQATests.swift:365-434: S=16, D=128, 8 q / 2 kv heads, causal, inputs in [-0.25, 0.25], |err| < 2e-3) plus
    kvSeqLen != seqLen with a query offset (GQATests.swift:277-324)."""
    rng = rng_for(31)
    gk = er.GQAKernel()
    S, D, H, Hkv = 16, 128, 8, 2
    q = rng.uniform(-0.25, 0.25, (S, H, D)).astype(np.float32)
    k = rng.uniform(-0.25, 0.25, (S, Hkv, D)).astype(np.float32)
    v = rng.uniform(-0.25, 0.25, (S, Hkv, D)).astype(np.float32)
    got = gk.execute_f16kv(q, k, v, S, D, H, Hkv, causal=True)
    assert np.max(np.abs(got - oracle.gqa_f32(q, k, v, causal=True))) < GOLD["gqa_f16kv_tolerance"]["abs_tolerance"]
    k16, v16 = k.astype(np.float16), v.astype(np.float16)
    assert max_rel_err(got, oracle.gqa_f16kv(q, k16.view(np.uint16), v16.view(np.uint16), causal=True)) < TOL
    S, T, off = 3, 150, 147
    q = normal_f16(rng, (S, H, D))
    k16, v16 = normal_f16(rng, (T, Hkv, D)).astype(np.float16), normal_f16(rng, (T, Hkv, D)).astype(np.float16)
    got = gk.execute_f16kv(q, k16, v16, S, D, H, Hkv, causal=True, kv_seq_len=T, q_offset=off)
    want = oracle.gqa_f16kv(q, k16.view(np.uint16), v16.view(np.uint16), causal=True, q_offset=off)
    assert max_rel_err(got, want) < TOL
    got = gk.execute_f16kv(q, k16, v16, S, D, H, Hkv, causal=False, kv_seq_len=T)
    assert max_rel_err(got, oracle.gqa_f16kv(q, k16.view(np.uint16), v16.view(np.uint16), causal=False)) < TOL
    # a chunk large enough for the tcgen05 kernel (S * group >= 128), ragged against its 64-token tiles and 128-row CTAs
    S, T, off = 200, 333, 133
    q = normal_f16(rng, (S, H, D))
    k16, v16 = normal_f16(rng, (T, Hkv, D)).astype(np.float16), normal_f16(rng, (T, Hkv, D)).astype(np.float16)
    got = gk.execute_f16kv(q, k16, v16, S, D, H, Hkv, causal=True, kv_seq_len=T, q_offset=off)
    want = oracle.gqa_f16kv(q, k16.view(np.uint16), v16.view(np.uint16), causal=True, q_offset=off, threads=8)
    assert max_rel_err(got, want) < TOL
    got = gk.execute_f16kv(q, k16, v16, S, D, H, Hkv, causal=False, kv_seq_len=T)
    assert max_rel_err(got, oracle.gqa_f16kv(q, k16.view(np.uint16), v16.view(np.uint16), causal=False, threads=8)) < TOL


# --------------------------------------------------------------------------------------------- TurboQuant cache + decode

def _run_turbo_config(er, oracle, torch, L, B, Hq, Hkv, ctx, steps, seed, kbits, vbits, norm_format, layout, page_size=0,
                      ragged=False, outliers=False, theta=THETA_QWEN3):
    """Cache bytes (codes, norms) are compared bit for bit.  Attention outputs are held to the same element-wise bound
    as the fp16 cache (helpers.max_rel_err < 2e-3): queries, probabilities and both codebooks enter the tensor-core
    products as fp16 hi + lo pairs."""
    D = 128
    rng = rng_for(seed)
    lens = [ctx] * B if not ragged else [int(x) for x in rng.integers(max(1, ctx // 8), ctx + 1, size=B)]
    T = (max(lens) + steps + 15) // 16 * 16
    kw = {}
    if layout == er.Layout.paged:
        pages_per_seq = (T + page_size - 1) // page_size
        num_pages = pages_per_seq * B + 2
        kw = dict(page_size=page_size, num_pages=num_pages)
        alloc = er.BlockTableAllocator(num_pages, page_size, free_order=rng.permutation(num_pages))
    fp16_norm = norm_format == er.NormFormat.float16
    cache = er.KVCache(T, L, Hkv, D, er.Precision.turboquantV2, key_type=kbits, value_type=vbits, norm_format=norm_format,
                       max_batch=B, layout=layout, **kw)
    if layout == er.Layout.paged:
        for b in range(B):
            cache.set_block_table(b, alloc.ensure(b, lens[b] + steps))
    sp = er.step_params(rope_theta=theta)
    kscale = outlier_channels(rng, (Hkv, D)) if outliers else np.ones((Hkv, D), np.float32)
    vscale = outlier_channels(rng, (Hkv, D)) if outliers else np.ones((Hkv, D), np.float32)
    kwid, vwid = (128 * kbits + 31) // 32, (128 * vbits + 31) // 32
    st = {}
    round16 = (lambda a: a.astype(np.float16).astype(np.float32)) if fp16_norm else (lambda a: a)
    for l in range(L):
        for b in range(B):
            n = lens[b]
            K = (rng.standard_normal((n, Hkv, D), dtype=np.float32) * kscale).astype(np.float16).astype(np.float32)
            V = (rng.standard_normal((n, Hkv, D), dtype=np.float32) * vscale).astype(np.float16).astype(np.float32)
            cache.write_rows(l, b, 0, n, dev(torch, K), dev(torch, V), sp)
            Kr = np.concatenate([oracle.rope_neox(K[t:t + 1], t, theta) for t in range(n)])
            kc, kn = oracle.tq_encode_rows(Kr.reshape(-1, D), kbits)
            vc, vn = oracle.tq_encode_rows(V.reshape(-1, D), vbits)
            pad = steps * Hkv
            st[l, b] = [np.concatenate([kc, np.zeros((pad, kwid), np.uint32)]), np.concatenate([round16(kn), np.zeros(pad, np.float32)]),
                        np.concatenate([vc, np.zeros((pad, vwid), np.uint32)]), np.concatenate([round16(vn), np.zeros(pad, np.float32)])]
    torch.cuda.synchronize()
    worst = 0.0
    for s in range(steps):
        q = normal_f16(rng, (L, B, Hq, D))
        k = (rng.standard_normal((L, B, Hkv, D), dtype=np.float32) * kscale).astype(np.float16).astype(np.float32)
        v = (rng.standard_normal((L, B, Hkv, D), dtype=np.float32) * vscale).astype(np.float16).astype(np.float32)
        out = torch.full((L, B, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
        torch.cuda.synchronize()
        assert cache.device_status() == 0
        got = out.cpu().numpy()
        for l in range(L):
            for b in range(B):
                kc, kn, vc, vn = st[l, b]
                want = oracle.decode_step_turboquant(q[l, b], k[l, b], v[l, b], kc, kn, kbits, vc, vn, vbits, lens[b] + s,
                                                     theta, norm_fp16=fp16_norm, threads=8)
                worst = max(worst, max_rel_err(got[l, b], want))
                assert attention_err(got[l, b], want) < 4e-5   # measured: up to 2.4e-5 with x20 outlier channels, 3e-6 without
    print("TurboQuant K%d/V%d decode: worst element-wise relative error %.2e" % (kbits, vbits, worst))
    assert worst < TOL, worst
    # stored rows, exported in the reference's split-buffer format: codes and float32 norms bit-exact
    for l in range(L):
        for b in range(B):
            n = (lens[b] + steps) * Hkv
            (gkc, gks, gkm, gkmeta), (gvc, gvs, gvm, gvmeta) = cache.retrieve_turboquant_runtime_rows(l, seq=b)
            kc, kn, vc, vn = st[l, b]
            assert np.array_equal(gkc, kc[:n]) and np.array_equal(gvc, vc[:n])
            assert np.array_equal(gkmeta[:, 0], kn[:n]) and np.array_equal(gvmeta[:, 0], vn[:n])
            assert not gkmeta[:, 1].any() and not gks.any() and not gkm.any() and not gvs.any() and not gvm.any()
    return worst


@pytest.mark.parametrize("preset", ["balanced", "aggressive"])
@pytest.mark.parametrize("Hq,Hkv,layout,scales", [(16, 8, "head_major", (0.0, 0.0)), (8, 2, "paged", (1.0 / 128, 1.0 / 128)),
                                                   (4, 4, "head_major", (0.0, 1.0 / 64)), (16, 2, "paged", (0.0, 0.0))])
def test_outlier_preset_caches(er, oracle, torch, preset, Hq, Hkv, layout, scales):
    """Caches of balanced / aggressive rows (32 high-precision channels, QJL residual signs, two norms per row): rows written
    by prefill fill, by the host append and by decode steps are bit-identical to the CPU encoder's (keys selected by magnitude,
    values by quantisation benefit, TurboQuantV2Contract); decode attention (gqa_attention_turboquant_decode's general form,
    Shaders/TurboQuant.metal:1794-2001), chunked prefill attention and approximateDecode against the CPU restatements, with
    the residual term off (the reference's contract) and on."""
    D, L, B, steps = 128, 2, 2, 2
    rng = rng_for(700 + Hq + len(preset))
    prec = er.Precision.turboQuantBalanced if preset == "balanced" else er.Precision.turboQuantAggressive
    lens = [150, 37]
    T = 208
    kw = {}
    if layout == "paged":
        ps = 16
        pages = (T // ps) * B + 1
        kw = dict(layout=er.Layout.paged, page_size=ps, num_pages=pages)
        alloc = er.BlockTableAllocator(pages, ps, free_order=rng.permutation(pages))
    ks, vs = scales
    cache = er.KVCache(T, L, Hkv, D, prec, max_batch=B, key_residual_scale=ks, value_residual_scale=vs, **kw)
    if layout == "paged":
        for b in range(B):
            cache.set_block_table(b, alloc.ensure(b, T))
    theta = THETA_QWEN3
    sp = er.step_params(rope_theta=theta)
    rows = {}

    def encode(Krot, V):
        return [oracle.tq_encode_rows_preset(Krot.reshape(-1, D), preset, False), oracle.tq_encode_rows_preset(V.reshape(-1, D), preset, True)]

    def cat(a, b_):
        return [tuple(np.concatenate([x, y]) for x, y in zip(a[i], b_[i])) for i in range(2)]

    for l in range(L):
        for b in range(B):
            n = lens[b]
            K, V = normal_f16(rng, (n, Hkv, D)), normal_f16(rng, (n, Hkv, D))
            cache.write_rows(l, b, 0, n, dev(torch, K), dev(torch, V), sp)
            Kr = np.concatenate([oracle.rope_neox(K[t:t + 1], t, theta) for t in range(n)])
            rows[l, b] = encode(Kr, V)
    torch.cuda.synchronize()
    worst = 0.0
    for s in range(steps):
        q, k, v = normal_f16(rng, (L, B, Hq, D)), normal_f16(rng, (L, B, Hkv, D)), normal_f16(rng, (L, B, Hkv, D))
        out = torch.full((L, B, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
        torch.cuda.synchronize()
        assert cache.device_status() == 0
        got = out.cpu().numpy()
        for l in range(L):
            for b in range(B):
                pos = lens[b] + s
                rows[l, b] = cat(rows[l, b], encode(oracle.rope_neox(k[l, b][None], pos, theta), v[l, b][None]))
                qr = oracle.rope_neox(q[l, b][None], pos, theta)[0]
                want = oracle.tq_attention_decode_preset(qr, rows[l, b][0], rows[l, b][1], preset, Hkv, pos + 1, ks, vs, threads=8)
                worst = max(worst, max_rel_err(got[l, b], want))
    print("%s rows, residual scales %s: decode worst element-wise relative error %.2e" % (preset, scales, worst))
    assert worst < TOL, worst
    # stored rows in the reference's split buffers, bit for bit; decoded rows (approximateDecode: keys with residualWeight 1,
    # values with the contract's scale)
    for l in range(L):
        for b in range(B):
            got_k, got_v = cache.retrieve_turboquant_runtime_rows(l, seq=b)
            for got_rows, want_rows in ((got_k, rows[l, b][0]), (got_v, rows[l, b][1])):
                for g, w_ in zip(got_rows, want_rows):
                    assert np.array_equal(np.asarray(g).view(np.uint32), np.asarray(w_).view(np.uint32)), (l, b)
    dk, dv = cache.retrieve_decoded_turboquant(0, seq=1)
    n1 = lens[1] + steps
    for got_dec, want_rows, weight in ((dk, rows[0, 1][0], 1.0), (dv, rows[0, 1][1], vs)):
        c_, s_, m_, meta = want_rows
        want = np.stack([oracle.tq_decode_preset(c_[i], s_[i], m_[i], preset, meta[i, 0], meta[i, 1], weight) for i in range(n1 * Hkv)])
        assert np.array_equal(np.asarray(got_dec).reshape(-1, D).view(np.uint32), want.view(np.uint32))
    # one more row through the host append (no rotation: rows as given, KVCache.swift:909-975)
    hk, hv = normal_f16(rng, (Hkv, D)), normal_f16(rng, (Hkv, D))
    cache.append(1, hk, hv, seq=1)
    (gk, _), (gv, _) = [(r[0][-Hkv:], None) for r in cache.retrieve_turboquant_runtime_rows(1, seq=1)]
    want_h = encode(hk, hv)
    assert np.array_equal(gk, want_h[0][0]) and np.array_equal(gv, want_h[1][0])
    cache.set_position(n1, seq=1)
    # chunked prefill over sequence 0 of layer 0: 64 query rows at the end of the context
    S = 64
    n0 = lens[0] + steps
    qc = normal_f16(rng, (S, Hq, D))
    outp = torch.full((S, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    cache.attention_prefill(0, 0, dev(torch, qc), outp, Hq, S, sp, q_offset=n0 - S)
    torch.cuda.synchronize()
    gp = outp.cpu().numpy()
    wp = 0.0
    for r in range(0, S, 7):
        pos = n0 - S + r
        qr = oracle.rope_neox(qc[r][None], pos, theta)[0]
        want = oracle.tq_attention_decode_preset(qr, rows[0, 0][0], rows[0, 0][1], preset, Hkv, pos + 1, ks, vs, threads=8)
        wp = max(wp, max_rel_err(gp[r], want))
    print("%s rows: prefill worst element-wise relative error %.2e" % (preset, wp))
    assert wp < TOL, wp


@pytest.mark.parametrize("kbits,vbits", [(4, 3), (4, 4), (3, 3), (3, 4), (4, 2), (3, 2), (2, 2), (2, 3), (2, 4)])
def test_turboquant_decode_presets(er, oracle, torch, kbits, vbits):
    """Every pair of the fixed presets turbo2 / turbo3 / turbo4 on the tensor-core policy of the persistent kernel."""
    w = _run_turbo_config(er, oracle, torch, L=2, B=1, Hq=16, Hkv=8, ctx=333, steps=2, seed=40 + kbits * 4 + vbits, kbits=kbits,
                          vbits=vbits, norm_format=er.NormFormat.float32, layout=er.Layout.head_major)
    print("turbo K%d/V%d max rel err %.3e" % (kbits, vbits, w))


@pytest.mark.parametrize("Hq,Hkv", [(8, 8), (32, 8), (16, 2)])
def test_turboquant_two_bit_values_other_groups(er, oracle, torch, Hq, Hkv):
    """turbo4 keys with turbo2 values (the value type of the reference's boundary modes) for 1, 4 and 8 heads per kv head, paged."""
    _run_turbo_config(er, oracle, torch, L=1, B=2, Hq=Hq, Hkv=Hkv, ctx=500, steps=2, seed=90 + Hq, kbits=4, vbits=2,
                      norm_format=er.NormFormat.float16, layout=er.Layout.paged, page_size=32, ragged=True)


def test_turboquant_config2_shape_compact_norms(er, oracle, torch):
    """Configuration-2-shaped: batch of sequences, turbo4 K / turbo3 V, fp16 norms, 1% outlier channels x20."""
    _run_turbo_config(er, oracle, torch, L=2, B=3, Hq=16, Hkv=8, ctx=700, steps=2, seed=1, kbits=4, vbits=3,
                      norm_format=er.NormFormat.float16, layout=er.Layout.head_major, ragged=True, outliers=True)


def test_turboquant_config4_shape_paged(er, oracle, torch):
    """Configuration-4-shaped: 32 q / 8 kv heads, turbo4 / turbo4, 64-token pages."""
    _run_turbo_config(er, oracle, torch, L=1, B=3, Hq=32, Hkv=8, ctx=900, steps=2, seed=4, kbits=4, vbits=4,
                      norm_format=er.NormFormat.float16, layout=er.Layout.paged, page_size=64, ragged=True)


@pytest.mark.parametrize("kbits,vbits", [(4, 4), (4, 3), (3, 3)])
def test_turboquant_group8(er, oracle, torch, kbits, vbits):
    """8 query heads per kv head (one full n-tile of the tensor-core policy) on TurboQuant rows."""
    _run_turbo_config(er, oracle, torch, L=1, B=2, Hq=32, Hkv=4, ctx=600, steps=2, seed=60 + kbits + vbits, kbits=kbits, vbits=vbits,
                      norm_format=er.NormFormat.float32, layout=er.Layout.head_major, ragged=True)


def test_turboquant_host_append_and_decoded_retrieve(er, oracle):
    """KVCache.append on a TurboQuant cache + retrieveDecodedTurboQuant (KVCacheTests.swift:221-240) against the
    oracle's cache; decoded rows equal up to the float rounding of the inverse transform's scale order."""
    sig = lambda s: np.array([(math.sin(x * 0.17) + math.cos(x * 0.07) * 0.5) * s for x in range(128)], dtype=np.float32)
    keys = np.concatenate([sig(1.0), sig(0.7)])
    values = np.concatenate([sig(0.5), sig(1.2)])
    c = er.KVCache(8, 1, 2, 128, er.Precision.turboquantV2, key_type=4, value_type=3)
    o = oracle.OracleKVCache(8, 1, 2, 128, oracle.PREC_TURBO_V2, key_bits=4, value_bits=3)
    for i in range(3):
        c.append(0, keys * (i + 1), values - i)
        o.append(0, keys * (i + 1), values - i)
    assert c.current_length == 3
    (kc, _, _, kmeta), (vc, _, _, vmeta) = c.retrieve_turboquant_runtime_rows(0)
    okc, okm = o.turbo_rows(0, False)
    ovc, ovm = o.turbo_rows(0, True)
    assert np.array_equal(kc, okc[:6]) and np.array_equal(vc, ovc[:6])
    assert np.array_equal(kmeta, okm[:6]) and np.array_equal(vmeta, ovm[:6])
    dk, dv = c.retrieve_decoded_turboquant(0)
    wk, wv = o.retrieve_decoded_turboquant(0)
    assert dk.size == 3 * 256 and np.isfinite(dk).all()
    assert np.array_equal(dk, wk) and np.array_equal(dv, wv)


# --------------------------------------------------------------------------------------------- the contract's full sizes

def test_config1_full_size_first_and_last_layers(er, oracle, torch):
    """Configuration 1 at its full size (28 independent layers, context 4096, 16 q / 8 kv heads): two consecutive
    decode steps through the layer-batched entry point; layers 0, 13 and 27 are checked against the oracle, every
    layer through a size-independent property: the output row of a head is a convex combination of V rows, so each
    coordinate lies inside the [min, max] of the cached V column (plus the appended row)."""
    L, Hq, Hkv, D, ctx, theta = 28, 16, 8, 128, 4096, THETA_QWEN3
    rng = rng_for(100)
    cache = er.KVCache(ctx + 16, L, Hkv, D, er.Precision.float16)
    sp = er.step_params(rope_theta=theta)
    check_layers = (0, 13, 27)
    ok, ov, vmin, vmax = {}, {}, [], []
    for l in range(L):
        K, V = normal_f16(rng, (ctx, Hkv, D)), normal_f16(rng, (ctx, Hkv, D))
        cache.write_rows(l, 0, 0, ctx, dev(torch, K), dev(torch, V), sp)
        vmin.append(V.min(axis=0))
        vmax.append(V.max(axis=0))
        if l in check_layers:
            kc = np.concatenate([oracle.rope_neox_to_f16(K[t:t + 1], t, theta) for t in range(ctx)])
            ok[l] = np.concatenate([kc, np.zeros((2, Hkv, D), np.uint16)])
            ov[l] = np.concatenate([oracle.f32_to_f16_bits(V), np.zeros((2, Hkv, D), np.uint16)])
    for s in range(2):
        q, k, v = normal_f16(rng, (L, 1, Hq, D)), normal_f16(rng, (L, 1, Hkv, D)), normal_f16(rng, (L, 1, Hkv, D))
        out = torch.full((L, 1, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        for l in range(L):
            lo = np.minimum(vmin[l], v[l, 0]) - 1e-3
            hi = np.maximum(vmax[l], v[l, 0]) + 1e-3
            vmin[l], vmax[l] = np.minimum(vmin[l], v[l, 0]), np.maximum(vmax[l], v[l, 0])
            o = got[l, 0].reshape(Hkv, Hq // Hkv, D)
            assert (o >= lo[:, None, :]).all() and (o <= hi[:, None, :]).all(), l
        for l in check_layers:
            want, _ = oracle.decode_step_f16(q[l, 0], k[l, 0], v[l, 0], ok[l], ov[l], ctx + s, theta, threads=8)
            assert max_rel_err(got[l, 0], want) < TOL, l
    assert cache.total_written(27, 0) == ctx + 2


def test_config2_shape_long_context_sampled(er, oracle, torch):
    """Configuration 2's per-sequence shape (TurboQuant turbo4 K / turbo3 V, fp16 norms, context 32768, outlier channels)
    on one layer and two sequences: appended rows' codes bit-exact, attention against the oracle over the same codes."""
    L, B, Hq, Hkv, D, ctx, theta = 1, 2, 16, 8, 128, 32768, THETA_QWEN3
    rng = rng_for(101)
    cache = er.KVCache(ctx + 16, L, Hkv, D, er.Precision.turboquantV2, key_type=4, value_type=3, norm_format=er.NormFormat.float16,
                       max_batch=B)
    sp = er.step_params(rope_theta=theta)
    ks, vs = outlier_channels(rng, (Hkv, D)), outlier_channels(rng, (Hkv, D))
    for b in range(B):
        for s0 in range(0, ctx, 8192):
            K = (rng.standard_normal((8192, Hkv, D), dtype=np.float32) * ks).astype(np.float16).astype(np.float32)
            V = (rng.standard_normal((8192, Hkv, D), dtype=np.float32) * vs).astype(np.float16).astype(np.float32)
            cache.write_rows(0, b, s0, 8192, dev(torch, K), dev(torch, V), sp)
    q = normal_f16(rng, (L, B, Hq, D))
    k = (rng.standard_normal((L, B, Hkv, D), dtype=np.float32) * ks).astype(np.float16).astype(np.float32)
    v = (rng.standard_normal((L, B, Hkv, D), dtype=np.float32) * vs).astype(np.float16).astype(np.float32)
    out = torch.full((L, B, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    for b in range(B):
        (kc, _, _, kmeta), (vc, _, _, vmeta) = cache.retrieve_turboquant_runtime_rows(0, seq=b)
        assert kc.shape[0] == (ctx + 1) * Hkv
        # the appended row: codes equal the oracle's encoding of the RoPE'd row
        kr = oracle.rope_neox(k[0, b][None], ctx, theta)[0]
        wkc, wkn = oracle.tq_encode_rows(kr, 4)
        wvc, wvn = oracle.tq_encode_rows(v[0, b], 3)
        assert np.array_equal(kc[-Hkv:], wkc) and np.array_equal(vc[-Hkv:], wvc)
        assert np.array_equal(kmeta[-Hkv:, 0], wkn.astype(np.float16).astype(np.float32))
        # attention over the codes the cache holds
        q_rot = oracle.rope_neox(q[0, b][None], ctx, theta)[0]
        want = oracle.tq_attention_decode(q_rot, kc, kmeta[:, 0], 4, vc, vmeta[:, 0], 3, Hkv, ctx + 1, threads=8)
        assert max_rel_err(got[0, b], want) < TOL


# --------------------------------------------------------------------------------------------- Q/K head norm (fused_qk_norm_rope_neox)

@pytest.mark.parametrize("precision,Hq,Hkv,dk", [("float16", 16, 8, 1), ("float16", 16, 8, 2), ("float16", 32, 8, 1), ("float16", 32, 8, 2),
                                                 ("float16", 32, 4, 1), ("turbo", 16, 8, 0), ("q8_0", 16, 8, 0)])
def test_qk_head_norm_then_rope_decode_and_prefill(er, oracle, torch, precision, Hq, Hkv, dk):
    """er_step_params.q_norm_weight / k_norm_weight: per-head RMS norm before RoPE (fused_qk_norm_rope_neox,
    Shaders/RoPE.metal:119-173) on every cache kind.  The K rows the cache ends up holding are compared bit for bit with
    the oracle's norm -> RoPE -> store; the attention outputs within the usual bounds."""
    L, B, D, ctx, theta, eps = 2, 2, 128, 90, THETA_QWEN3, 1e-6
    rng = rng_for(90)
    wq = (1.0 + 0.1 * rng.standard_normal((L, D), dtype=np.float32)).astype(np.float32)
    wk = (1.0 + 0.1 * rng.standard_normal((L, D), dtype=np.float32)).astype(np.float32)
    dwq, dwk = dev(torch, wq), dev(torch, wk)
    sp = er.step_params(rope_theta=theta, q_norm_weight=dwq, k_norm_weight=dwk, rms_eps=eps, norm_weight_layer_stride=D)
    T = 128
    if precision == "float16":
        cache = er.KVCache(T, L, Hkv, D, er.Precision.float16, max_batch=B, decode_kernel=dk)   # 1 = persistent, 2 = slim kernel
    elif precision == "turbo":
        cache = er.KVCache(T, L, Hkv, D, er.Precision.turboquantV2, key_type=4, value_type=3, max_batch=B)
    else:
        cache = er.KVCache(T, L, Hkv, D, er.Precision.q8_0, max_batch=B)
    Kraw = normal_f16(rng, (L, B, ctx + 1, Hkv, D)) * 3.0
    V = normal_f16(rng, (L, B, ctx + 1, Hkv, D))
    for l in range(L):
        for b in range(B):
            cache.write_rows(l, b, 0, ctx, dev(torch, Kraw[l, b, :ctx]), dev(torch, V[l, b, :ctx]), sp)
    q = normal_f16(rng, (L, B, Hq, D)) * 2.0
    out = torch.full((L, B, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    cache.decode_step(dev(torch, q), dev(torch, Kraw[:, :, ctx]), dev(torch, V[:, :, ctx]), out, Hq, sp)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    for l in range(L):
        for b in range(B):
            Kn = oracle.head_rms_norm(Kraw[l, b], wk[l], eps)                   # [ctx+1, Hkv, D]
            qn = oracle.head_rms_norm(q[l, b], wq[l], eps)
            Kr = np.concatenate([oracle.rope_neox(Kn[t:t + 1], t, theta) for t in range(ctx + 1)])
            qr = oracle.rope_neox(qn[None], ctx, theta)
            if precision == "float16":
                k16 = np.concatenate([oracle.rope_neox_to_f16(Kn[t:t + 1], t, theta) for t in range(ctx + 1)])
                v16 = oracle.f32_to_f16_bits(V[l, b])
                gk, gv = cache.retrieve(l, np.float16, seq=b)
                assert np.array_equal(gk.view(np.uint16).reshape(-1, Hkv, D), k16)
                want = oracle.gqa_f16kv(qr, k16, v16, causal=True, q_offset=ctx)[0]
                assert max_rel_err(got[l, b], want) < TOL
            elif precision == "q8_0":
                k8, v8 = oracle.q8_encode_rows(Kr), oracle.q8_encode_rows(V[l, b])
                gk, gv = cache.retrieve_q8_0_rows(l, seq=b)
                assert np.array_equal(gk, k8) and np.array_equal(gv, v8)
                want = oracle.gqa_q8kv(qr, k8, v8, causal=True, q_offset=ctx)[0]
                assert max_rel_err(got[l, b], want) < TOL
            else:
                kc, kn = oracle.tq_encode_rows(Kr.reshape(-1, D), 4)
                vc, vn = oracle.tq_encode_rows(V[l, b].reshape(-1, D), 3)
                (gkc, _, _, gkm), _ = cache.retrieve_turboquant_runtime_rows(l, seq=b)
                assert np.array_equal(gkc, kc) and np.array_equal(gkm[:, 0], kn)
                want = oracle.tq_attention_decode(qr[0], kc, kn, 4, vc, vn, 3, Hkv, ctx + 1)
                assert max_rel_err(got[l, b], want) < TOL
    # chunked prefill with the query norm: the last 40 rows of sequence 0, layer 1, as a chunk
    if precision == "float16":
        S = 40
        qc = normal_f16(rng, (S, Hq, D))
        o2 = torch.full((S, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        cache.attention_prefill(1, 0, dev(torch, qc), o2, Hq, S, sp)
        torch.cuda.synchronize()
        Kn = oracle.head_rms_norm(Kraw[1, 0], wk[1], eps)
        k16 = np.concatenate([oracle.rope_neox_to_f16(Kn[t:t + 1], t, theta) for t in range(ctx + 1)])
        v16 = oracle.f32_to_f16_bits(V[1, 0])
        qr = oracle.rope_neox(oracle.head_rms_norm(qc, wq[1], eps), ctx + 1 - S, theta)
        want = oracle.gqa_f16kv(qr, k16, v16, causal=True, q_offset=ctx + 1 - S)
        assert max_rel_err(o2.cpu().numpy(), want) < TOL


# --------------------------------------------------------------------------------------------- q8_0 cache

def test_q8_0_quantize_rows_operator_bit_exact(er, oracle):
    """er_quantize_q8_0_rows (quantize_q8_0_rows, Dequant_Q8_0.metal:19-49) against the oracle's encodeQ8Row: scales and
    int8 codes bit for bit, including zero blocks, huge and tiny magnitudes, a row stride and exact ties."""
    rng = rng_for(60)
    rows = rng.standard_normal((257, 160), dtype=np.float32)
    rows[3, :32] = 0.0
    rows[4] *= 1e30
    rows[5] *= 1e-30
    rows[6, :4] = [127.0, 0.5, -0.5, 2.5]
    rows[6, 4:32] = 0.0
    got = er.Q8Kernel().execute_quantize_rows(rows)
    want = oracle.q8_encode_rows(np.ascontiguousarray(rows[:, :128]))
    assert np.array_equal(got, want)


def _run_q8_config(er, oracle, torch, L, B, Hq, Hkv, ctx, steps, seed, layout, page_size=0, ragged=False, theta=THETA_QWEN3):
    D = 128
    rng = rng_for(seed)
    lens = [ctx] * B if not ragged else [int(x) for x in rng.integers(max(1, ctx // 8), ctx + 1, size=B)]
    T = (max(lens) + steps + 15) // 16 * 16
    kw = {}
    if layout == er.Layout.paged:
        pages_per_seq = (T + page_size - 1) // page_size
        num_pages = pages_per_seq * B + 2
        kw = dict(page_size=page_size, num_pages=num_pages)
        alloc = er.BlockTableAllocator(num_pages, page_size, free_order=rng.permutation(num_pages))
    cache = er.KVCache(T, L, Hkv, D, er.Precision.q8_0, max_batch=B, layout=layout, **kw)
    if layout == er.Layout.paged:
        for b in range(B):
            cache.set_block_table(b, alloc.ensure(b, lens[b] + steps))
    sp = er.step_params(rope_theta=theta)
    st = {}
    for l in range(L):
        for b in range(B):
            n = lens[b]
            K, V = normal_f16(rng, (n, Hkv, D)), normal_f16(rng, (n, Hkv, D))
            cache.write_rows(l, b, 0, n, dev(torch, K), dev(torch, V), sp)
            Kr = np.concatenate([oracle.rope_neox(K[t:t + 1], t, theta) for t in range(n)])
            kc = np.zeros((n + steps, Hkv, 136), np.uint8)
            vc = np.zeros((n + steps, Hkv, 136), np.uint8)
            kc[:n], vc[:n] = oracle.q8_encode_rows(Kr), oracle.q8_encode_rows(V)
            st[l, b] = [kc, vc]
    torch.cuda.synchronize()
    worst = 0.0
    for s in range(steps):
        q, k, v = normal_f16(rng, (L, B, Hq, D)), normal_f16(rng, (L, B, Hkv, D)), normal_f16(rng, (L, B, Hkv, D))
        out = torch.full((L, B, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
        torch.cuda.synchronize()
        assert cache.device_status() == 0
        got = out.cpu().numpy()
        for l in range(L):
            for b in range(B):
                kc, vc = st[l, b]
                want = oracle.decode_step_q8(q[l, b], k[l, b], v[l, b], kc, vc, lens[b] + s, theta, threads=8)
                worst = max(worst, max_rel_err(got[l, b], want))
    assert worst < TOL, worst
    # stored rows in the reference's 34-byte block format: bit-exact, every row including the appended ones
    for l in range(L):
        for b in range(B):
            gk, gv = cache.retrieve_q8_0_rows(l, seq=b)
            kc, vc = st[l, b]
            assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
            dk, dv = cache.retrieve_decoded_q8_0(l, seq=b)
            assert np.array_equal(dk.reshape(-1, Hkv, D), oracle.q8_decode_rows(kc))
            assert np.array_equal(dv.reshape(-1, Hkv, D), oracle.q8_decode_rows(vc))
    return worst


@pytest.mark.parametrize("Hq,Hkv", [(16, 8), (8, 8), (32, 8), (16, 2)])
def test_q8_0_decode_groups(er, oracle, torch, Hq, Hkv):
    w = _run_q8_config(er, oracle, torch, L=2, B=1, Hq=Hq, Hkv=Hkv, ctx=333, steps=2, seed=70 + Hq, layout=er.Layout.head_major)
    print("q8_0 group %d max rel err %.3e" % (Hq // Hkv, w))


def test_q8_0_decode_batched_ragged_paged(er, oracle, torch):
    _run_q8_config(er, oracle, torch, L=2, B=3, Hq=16, Hkv=8, ctx=700, steps=2, seed=75, layout=er.Layout.paged, page_size=32, ragged=True)


def test_q8_0_host_append_errors_and_prefill(er, oracle, torch):
    """KVCache.append on a q8_0 cache (appendQ8_0, KVCache.swift:977-1005), the typed-retrieve error, and chunked prefill
    (gqa_attention_q8kv with seqLen > 1)."""
    D, Hq, Hkv, theta = 128, 16, 8, 1.0e6
    rng = rng_for(80)
    c = er.KVCache(8, 1, Hkv, D, er.Precision.q8_0)
    rows = []
    for t in range(11):                                   # wraps the 8-slot ring
        k, v = rng.standard_normal(Hkv * D, dtype=np.float32), rng.standard_normal(Hkv * D, dtype=np.float32)
        c.append(0, k, v)
        rows.append((k, v))
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        c.retrieve(0, np.float32)
    assert e.value.name == "compressedRetrieveRequiresDecodedAPI"
    gk, gv = c.retrieve_q8_0_rows(0)
    want_k = np.stack([oracle.q8_encode_rows(k.reshape(Hkv, D)) for k, _ in rows[3:]])
    want_v = np.stack([oracle.q8_encode_rows(v.reshape(Hkv, D)) for _, v in rows[3:]])
    assert np.array_equal(gk, want_k) and np.array_equal(gv, want_v)       # oldest-first after the wrap
    # chunked prefill: 150 new rows after 70 cached ones
    ctx, S = 70, 150
    cache = er.KVCache(256, 1, Hkv, D, er.Precision.q8_0)
    sp = er.step_params(rope_theta=theta)
    K, V = normal_f16(rng, (ctx + S, Hkv, D)), normal_f16(rng, (ctx + S, Hkv, D))
    cache.write_rows(0, 0, 0, ctx + S, dev(torch, K), dev(torch, V), sp)
    q = normal_f16(rng, (S, Hq, D))
    out = torch.full((S, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    cache.attention_prefill(0, 0, dev(torch, q), out, Hq, S, sp)
    torch.cuda.synchronize()
    Kr = np.concatenate([oracle.rope_neox(K[t:t + 1], t, theta) for t in range(ctx + S)])
    want = oracle.gqa_q8kv(oracle.rope_neox(q, ctx, theta), oracle.q8_encode_rows(Kr), oracle.q8_encode_rows(V), causal=True,
                           q_offset=ctx, threads=8)
    assert max_rel_err(out.cpu().numpy(), want) < TOL     # keys and values both enter the products as exact fp16 hi + lo pairs


# --------------------------------------------------------------------------------------------- chunked prefill (tensor cores)

@pytest.mark.parametrize("layout,page_size,Hq,Hkv,ctx,S", [
    ("head_major", 0, 16, 8, 300, 77),        # Qwen3-0.6B heads, ragged sizes (partial tiles on both axes)
    ("paged", 64, 32, 8, 1000, 130),          # configuration-4-shaped: 32 q / 8 kv heads, 64-token pages
    ("token_major", 0, 8, 8, 0, 64),          # group 1, prompt from an empty cache
    ("paged", 16, 16, 2, 129, 5),             # group 8
    ("token_major", 0, 8, 8, 70, 150),        # group 1 on the tcgen05 kernel, token-major tensor maps
    ("paged", 16, 16, 2, 1000, 40),           # group 8 on the tcgen05 kernel, 16-token pages (four TMA boxes per tile)
    ("paged", 32, 16, 8, 63, 1),              # single row: falls back to the mma.sync kernel
    ("head_major", 0, 32, 8, 700, 300),       # several CTAs per kv head
    ("head_major", 0, 32, 8, 2000, 513),      # long context
])
def test_chunked_prefill_attention(er, oracle, torch, layout, page_size, Hq, Hkv, ctx, S):
    """er_kv_attention_prefill: a chunk of S new tokens appended after `ctx` cached tokens; query row r (position ctx + r)
    sees keys 0 .. ctx + r.  Oracle: cpuGQA over the fp16 cache contents with kvSeqLen = ctx + S, qOffset = ctx."""
    D, theta = 128, 1.0e6
    rng = rng_for(200 + S)
    T = (ctx + S + 15) // 16 * 16
    kw = {}
    lay = getattr(er.Layout, layout)
    if lay == er.Layout.paged:
        n_pages = (T + page_size - 1) // page_size + 3
        kw = dict(page_size=page_size, num_pages=n_pages)
    cache = er.KVCache(T, 2, Hkv, D, er.Precision.float16, layout=lay, **kw)
    if lay == er.Layout.paged:
        alloc = er.BlockTableAllocator(n_pages, page_size, free_order=rng.permutation(n_pages))
        cache.set_block_table(0, alloc.ensure(0, ctx + S))
    sp = er.step_params(rope_theta=theta)
    layer = 1
    K, V = normal_f16(rng, (ctx + S, Hkv, D)), normal_f16(rng, (ctx + S, Hkv, D))
    if ctx:
        cache.write_rows(layer, 0, 0, ctx, dev(torch, K[:ctx]), dev(torch, V[:ctx]), sp)
    cache.write_rows(layer, 0, ctx, S, dev(torch, K[ctx:]), dev(torch, V[ctx:]), sp)
    q = normal_f16(rng, (S, Hq, D))
    out = torch.full((S, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    cache.attention_prefill(layer, 0, dev(torch, q), out, Hq, S, sp)
    torch.cuda.synchronize()
    kc = np.concatenate([oracle.rope_neox_to_f16(K[t:t + 1], t, theta) for t in range(ctx + S)])
    vc = oracle.f32_to_f16_bits(V)
    q_rot = oracle.rope_neox(q, ctx, theta)
    want = oracle.gqa_f16kv(q_rot, kc, vc, causal=True, q_offset=ctx, threads=8)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    if ctx + S > 2048:
        # thousands of fp32 accumulation steps leave ~2e-7 absolute noise on outputs of size 0.03: bound the error by
        # the head row's largest output instead of element by element
        assert attention_err(got, want) < 2e-5
    else:
        assert max_rel_err(got, want) < TOL
    # explicit offset form gives the same rows
    out2 = torch.empty_like(out)
    cache.attention_prefill(layer, 0, dev(torch, q), out2, Hq, S, sp, q_offset=ctx)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


@pytest.mark.parametrize("layout,page_size,Hq,Hkv,kbits,vbits,ctx,S,fp16_norm", [
    ("head_major", 0, 16, 8, 4, 3, 300, 70, True),
    ("paged", 64, 32, 8, 4, 4, 515, 130, True),       # configuration-4-shaped: 64-token pages, turbo4 / turbo4
    ("head_major", 0, 8, 8, 3, 3, 0, 37, False),
    ("token_major", 0, 16, 8, 3, 4, 90, 2, False),
])
def test_chunked_prefill_attention_turboquant(er, oracle, torch, layout, page_size, Hq, Hkv, kbits, vbits, ctx, S, fp16_norm):
    """er_kv_attention_prefill on a TurboQuant cache (gqa_attention_turboquant with qSeqLen > 1,
    Shaders/TurboQuant.metal:1454-1649): row r at position ctx + r sees codes 0 .. ctx + r.  The tensor-core path rounds
    norm*centroid to fp16 (2^-12 relative), so the bound is the 2e-3 attention metric (error relative to the row's
    largest output), not the element-wise one."""
    D, theta = 128, 1.0e6
    rng = rng_for(400 + S)
    T = (ctx + S + 15) // 16 * 16
    kw = {}
    lay = getattr(er.Layout, layout)
    if lay == er.Layout.paged:
        n_pages = (T + page_size - 1) // page_size + 3
        kw = dict(page_size=page_size, num_pages=n_pages)
    cache = er.KVCache(T, 2, Hkv, D, er.Precision.turboquantV2, key_type=kbits, value_type=vbits, layout=lay,
                       norm_format=er.NormFormat.float16 if fp16_norm else er.NormFormat.float32, **kw)
    if lay == er.Layout.paged:
        alloc = er.BlockTableAllocator(n_pages, page_size, free_order=rng.permutation(n_pages))
        cache.set_block_table(0, alloc.ensure(0, ctx + S))
    sp = er.step_params(rope_theta=theta)
    layer = 1
    n = ctx + S
    K, V = normal_f16(rng, (n, Hkv, D)), normal_f16(rng, (n, Hkv, D))
    cache.write_rows(layer, 0, 0, n, dev(torch, K), dev(torch, V), sp)
    q = normal_f16(rng, (S, Hq, D))
    out = torch.full((S, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    cache.attention_prefill(layer, 0, dev(torch, q), out, Hq, S, sp)
    torch.cuda.synchronize()
    Kr = np.concatenate([oracle.rope_neox(K[t:t + 1], t, theta) for t in range(n)])
    kc, kn = oracle.tq_encode_rows(Kr.reshape(-1, D), kbits)
    vc, vn = oracle.tq_encode_rows(V.reshape(-1, D), vbits)
    if fp16_norm:
        kn, vn = kn.astype(np.float16).astype(np.float32), vn.astype(np.float16).astype(np.float32)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    worst = 0.0
    for r in range(S):
        qr = oracle.rope_neox(q[r:r + 1], ctx + r, theta)[0]
        want = oracle.tq_attention_decode(qr, kc, kn, kbits, vc, vn, vbits, Hkv, ctx + r + 1, threads=8)
        worst = max(worst, max_rel_err(got[r], want))
    print("turbo prefill K%d/V%d worst element-wise relative error %.3e" % (kbits, vbits, worst))
    assert worst < TOL
    out2 = torch.empty_like(out)
    cache.attention_prefill(layer, 0, dev(torch, q), out2, Hq, S, sp, q_offset=ctx)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


def test_prefill_then_decode_consistency(er, oracle, torch):
    """The last row of a prefill chunk equals a decode step that appends the same token."""
    D, Hq, Hkv, ctx, theta = 128, 16, 8, 200, 1.0e6
    rng = rng_for(300)
    K, V = normal_f16(rng, (ctx + 1, Hkv, D)), normal_f16(rng, (ctx + 1, Hkv, D))
    q = normal_f16(rng, (1, Hq, D))
    sp = er.step_params(rope_theta=theta)
    a = er.KVCache(256, 1, Hkv, D, er.Precision.float16)
    b = er.KVCache(256, 1, Hkv, D, er.Precision.float16)
    for c in (a, b):
        c.write_rows(0, 0, 0, ctx, dev(torch, K[:ctx]), dev(torch, V[:ctx]), sp)
    o_dec = torch.empty((1, 1, Hq, D), dtype=torch.float32, device="cuda")
    a.decode_step(dev(torch, q[None]), dev(torch, K[ctx][None, None]), dev(torch, V[ctx][None, None]), o_dec, Hq, sp)
    b.write_rows(0, 0, ctx, 1, dev(torch, K[ctx:]), dev(torch, V[ctx:]), sp)
    # two query rows so the tensor-core kernel is the one that runs: rows at positions ctx-1 and ctx
    q2 = np.concatenate([normal_f16(rng, (1, Hq, D)), q])
    o_pf = torch.empty((2, Hq, D), dtype=torch.float32, device="cuda")
    b.attention_prefill(0, 0, dev(torch, q2), o_pf, Hq, 2, sp)
    torch.cuda.synchronize()
    assert max_rel_err(o_pf[1].cpu().numpy(), o_dec[0, 0].cpu().numpy()) < TOL


# ------------------------------------------------------------------ sliding window / ring-range decode (fp16 rows)

@pytest.mark.parametrize("Hq,Hkv,capacity,kv_start,kv_count,scale", [
    (8, 2, 8, 5, 6, None),          # Gemma4DecodeKernelTests.windowedF16KVGQA: the range wraps the 8-slot ring
    (8, 2, 4, 0, 4, 1.0),           # ...UnscaledAttention
    (8, 2, 512, 0, 512, None),      # the "real Gemma cache capacities" list of the fast kernel's test
    (8, 2, 512, 33, 512, None),
    (16, 8, 4096, 127, 384, None),
    (16, 8, 4096, 1536, 512, 1.0 / 16),
    (4, 4, 4096, 3584, 512, None),
    (16, 8, 700, 650, 333, None),   # capacity that is no multiple of the 16-row unit, wrapped, ragged ends
    (8, 2, 8, 3, 0, None),          # empty range -> zeros
])
def test_windowed_gqa_operator(er, oracle, torch, Hq, Hkv, capacity, kv_start, kv_count, scale):
    """er_gqa_attention_f16kv_windowed against the restatement of gemma4_decode_gqa_f16kv_windowed."""
    D = 128
    rng = rng_for(900 + capacity + kv_start)
    q = normal_f16(rng, (Hq, D))
    if scale == 1.0:
        q *= 0.1      # unscaled attention: keep the scores in the range the reference's test uses
    k, v = normal_f16(rng, (capacity, Hkv, D)), normal_f16(rng, (capacity, Hkv, D))
    got = er.Gemma4DecodeKernels().run_decode_gqa_f16kv_windowed(q, k, v, Hq, Hkv, D, kv_start, kv_count, capacity, scale)
    want = oracle.gqa_f16kv_windowed(q, k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16),
                                     kv_start, kv_count, scale)
    if kv_count == 0:
        assert not got.any()
    else:
        assert max_rel_err(got, want) < TOL


def test_windowed_gqa_operator_errors(er, torch):
    z = torch.zeros(8 * 1024 * 8, dtype=torch.float32, device="cuda")
    g = er.Gemma4DecodeKernels()
    with pytest.raises(er.EdgeRunnerCUDAError):      # more rows than the ring holds
        g.encode_decode_gqa_f16kv_windowed(z, z, z, z, 8, 2, 128, 0, 9, 8)
    with pytest.raises(er.EdgeRunnerCUDAError):      # head sizes above 512 (and odd ones) are not built
        g.encode_decode_gqa_f16kv_windowed(z, z, z, z, 8, 2, 1024, 0, 4, 8)
    with pytest.raises(er.EdgeRunnerCUDAError):
        g.encode_decode_gqa_f16kv_windowed(z, z, z, z, 8, 2, 127, 0, 4, 8)


def _formula_inputs(num_heads, num_kv_heads, head_dim, capacity, mods):
    """Generated inputs of the reference's windowed-attention tests (Gemma4DecodeKernelTests.swift:344-346, 389-391)."""
    (qm, qo, qd), (km, ko, kd), (vm, vo, vd) = mods
    q = np.array([((i % qm) - qo) / qd for i in range(num_heads * head_dim)], np.float32).reshape(num_heads, head_dim)
    shape = (capacity, num_kv_heads, head_dim)
    n = capacity * num_kv_heads * head_dim
    k = np.array([((i % km) - ko) / kd for i in range(n)], np.float32).astype(np.float16).reshape(shape)
    v = np.array([((i % vm) - vo) / vd for i in range(n)], np.float32).astype(np.float16).reshape(shape)
    return q, k, v


@pytest.mark.parametrize("head_dim,capacity,kv_start,kv_count,scale,mods", [
    (256, 8, 5, 6, None, ((13, 6, 17.0), (11, 5, 19.0), (7, 3, 11.0))),    # windowedF16KVGQA, both Gemma head sizes
    (512, 8, 5, 6, None, ((13, 6, 17.0), (11, 5, 19.0), (7, 3, 11.0))),
    (256, 4, 0, 4, 1.0, ((17, 8, 11.0), (13, 6, 13.0), (7, 3, 7.0))),      # windowedF16KVGQAUnscaledAttention
    (256, 512, 0, 512, None, None),        # "real Gemma cache capacities" (fast kernel's test), seeded random inputs
    (256, 512, 33, 512, None, None),
    (512, 4096, 127, 384, None, None),
    (512, 4096, 1536, 512, None, None),
    (512, 4096, 3584, 512, None, None),
    (64, 100, 90, 77, None, None),         # small head size, odd capacity, wrapped
])
def test_windowed_gqa_operator_reference_test_shapes(er, oracle, torch, head_dim, capacity, kv_start, kv_count, scale, mods):
    """The shapes of Gemma4DecodeKernelTests (8 q / 2 kv heads, head sizes 256 and 512) with the tests' generated inputs,
    at the tests' tolerance of 2e-3 absolute and at this suite's relative bound."""
    Hq, Hkv = 8, 2
    if mods is not None:
        q, k, v = _formula_inputs(Hq, Hkv, head_dim, capacity, mods)
    else:
        rng = rng_for(970 + capacity + kv_start)
        q, k, v = normal_f16(rng, (Hq, head_dim)) * 0.5, normal_f16(rng, (capacity, Hkv, head_dim)), normal_f16(rng, (capacity, Hkv, head_dim))
    got = er.Gemma4DecodeKernels().run_decode_gqa_f16kv_windowed(q, k, v, Hq, Hkv, head_dim, kv_start, kv_count, capacity, scale)
    want = oracle.gqa_f16kv_windowed(q, k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16),
                                     kv_start, kv_count, scale)
    assert np.abs(got - want).max() < 2e-3
    assert attention_err(got, want) < 1e-4


@pytest.mark.parametrize("Hq,Hkv,D,S,T,q_offset,causal", [
    (6, 2, 64, 5, 40, 35, True),       # group 3, head size 64: neither is a template of the persistent kernels
    (12, 4, 128, 1, 300, 0, False),    # group 3 at head size 128
    (40, 20, 96, 3, 50, 47, True),     # more than 16 kv heads
    (4, 4, 256, 2, 64, 62, True),
])
def test_gqa_operator_other_head_sizes_and_groups(er, oracle, torch, Hq, Hkv, D, S, T, q_offset, causal):
    """er_gqa_attention_f16kv outside the persistent kernels' shapes: one launch of the generic kernel per query row."""
    rng = rng_for(980 + D + Hq)
    q, k, v = normal_f16(rng, (S, Hq, D)), normal_f16(rng, (T, Hkv, D)), normal_f16(rng, (T, Hkv, D))
    got = er.GQAKernel().execute_f16kv(q, k, v, S, D, Hq, Hkv, causal, kv_seq_len=T, q_offset=q_offset).reshape(S, Hq, D)
    want = oracle.gqa_f16kv(q, k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16), causal=causal,
                            q_offset=q_offset)
    assert max_rel_err(got, want) < TOL


@pytest.mark.parametrize("layout,page_size,T,window,B,Hq", [
    ("head_major", 0, 48, 20, 2, 8),      # window inside a larger ring: the range wraps with the ring
    ("token_major", 0, 48, 20, 1, 8),
    ("paged", 16, 48, 37, 2, 8),
    ("head_major", 0, 40, 40, 1, 8),      # Gemma4GPUKVCache's shape: ring capacity == slidingWindow
    ("head_major", 0, 24, 100, 1, 8),     # window wider than the ring: every slot
    ("paged", 16, 208, 190, 2, 16),       # 4 heads per kv head (tensor-core policy), tiles that cross the ring end
    ("token_major", 0, 64, 33, 1, 32),    # 8 heads per kv head
])
def test_sliding_window_decode(er, oracle, torch, layout, page_size, T, window, B, Hq):
    """er_step_params.sliding_window: each decode step attends to the newest min(window, rows held) rows
    (Gemma4GPUKVCache.attentionRange), fused step and split calls alike, before and after the ring wraps."""
    D, Hkv, theta = 128, 4, 1e4
    rng = rng_for(950 + T + window)
    lay = getattr(er.Layout, layout)
    kw = {}
    if lay == er.Layout.paged:
        per_seq = (T + page_size - 1) // page_size
        kw = dict(page_size=page_size, num_pages=per_seq * B + 1)
    cache = er.KVCache(T, 1, Hkv, D, er.Precision.float16, max_batch=B, layout=lay, **kw)
    if lay == er.Layout.paged:
        alloc = er.BlockTableAllocator(per_seq * B + 1, page_size, free_order=rng.permutation(per_seq * B + 1))
        for b in range(B):
            cache.set_block_table(b, alloc.ensure(b, T))
    sp = er.step_params(rope_theta=theta, sliding_window=window)
    pre = [0, 5][:B]                       # sequence 1 starts with 5 rows: the two ranges differ
    kc = np.zeros((B, T, Hkv, D), np.uint16)
    vc = np.zeros((B, T, Hkv, D), np.uint16)
    for b in range(B):
        if pre[b]:
            K, V = normal_f16(rng, (pre[b], Hkv, D)), normal_f16(rng, (pre[b], Hkv, D))
            cache.write_rows(0, b, 0, pre[b], dev(torch, K), dev(torch, V), sp)
            for t in range(pre[b]):
                kc[b, t] = oracle.rope_neox_to_f16(K[t:t + 1], t, theta)[0]
            vc[b, :pre[b]] = oracle.f32_to_f16_bits(V)
    for s in range(T + 21):
        q, k, v = normal_f16(rng, (1, B, Hq, D)), normal_f16(rng, (1, B, Hkv, D)), normal_f16(rng, (1, B, Hkv, D))
        out = torch.full((1, B, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        if s % 3 == 2:      # split form
            cache.append_rope_kv(dev(torch, k), dev(torch, v), sp)
            cache.attention_decode(dev(torch, q), out, Hq, sp, pending=1)
            cache.advance(1)
        else:
            cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
        torch.cuda.synchronize()
        assert cache.device_status() == 0
        got = out.cpu().numpy()
        for b in range(B):
            pos = pre[b] + s
            kc[b, pos % T] = oracle.rope_neox_to_f16(k[0, b][None], pos, theta)[0]
            vc[b, pos % T] = oracle.f32_to_f16_bits(v[0, b])
            count = min(pos + 1, T, window)
            want = oracle.gqa_f16kv_windowed(oracle.rope_neox(q[0, b][None], pos, theta)[0], kc[b], vc[b],
                                             (pos + 1 - count) % T, count)
            assert max_rel_err(got[0, b], want) < TOL, (s, b)
    for b in range(B):      # the ring itself is untouched by the window: newest T rows, oldest first
        gk, gv = cache.retrieve(0, np.float16, seq=b)
        n = pre[b] + T + 21
        order = [(n + i) % T for i in range(T)]
        assert np.array_equal(gk.view(np.uint16).reshape(T, Hkv, D), kc[b][order])
        assert np.array_equal(gv.view(np.uint16).reshape(T, Hkv, D), vc[b][order])


@pytest.mark.parametrize("precision,kw", [("q8_0", {}), ("turboquantV2", dict(key_type=4, value_type=3)), ("turboQuantBalanced", {})])
def test_sliding_window_on_compressed_caches(er, oracle, torch, precision, kw):
    """er_step_params.sliding_window on q8_0 / TurboQuant caches (decode steps over a wrapping ring, and a windowed chunk):
    each query row attends to the newest min(window, rows held) rows.  Checked against fp32 attention over the rows the
    cache decodes to (retrieve_decoded_*: logical order)."""
    D, Hq, Hkv, T, window, theta = 128, 8, 2, 48, 20, 1e6
    cache = er.KVCache(T, 1, Hkv, D, getattr(er.Precision, precision), **kw)
    sp = er.step_params(rope_theta=theta, sliding_window=window)
    rng = rng_for(515)
    ctx = 40
    cache.write_rows(0, 0, 0, ctx, dev(torch, normal_f16(rng, (ctx, Hkv, D))), dev(torch, normal_f16(rng, (ctx, Hkv, D))), er.step_params(rope_theta=theta))

    preset = {"turboQuantBalanced": "balanced"}.get(precision)

    def decoded():
        if preset:      # decoded key rows of these presets carry the residual term (approximateDecode's default weight): use the stored rows
            kr, vr = cache.retrieve_turboquant_runtime_rows(0)
            return kr, vr
        k, v = cache.retrieve_decoded_q8_0(0) if precision == "q8_0" else cache.retrieve_decoded_turboquant(0)
        return np.asarray(k).reshape(-1, Hkv, D), np.asarray(v).reshape(-1, Hkv, D)

    def held_rows(rows):
        return rows[0].shape[0] // Hkv if preset else rows.shape[0]

    def reference(qr, Kd, Vd, lo, hi):
        """Attention of the rotated query over logical rows [lo, hi)."""
        if preset:
            cut = lambda rows: tuple(a[lo * Hkv:hi * Hkv] for a in rows)
            return oracle.tq_attention_decode_preset(qr[0], cut(Kd), cut(Vd), preset, Hkv, hi - lo, threads=4)
        return oracle.gqa_f32(qr, Kd[lo:hi], Vd[lo:hi], causal=False)[0]

    worst = 0.0
    for s_ in range(14):                                   # the ring (48 slots) wraps after 8 steps
        q, k, v = normal_f16(rng, (1, 1, Hq, D)), normal_f16(rng, (1, 1, Hkv, D)), normal_f16(rng, (1, 1, Hkv, D))
        out = torch.full((1, 1, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        cache.decode_step(dev(torch, q), dev(torch, k), dev(torch, v), out, Hq, sp)
        torch.cuda.synchronize()
        Kd, Vd = decoded()                                  # logical order: the newest rows last
        held = held_rows(Kd)
        n = min(window, held)
        qr = oracle.rope_neox(q[0], ctx + s_, theta)
        want = reference(qr, Kd, Vd, held - n, held)
        worst = max(worst, max_rel_err(out.cpu().numpy()[0, 0], want))
    assert cache.total_written(0, 0) == ctx + 14
    # a windowed chunk: the 12 newest rows as queries
    S, total = 12, ctx + 14
    qc = normal_f16(rng, (S, Hq, D))
    outp = torch.full((S, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    cache.attention_prefill(0, 0, dev(torch, qc), outp, Hq, S, sp)
    torch.cuda.synchronize()
    Kd, Vd = decoded()
    held = held_rows(Kd)
    for r in range(S):
        end = held - (S - 1 - r)                           # rows visible to query row r
        n = min(window, end)
        qr = oracle.rope_neox(qc[r][None], total - S + r, theta)
        want = reference(qr, Kd, Vd, end - n, end)
        worst = max(worst, max_rel_err(outp.cpu().numpy()[r], want))
    print("%s rows, sliding window %d: worst element-wise relative error %.2e" % (precision, window, worst))
    assert worst < TOL
    assert cache.device_status() == 0


@pytest.mark.parametrize("layout,page_size,Hq,Hkv,ctx,S,window", [
    ("head_major", 0, 8, 4, 300, 200, 64),       # window much shorter than the context: leading tiles are skipped
    ("paged", 32, 16, 4, 50, 130, 100),          # window longer than the context of the first rows
    ("token_major", 0, 8, 8, 0, 77, 1),          # every row sees only itself
    ("head_major", 0, 32, 4, 700, 40, 5000),     # window wider than everything: plain causal attention
    ("paged", 64, 16, 8, 3000, 512, 700),        # tcgen05 kernel: several leading 128-token tiles skipped per CTA, split tail
])
def test_sliding_window_prefill(er, oracle, torch, layout, page_size, Hq, Hkv, ctx, S, window):
    """er_kv_attention_prefill with er_step_params.sliding_window: query row at position P sees keys
    max(0, P - window + 1) .. P (Gemma4GPUKVCache.attentionRange applied per row of the chunk)."""
    D, theta = 128, 1.0e4
    rng = rng_for(990 + S + window)
    T = (ctx + S + 15) // 16 * 16
    lay = getattr(er.Layout, layout)
    kw = {}
    if lay == er.Layout.paged:
        n_pages = (T + page_size - 1) // page_size + 2
        kw = dict(page_size=page_size, num_pages=n_pages)
    cache = er.KVCache(T, 1, Hkv, D, er.Precision.float16, layout=lay, **kw)
    if lay == er.Layout.paged:
        alloc = er.BlockTableAllocator(n_pages, page_size, free_order=rng.permutation(n_pages))
        cache.set_block_table(0, alloc.ensure(0, ctx + S))
    sp = er.step_params(rope_theta=theta, sliding_window=window)
    K, V = normal_f16(rng, (ctx + S, Hkv, D)), normal_f16(rng, (ctx + S, Hkv, D))
    cache.write_rows(0, 0, 0, ctx + S, dev(torch, K), dev(torch, V), sp)
    q = normal_f16(rng, (S, Hq, D))
    out = torch.full((S, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    cache.attention_prefill(0, 0, dev(torch, q), out, Hq, S, sp)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    kc = np.concatenate([oracle.rope_neox_to_f16(K[t:t + 1], t, theta) for t in range(ctx + S)])
    vc = oracle.f32_to_f16_bits(V)
    q_rot = oracle.rope_neox(q, ctx, theta)
    for r in range(S):
        pos = ctx + r
        count = min(window, pos + 1)
        want = oracle.gqa_f16kv_windowed(q_rot[r], kc, vc, pos + 1 - count, count)
        assert max_rel_err(got[r], want) < TOL, r


# ------------------------------------------------------------------ seeded random shapes

def test_seeded_random_decode_shapes(er, oracle, torch):
    """40 decode configurations drawn from a fixed seed: storage format x layout x page size x heads per kv head x batch x
    context x steps x ragged lengths, each checked like the hand-written cases (cache bytes bit-exact, attention within bound)."""
    rng = rng_for(31337)
    for _ in range(40):
        kind = str(rng.choice(["dense", "q8", "turbo"]))
        Hkv, group = int(rng.choice([1, 2, 4, 8])), int(rng.choice([1, 2, 4, 8]))
        layout = str(rng.choice(["head_major", "token_major", "paged"])) if kind == "dense" else str(rng.choice(["head_major", "paged"]))
        ps = int(rng.choice([16, 32, 64])) if layout == "paged" else 0
        L, B, ctx, steps = int(rng.integers(1, 4)), int(rng.integers(1, 5)), int(rng.integers(1, 1200)), int(rng.integers(1, 4))
        ragged, seed = bool(rng.integers(0, 2)), int(rng.integers(0, 1 << 30))
        common = dict(L=L, B=B, Hq=Hkv * group, Hkv=Hkv, ctx=ctx, steps=steps, seed=seed, page_size=ps, ragged=ragged)
        lay = getattr(er.Layout, layout)
        if kind == "dense":
            _run_dense_config(er, oracle, torch, lay, **common)
        elif kind == "q8":
            _run_q8_config(er, oracle, torch, layout=lay, **common)
        else:
            _run_turbo_config(er, oracle, torch, kbits=int(rng.choice([3, 4])), vbits=int(rng.choice([3, 4])),
                              norm_format=er.NormFormat.float16 if rng.integers(0, 2) else er.NormFormat.float32, layout=lay, **common)


def test_seeded_random_windowed_operator_shapes(er, oracle, torch):
    """60 ring ranges drawn from a fixed seed over head sizes 64 / 128 / 256 / 512 and 1 / 2 / 4 / 8 heads per kv head."""
    rng = rng_for(31338)
    for _ in range(60):
        Hkv, group = int(rng.choice([1, 2, 4, 8])), int(rng.choice([1, 2, 4, 8]))
        cap = int(rng.integers(1, 3000))
        cnt, st, D = int(rng.integers(0, cap + 1)), int(rng.integers(0, cap)), int(rng.choice([128, 128, 64, 256, 512]))
        q, k, v = normal_f16(rng, (Hkv * group, D)), normal_f16(rng, (cap, Hkv, D)), normal_f16(rng, (cap, Hkv, D))
        got = er.Gemma4DecodeKernels().run_decode_gqa_f16kv_windowed(q, k, v, Hkv * group, Hkv, D, st, cnt, cap)
        want = oracle.gqa_f16kv_windowed(q, k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16), st, cnt)
        if cnt == 0:
            assert not got.any()
        else:
            assert max_rel_err(got, want) < TOL, (Hkv, group, D, cap, st, cnt)


def test_full_size_shapes_constant_value_rows(er, torch):
    """A size-independent property at the benchmark contract's full sequence sizes (no CPU reference finishes there): when every V row of a
    kv head is the same vector, attention returns that vector whatever the keys and the scores are (the probabilities sum to
    one).  Configuration 3's full batch (64 sequences, contexts U[1024, 16384], fp16 rows in 16-token pages behind a random
    block table, 32 / 8 heads; one of its 32 layers) and configuration 4's full context (131072 tokens, turbo4 / turbo4 in
    64-token pages; one layer, one sequence) -- the decode step, and for configuration 4 also a 256-row prefill chunk."""
    D = 128
    g = torch.Generator(device="cuda")
    g.manual_seed(2024)
    # ---- configuration 3 ----
    B, Hq, Hkv, ps = 64, 32, 8, 16
    rng = rng_for(33)
    lens = [int(x) for x in rng.integers(1024, 16385, size=B)]
    pages = sum((n + 1 + ps - 1) // ps for n in lens)
    cache = er.KVCache(max(lens) + 16, 1, Hkv, D, er.Precision.float16, max_batch=B, layout=er.Layout.paged, page_size=ps, num_pages=pages)
    alloc = er.BlockTableAllocator(pages, ps, free_order=rng.permutation(pages))
    sp = er.step_params(rope_theta=5e5)
    pattern = torch.randn((Hkv, D), generator=g, device="cuda").half().float()
    for b, n in enumerate(lens):
        cache.set_block_table(b, alloc.ensure(b, n + 1))
        cache.write_rows(0, b, 0, n, torch.randn((n, Hkv, D), generator=g, device="cuda"), pattern.expand(n, Hkv, D).contiguous(), sp)
    q = torch.randn((1, B, Hq, D), generator=g, device="cuda")
    k = torch.randn((1, B, Hkv, D), generator=g, device="cuda")
    out = torch.full((1, B, Hq, D), float("nan"), device="cuda")
    cache.decode_step(q, k, pattern.expand(1, B, Hkv, D).contiguous(), out, Hq, sp)
    torch.cuda.synchronize()
    assert cache.device_status() == 0
    want = pattern.repeat_interleave(Hq // Hkv, dim=0).expand(B, Hq, D)
    err = float((out[0] - want).abs().max() / want.abs().max())
    print("configuration 3, full batch: constant-V error %.2e of the largest value" % err)
    assert err < 1e-5           # fp32 rounding of the hi + lo products; the bound of the path is 2e-3
    cache.close()
    # ---- configuration 4 ----
    Hq, Hkv, ps, ctx = 32, 8, 64, 131072
    T = ctx + 64
    cache = er.KVCache(T, 1, Hkv, D, er.Precision.turboquantV2, key_type=4, value_type=4, norm_format=er.NormFormat.float16,
                       layout=er.Layout.paged, page_size=ps, num_pages=T // ps)
    cache.set_block_table(0, rng.permutation(T // ps))
    sp = er.step_params(rope_theta=1e6)
    pattern = torch.randn((Hkv, D), generator=g, device="cuda").half().float()
    for s0 in range(0, ctx, 16384):
        cache.write_rows(0, 0, s0, 16384, torch.randn((16384, Hkv, D), generator=g, device="cuda"), pattern.expand(16384, Hkv, D).contiguous(), sp)
    one = er.KVCache(16, 1, Hkv, D, er.Precision.turboquantV2, key_type=4, value_type=4, norm_format=er.NormFormat.float16)
    one.write_rows(0, 0, 0, 1, pattern[None].contiguous(), pattern[None].contiguous(), er.step_params(apply_rope=0))
    decoded = torch.as_tensor(np.asarray(one.retrieve_decoded_turboquant(0)[1]).reshape(Hkv, D)).cuda()     # what a stored pattern row decodes to
    want = decoded.repeat_interleave(Hq // Hkv, dim=0)
    q = torch.randn((1, 1, Hq, D), generator=g, device="cuda")
    out = torch.full((1, 1, Hq, D), float("nan"), device="cuda")
    cache.decode_step(q, torch.randn((1, 1, Hkv, D), generator=g, device="cuda"), pattern[None, None].contiguous(), out, Hq, sp)
    S = 256
    qc = torch.randn((S, Hq, D), generator=g, device="cuda")
    outp = torch.full((S, Hq, D), float("nan"), device="cuda")
    cache.attention_prefill(0, 0, qc, outp, Hq, S, sp)
    torch.cuda.synchronize()
    assert cache.device_status() == 0 and cache.total_written(0, 0) == ctx + 1
    scale = float(want.abs().max())
    e_dec = float((out[0, 0] - want).abs().max()) / scale
    e_pre = float((outp - want[None]).abs().max()) / scale
    print("configuration 4, 131072 tokens: constant-V error %.2e (decode), %.2e (prefill chunk) of the largest value" % (e_dec, e_pre))
    assert e_dec < 1e-5 and e_pre < 1e-5


@pytest.mark.parametrize("precision,kbits,vbits", [("float16", 0, 0), ("q8_0", 0, 0), ("turboquantV2", 4, 3), ("turboquantV2", 4, 4),
                                                   ("turboQuantBalanced", 0, 0), ("turboQuantAggressive", 0, 0)])
def test_constant_value_rows_over_long_visits(er, torch, precision, kbits, vbits):
    """The same size-independent property (constant V rows of a kv head come back unchanged) on launches large enough that every
    consumer warp of a CTA walks more than 32 units of one visit -- the tensor-core policies then fold their accumulators into
    the merge buffer several times (per-lane denominators gathered, packed column halves joined) before the visit is published.
    Group 2 on head-major rings of 32832 slots: fp16 rows take the tensor-core policy there too."""
    D, Hq, Hkv, B, L, ctx = 128, 16, 8, 4, 2, 32768
    g = torch.Generator(device="cuda")
    g.manual_seed(77)
    prec = getattr(er.Precision, precision)
    kw = dict(key_type=kbits, value_type=vbits, norm_format=er.NormFormat.float16) if precision == "turboquantV2" else {}
    cache = er.KVCache(ctx + 64, L, Hkv, D, prec, max_batch=B, **kw)
    sp = er.step_params(rope_theta=1e6)
    pattern = torch.randn((Hkv, D), generator=g, device="cuda").half().float()
    for l in range(L):
        for b in range(B):
            for s0 in range(0, ctx, 16384):
                cache.write_rows(l, b, s0, 16384, torch.randn((16384, Hkv, D), generator=g, device="cuda"),
                                 pattern.expand(16384, Hkv, D).contiguous(), sp)
    # what a stored pattern row reads back as in this format
    one = er.KVCache(16, 1, Hkv, D, prec, **kw)
    one.write_rows(0, 0, 0, 1, pattern[None].contiguous(), pattern[None].contiguous(), er.step_params(apply_rope=0))
    if precision == "float16":
        stored = pattern
    elif precision == "q8_0":
        stored = torch.as_tensor(np.asarray(one.retrieve_decoded_q8_0(0)[1]).reshape(Hkv, D)).cuda()
    else:
        stored = torch.as_tensor(np.asarray(one.retrieve_decoded_turboquant(0)[1]).reshape(Hkv, D)).cuda()
    want = stored.repeat_interleave(Hq // Hkv, dim=0)
    q = torch.randn((L, B, Hq, D), generator=g, device="cuda")
    k = torch.randn((L, B, Hkv, D), generator=g, device="cuda")
    out = torch.full((L, B, Hq, D), float("nan"), device="cuda")
    cache.decode_step(q, k, pattern.expand(L, B, Hkv, D).contiguous(), out, Hq, sp)
    torch.cuda.synchronize()
    assert cache.device_status() == 0
    err = float((out - want).abs().max() / want.abs().max())
    print("%s K%d/V%d, %d token-heads per launch: constant-V error %.2e of the largest value" % (precision, kbits, vbits, L * B * Hkv * ctx, err))
    assert err < 1e-5


@pytest.mark.parametrize("preset", ["turboQuantBalanced", "turboQuantAggressive"])
@pytest.mark.parametrize("Hq,Hkv,layout", [(16, 8, "head_major"), (32, 8, "paged"), (4, 4, "head_major")])
def test_outlier_presets_tensor_core_policy_against_simt_kernel(er, torch, preset, Hq, Hkv, layout):
    """Balanced / aggressive rows at contexts of several tiles, residual terms of both sides on: the tensor-core policy of the
    persistent kernel against the SIMT kernel on the same rows (both are held to the CPU restatement at small sizes by
    test_outlier_preset_caches; er_kv_config.decode_kernel picks the kernel)."""
    D, L, B = 128, 2, 3
    lens = [2900, 517, 1]
    T = 3008
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    kw = {}
    if layout == "paged":
        ps = 64
        pages = (T // ps) * B
        kw = dict(layout=er.Layout.paged, page_size=ps, num_pages=pages)
    outs = []
    fill = [(torch.randn((n, Hkv, D), generator=g, device="cuda"), torch.randn((n, Hkv, D), generator=g, device="cuda")) for n in lens]
    q = torch.randn((L, B, Hq, D), generator=g, device="cuda")
    k = torch.randn((L, B, Hkv, D), generator=g, device="cuda")
    v = torch.randn((L, B, Hkv, D), generator=g, device="cuda")
    sp = er.step_params(rope_theta=THETA_QWEN3)
    for dk in (0, 3):
        cache = er.KVCache(T, L, Hkv, D, getattr(er.Precision, preset), max_batch=B, key_residual_scale=1.0 / 64,
                           value_residual_scale=1.0 / 128, decode_kernel=dk, **kw)
        if layout == "paged":
            perm = np.random.default_rng(3).permutation(pages)
            for b in range(B):
                cache.set_block_table(b, perm[b * (T // ps):(b + 1) * (T // ps)])
        for l in range(L):
            for b, n in enumerate(lens):
                cache.write_rows(l, b, 0, n, fill[b][0], fill[b][1], sp)
        out = torch.full((L, B, Hq, D), float("nan"), device="cuda")
        for _ in range(2):   # two steps: the second one sees the row the first one appended
            cache.decode_step(q, k, v, out, Hq, sp)
        torch.cuda.synchronize()
        assert cache.device_status() == 0
        outs.append(out.cpu().numpy())
        cache.close()
    for l in range(L):
        for b in range(B):
            assert attention_err(outs[0][l, b], outs[1][l, b]) < 3e-5
            assert max_rel_err(outs[0][l, b], outs[1][l, b]) < TOL


def _pair_kernels_agree(er, torch, make_key_cache, make_value_cache, Hq, Hkv, layout):
    """Decode attention over a key cache and a value cache of different row formats: the tensor-core policy of the persistent
    kernel (decode_kernel 0) against the SIMT kernel (3) on the same rows -- contexts of several tiles, ragged, an appended row
    pending; paged caches lay their pages out independently of each other.  Then two prefill chunks the same way (the
    tensor-core prefill kernels on rows expanded from both caches against the SIMT kernel)."""
    D, L, B = 128, 2, 3
    lens = [2900, 517, 1]
    T = 3008
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    fill = [(torch.randn((n, Hkv, D), generator=g, device="cuda"), torch.randn((n, Hkv, D), generator=g, device="cuda")) for n in lens]
    q = torch.randn((L, B, Hq, D), generator=g, device="cuda")
    k = torch.randn((L, B, Hkv, D), generator=g, device="cuda")
    v = torch.randn((L, B, Hkv, D), generator=g, device="cuda")
    sp = er.step_params(rope_theta=THETA_QWEN3)
    outs = []
    for dk in (0, 3):
        kw = dict(max_batch=B, decode_kernel=dk)
        if layout == "paged":
            ps = 64
            pages = (T // ps) * B
            kw.update(layout=er.Layout.paged, page_size=ps, num_pages=pages)
        kc = make_key_cache(T, L, Hkv, D, **kw)
        vc = make_value_cache(T, L, Hkv, D, **kw)
        if layout == "paged":
            for cache, seed in ((kc, 3), (vc, 4)):
                perm = np.random.default_rng(seed).permutation(pages)
                for b in range(B):
                    cache.set_block_table(b, perm[b * (T // ps):(b + 1) * (T // ps)])
        for cache in (kc, vc):
            for l in range(L):
                for b, n in enumerate(lens):
                    cache.write_rows(l, b, 0, n, fill[b][0], fill[b][1], sp)
        out = torch.full((L, B, Hq, D), float("nan"), device="cuda")
        for _ in range(2):   # two steps: the second one sees the row the first one appended
            kc.append_rope_kv(k, v, sp)
            vc.append_rope_kv(k, v, sp)
            kc.attention_decode_with_values_of(vc, q, out, Hq, sp, pending=1)
            kc.advance(1)
            vc.advance(1)
        # a chunk of 150 query rows at the end of the longest sequence and one of 9 rows at the end of the second (causal)
        chunks = []
        for b_, S in ((0, 150), (1, 9)):
            qc = torch.randn((S, Hq, D), generator=torch.Generator(device="cuda").manual_seed(100 + b_), device="cuda")
            oc = torch.full((S, Hq, D), float("nan"), device="cuda")
            kc.attention_prefill_with_values_of(vc, 1, b_, qc, oc, Hq, S, sp)
            chunks.append(oc)
        torch.cuda.synchronize()
        assert kc.device_status() == 0 and vc.device_status() == 0
        outs.append([out.cpu().numpy()] + [c_.cpu().numpy() for c_ in chunks])
        kc.close()
        vc.close()
    for l in range(L):
        for b in range(B):
            assert attention_err(outs[0][0][l, b], outs[1][0][l, b]) < 3e-5
            assert max_rel_err(outs[0][0][l, b], outs[1][0][l, b]) < TOL
    for i in (1, 2):     # prefill chunks: the tensor-core prefill kernels on rows expanded from both caches against the SIMT kernel
        for r in range(outs[0][i].shape[0]):
            assert attention_err(outs[0][i][r], outs[1][i][r]) < 3e-5
            assert max_rel_err(outs[0][i][r], outs[1][i][r]) < TOL


PAIR_SHAPES = [(16, 8, "head_major"), (32, 8, "paged"), (4, 4, "head_major"), (16, 2, "paged")]      # groups 2, 4, 1, 8


@pytest.mark.parametrize("vbits", [2, 3, 4])
@pytest.mark.parametrize("Hq,Hkv,layout", PAIR_SHAPES)
def test_q8_keys_with_turboquant_values_tensor_core_policy_against_simt_kernel(er, torch, vbits, Hq, Hkv, layout):
    """gqa_attention_q8k_turboquant_decode's layers (both kernels are held to fp32 attention over the decoded rows at small sizes
    by test_mixed_family_layers_through_pair_caches; er_kv_config.decode_kernel picks the kernel)."""
    _pair_kernels_agree(er, torch,
                        lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.q8_0, **kw),
                        lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.turboquantV2, key_type=vbits, value_type=vbits,
                                                               norm_format=er.NormFormat.float16, **kw),
                        Hq, Hkv, layout)


@pytest.mark.parametrize("kbits", [2, 3, 4])
@pytest.mark.parametrize("Hq,Hkv,layout", PAIR_SHAPES)
def test_turboquant_keys_with_float16_values_tensor_core_policy_against_simt_kernel(er, torch, kbits, Hq, Hkv, layout):
    """gqa_attention_turboquant_decode_f16v's layers (4-bit keys with eight heads per kv head stay on the SIMT kernel)."""
    _pair_kernels_agree(er, torch,
                        lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.turboquantV2, key_type=kbits, value_type=kbits,
                                                               norm_format=er.NormFormat.float32, **kw),
                        lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.float16,
                                                               **{**kw, "layout": kw.get("layout", er.Layout.head_major)}),
                        Hq, Hkv, layout)


@pytest.mark.parametrize("kbits", [2, 3, 4])
@pytest.mark.parametrize("Hq,Hkv,layout", PAIR_SHAPES)
def test_turboquant_keys_with_q8_values_tensor_core_policy_against_simt_kernel(er, torch, kbits, Hq, Hkv, layout):
    """TurboQuant keys with q8_0 values: the boundary layers of TurboQuantAdaptiveMode.boundaryQ8."""
    _pair_kernels_agree(er, torch,
                        lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.turboquantV2, key_type=kbits, value_type=kbits,
                                                               norm_format=er.NormFormat.float16, **kw),
                        lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.q8_0, **kw),
                        Hq, Hkv, layout)


@pytest.mark.parametrize("vbits", [2, 3, 4])
@pytest.mark.parametrize("Hq,Hkv,layout", PAIR_SHAPES)
def test_float16_keys_with_turboquant_values_tensor_core_policy_against_simt_kernel(er, torch, vbits, Hq, Hkv, layout):
    """float16 keys with TurboQuant values (a dense key cache type in TurboQuantV2Contract; 4-bit values with eight heads per kv
    head stay on the SIMT kernel)."""
    _pair_kernels_agree(er, torch,
                        lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.float16,
                                                               **{**kw, "layout": kw.get("layout", er.Layout.head_major)}),
                        lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.turboquantV2, key_type=vbits, value_type=vbits,
                                                               norm_format=er.NormFormat.float32, **kw),
                        Hq, Hkv, layout)


@pytest.mark.parametrize("q8_keys", [True, False])
@pytest.mark.parametrize("Hq,Hkv,layout", PAIR_SHAPES)
def test_q8_with_float16_rows_tensor_core_policy_against_simt_kernel(er, torch, q8_keys, Hq, Hkv, layout):
    """q8_0 keys with float16 values and float16 keys with q8_0 values."""
    q8 = lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.q8_0, **kw)
    f16 = lambda T, L, Hkv_, D, **kw: er.KVCache(T, L, Hkv_, D, er.Precision.float16, **{**kw, "layout": kw.get("layout", er.Layout.head_major)})
    _pair_kernels_agree(er, torch, q8 if q8_keys else f16, f16 if q8_keys else q8, Hq, Hkv, layout)
