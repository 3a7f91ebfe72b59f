"""GPU tests of the boundary's guard rails and of the float32 operator, all through the C ABI:

* GQAKernel.execute on float32 K/V with the additive mask -- the reference's own test inputs
  (Tests/EdgeRunnerMetalTests/GQATests.swift:232-324, closed-form fixtures) against the CPU oracle (cpuGQA);
* attention over a float32 cache;
* paged caches: a write past the pages a sequence owns is refused on the host, dropped (and flagged) on the device,
  and never lands in another sequence's page;
* raw-buffer operators refuse misaligned pointers before anything is launched; a cache refuses another device;
* a bounded wait that runs out comes back as ER_ERR_DEVICE_TIMEOUT with the context still usable (the launch returns
  by itself: the producer warp is told to stay idle and the waits get a 300-microsecond patience).
"""
import numpy as np
import pytest

from helpers import max_rel_err, normal_f16, rng_for

pytestmark = pytest.mark.gpu
TOL = 2e-3


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


def _closed_form(n, mod, shift, step):
    return ((np.arange(n) % mod) - shift).astype(np.float32) * np.float32(step)


def test_gqa_f32_additive_mask_reference_inputs(er, oracle):
    gk = er.GQAKernel()
    # gqaAdditiveMaskMatchesCPUReference (GQATests.swift:232-275)
    S, D, H, Hkv = 8, 128, 4, 2
    q, k, v = _closed_form(S * H * D, 17, 8, 0.025), _closed_form(S * Hkv * D, 13, 6, 0.025), _closed_form(S * Hkv * D, 11, 5, 0.02)
    mask = np.zeros((S, S), dtype=np.float32)
    mask[1, 0], mask[1, 2], mask[5, 4], mask[6, 7] = -np.inf, 2.0, -3.0, -np.inf
    want = oracle.gqa_f32(q.reshape(S, H, D), k.reshape(S, Hkv, D), v.reshape(S, Hkv, D), causal=False, additive_mask=mask)
    got = gk.execute(q, k, v, S, D, H, Hkv, False, additive_mask=mask).reshape(want.shape)
    assert np.abs(got - want).max() < 1e-4          # the reference's bound
    # gqaAdditiveMaskUsesEffectiveKVSeqLen (GQATests.swift:277-324)
    S, T, off, D = 2, 5, 3, 64
    q, k, v = _closed_form(S * H * D, 17, 8, 0.02), _closed_form(T * Hkv * D, 19, 9, 0.02), _closed_form(T * Hkv * D, 23, 11, 0.015)
    mask = np.zeros((S, T), dtype=np.float32)
    mask[0, 1], mask[0, 4], mask[1, 2] = -2.0, -np.inf, 1.5
    want = oracle.gqa_f32(q.reshape(S, H, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D), causal=True, q_offset=off, additive_mask=mask)
    got = gk.execute(q, k, v, S, D, H, Hkv, True, kv_seq_len=T, q_offset=off, additive_mask=mask).reshape(want.shape)
    assert np.abs(got - want).max() < 1e-4
    # a fully masked query row yields zeros (the shader's `maxScore == -inf` rule, GQA.metal:213-216)
    mask[:] = 0
    mask[0, :] = -np.inf
    got = gk.execute(q, k, v, S, D, H, Hkv, True, kv_seq_len=T, q_offset=off, additive_mask=mask).reshape(want.shape)
    assert np.all(got[0] == 0) and np.isfinite(got).all()


@pytest.mark.parametrize("D,H,Hkv,S,T", [(128, 4, 2, 4, 4), (256, 4, 2, 4, 4), (512, 8, 1, 3, 9), (64, 6, 3, 5, 37), (4, 2, 2, 1, 3)])
def test_gqa_f32_head_sizes_against_oracle(er, oracle, D, H, Hkv, S, T):
    """gqaHeadDim128AndWideDimensionsMatchCPUReference (GQATests.swift:326-363) and ragged shapes, seeded N(0,1)."""
    rng = rng_for(900 + D)
    q = rng.standard_normal((S, H, D), dtype=np.float32)
    k = rng.standard_normal((T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((T, Hkv, D), dtype=np.float32)
    gk = er.GQAKernel()
    for causal, off in ((True, T - S), (False, 0)):
        want = oracle.gqa_f32(q, k, v, causal=causal, q_offset=off)
        got = gk.execute(q, k, v, S, D, H, Hkv, causal, kv_seq_len=T, q_offset=off).reshape(want.shape)
        assert max_rel_err(got, want) < TOL, (D, causal)
        assert np.abs(got - want).max() < 1e-4


def test_float32_cache_attention_and_step(er, torch, oracle):
    """Decode over a float32 cache: host appends (KVCache.append), then device steps with RoPE; oracle = cpuGQA over the
    retrieved rows with the query rotated by the oracle's RoPE."""
    rng = rng_for(41)
    L, B, H, Hkv, D, T = 2, 2, 8, 4, 128, 37
    theta = 1.0e6
    c = er.KVCache(64, L, Hkv, D, er.Precision.float32, max_batch=B)
    sp = er.step_params(rope_theta=theta)
    ks = rng.standard_normal((L, B, T, Hkv, D), dtype=np.float32)
    vs = rng.standard_normal((L, B, T, Hkv, D), dtype=np.float32)
    for l in range(L):
        for b in range(B):
            c.write_rows(l, b, 0, T, dev(torch, ks[l, b]), dev(torch, vs[l, b]), sp)
    q = rng.standard_normal((L, B, H, D), dtype=np.float32)
    kn = rng.standard_normal((L, B, Hkv, D), dtype=np.float32)
    vn = rng.standard_normal((L, B, Hkv, D), dtype=np.float32)
    out = torch.full((L, B, H, D), float("nan"), device="cuda")
    c.decode_step(dev(torch, q), dev(torch, kn), dev(torch, vn), out, H, sp)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert c.total_written(0, 0) == T + 1 and c.total_written(1, 1) == T + 1
    for l in range(L):
        for b in range(B):
            kc, vc = c.retrieve(l, np.float32, seq=b)
            kc, vc = kc.reshape(T + 1, Hkv, D), vc.reshape(T + 1, Hkv, D)
            # rows in the cache are the oracle's RoPE of the inputs, bit for bit
            want_k = np.concatenate([oracle.rope_neox(ks[l, b], 0, theta), oracle.rope_neox(kn[l, b][None], T, theta)])
            assert np.array_equal(kc, want_k) and np.array_equal(vc[-1], vn[l, b])
            qr = oracle.rope_neox(q[l, b][None], T, theta)
            want = oracle.gqa_f32(qr, kc, vc, causal=False)[0]
            assert max_rel_err(got[l, b], want) < TOL


def test_paged_rows_without_a_page_are_refused_or_dropped(er, torch):
    L, B, Hkv, D, PS = 1, 2, 2, 128, 16
    rng = rng_for(5)
    sp = er.step_params(rope_theta=1e4)
    c = er.KVCache(64, L, Hkv, D, er.Precision.float16, max_batch=B, layout=er.Layout.paged, page_size=PS, num_pages=6)
    c.set_block_table(0, [0, 3])          # sequence 0 owns 32 rows; pool page 0 is ITS first page
    c.set_block_table(1, [5])             # sequence 1 owns 16 rows
    k0 = dev(torch, normal_f16(rng, (32, Hkv, D)))
    v0 = dev(torch, normal_f16(rng, (32, Hkv, D)))
    c.write_rows(0, 0, 0, 32, k0, v0, sp)
    c.write_rows(0, 1, 0, 16, k0[:16], v0[:16], sp)
    torch.cuda.synchronize()

    def snapshot():
        c.set_position(32, seq=0)
        c.set_position(16, seq=1)
        return [np.concatenate(c.retrieve(0, np.float16, seq=b)).view(np.uint16).copy() for b in range(B)]

    before = snapshot()
    # host side: refused before any launch
    launches = er.lib().er_kernel_launch_count()
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        c.write_rows(0, 1, 16, 4, k0[:4], v0[:4], sp)
    assert e.value.name == "outOfPages" and er.lib().er_kernel_launch_count() == launches
    # device side: sequence 1 is full (16 rows, one page); a decode step appends row 16 -> no page -> dropped + flagged
    H = 4
    q = dev(torch, normal_f16(rng, (L, B, H, D)))
    kn = dev(torch, normal_f16(rng, (L, B, Hkv, D)))
    vn = dev(torch, normal_f16(rng, (L, B, Hkv, D)))
    out = torch.zeros((L, B, H, D), device="cuda")
    c.set_position(31, seq=0)             # sequence 0 appends into its own second page (slot 31): legal
    c.decode_step(q, kn, vn, out, H, sp)
    torch.cuda.synchronize()
    assert c.device_status() == -10        # ER_ERR_OUT_OF_PAGES
    c.clear_device_status()
    after = snapshot()
    assert c.device_status() == 0
    # sequence 1 (whose row was dropped) is unchanged; sequence 0 -- the owner of pool page 0, where a table entry of 0
    # would have sent the dropped row -- changed in its own slot 31 only (K half and V half of the concatenation)
    assert np.array_equal(before[1], after[1])
    diff = np.nonzero(before[0] != after[0])[0]
    half, row = 32 * Hkv * D, Hkv * D
    assert diff.size > 0 and np.all((diff % half) // row == 31)
    c.set_position(31, seq=0)
    c.set_position(16, seq=1)
    hq = q.cpu().numpy()
    with pytest.raises(er.EdgeRunnerCUDAError) as e:    # the host-buffer step reports it by itself
        c.decode_step_host(hq, kn.cpu().numpy(), vn.cpu().numpy(), np.empty_like(hq), H, sp)
    assert e.value.name == "outOfPages"
    c.clear_device_status()


def test_raw_operators_refuse_misaligned_pointers(er, torch):
    gk = er.GQAKernel()
    H, Hkv, T = 4, 2, 40
    q = torch.zeros(H * 128 + 8, device="cuda")
    kv = torch.zeros(T * Hkv * 128 + 8, dtype=torch.float16, device="cuda")
    out = torch.zeros(H * 128 + 8, device="cuda")
    launches = er.lib().er_kernel_launch_count()
    for bad in ("q", "k", "out"):
        ptrs = dict(q=q.data_ptr(), k=kv.data_ptr(), v=kv.data_ptr(), out=out.data_ptr())
        ptrs[bad] += 4
        for fn in (gk.encode, gk.encode_static_workspace):
            with pytest.raises(er.EdgeRunnerCUDAError) as e:
                fn(ptrs["q"], ptrs["k"], ptrs["v"], ptrs["out"], 1, 128, H, Hkv, True, kv_seq_len=T, q_offset=T - 1)
            assert e.value.name == "invalidArgument" and "16-byte" in str(e.value)
    assert er.lib().er_kernel_launch_count() == launches          # nothing was launched


def test_cache_refuses_another_device(er, torch):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with torch.cuda.device(0):
        c = er.KVCache(32, 1, 2, 128, er.Precision.float16)
        k = torch.zeros((1, 1, 2, 128), device="cuda")
    sp = er.step_params()
    launches = er.lib().er_kernel_launch_count()
    with torch.cuda.device(1):
        with pytest.raises(er.EdgeRunnerCUDAError) as e:
            c.append_rope_kv(k, k, sp)
        assert e.value.name == "invalidArgument" and "device" in str(e.value)
    assert er.lib().er_kernel_launch_count() == launches


@pytest.mark.parametrize("precision", ["float16", "turboquant", "q8_0"])
def test_bounded_wait_runs_out_and_reports(er, torch, oracle, precision):
    rng = rng_for(123)
    L, B, H, Hkv, D, T = 1, 1, 4, 2, 128, 200
    kw = dict(max_batch=B)
    if precision == "turboquant":
        c = er.KVCache(256, L, Hkv, D, er.Precision.turboquantV2, key_type=4, value_type=3, **kw)
    else:
        c = er.KVCache(256, L, Hkv, D, getattr(er.Precision, precision), **kw)
    sp = er.step_params(rope_theta=1e4)
    k = dev(torch, normal_f16(rng, (T, Hkv, D)))
    v = dev(torch, normal_f16(rng, (T, Hkv, D)))
    c.write_rows(0, 0, 0, T, k, v, sp)
    q = dev(torch, normal_f16(rng, (L, B, H, D)))
    out = torch.zeros((L, B, H, D), device="cuda")
    c.attention_decode(q, out, H, sp)
    torch.cuda.synchronize()
    good = out.cpu().numpy().copy()
    assert c.device_status() == 0
    c.debug_wait_probe(wait_limit_us=300, withhold_tiles=True)
    c.attention_decode(q, out, H, sp)         # the tiles never arrive: every wait gives up after 300 us
    torch.cuda.synchronize()                  # the launch returns by itself
    assert c.device_status() == -12           # ER_ERR_DEVICE_TIMEOUT
    c.debug_wait_probe(0, False)
    c.clear_device_status()
    out.zero_()
    c.attention_decode(q, out, H, sp)         # the context, the cache and its counters are still good
    torch.cuda.synchronize()
    assert c.device_status() == 0
    assert np.array_equal(out.cpu().numpy(), good)


@pytest.mark.parametrize("precision", ["float16", "q8_0", "turboquant"])
def test_pages_exported_and_imported_for_prefix_reuse(er, torch, precision):
    """er_kv_export_pages / er_kv_import_pages: a prompt prefix written once into sequence 0 of cache A is parked in host
    memory, then attached (other page ids, another sequence) to cache B of the same shape and, through a device buffer, to a
    second sequence of cache A.  Rows read back from the copies must equal the original bit for bit, decode steps on them up to the summation order."""
    rng = np.random.Generator(np.random.PCG64(404))
    L, Hq, Hkv, D, ps, T, B = 3, 16, 8, 128, 16, 160, 3
    pages = (T // ps) * B
    prec = {"float16": er.Precision.float16, "q8_0": er.Precision.q8_0, "turboquant": er.Precision.turboquantV2}[precision]
    kw = dict(key_type=4, value_type=3, norm_format=er.NormFormat.float16) if precision == "turboquant" else {}
    sp = er.step_params(rope_theta=1e6)

    def make(order_seed):
        c = er.KVCache(T, L, Hkv, D, prec, max_batch=B, layout=er.Layout.paged, page_size=ps, num_pages=pages, **kw)
        return c, er.BlockTableAllocator(pages, ps, free_order=np.random.Generator(np.random.PCG64(order_seed)).permutation(pages))

    a, alloc_a = make(1)
    b, alloc_b = make(2)
    n = 70                                                     # 4 full pages + 6 rows of a fifth
    src_pages = alloc_a.ensure(0, n)
    a.set_block_table(0, src_pages)
    for l in range(L):
        k = torch.as_tensor(rng.standard_normal((n, Hkv, D), dtype=np.float32)).cuda()
        v = torch.as_tensor(rng.standard_normal((n, Hkv, D), dtype=np.float32)).cuda()
        a.write_rows(l, 0, 0, n, k, v, sp)
    per_page = a.page_bytes()
    assert per_page == b.page_bytes() and per_page > 0
    parked = a.export_pages(src_pages)                         # numpy bytes on the host
    assert parked.nbytes == per_page * len(src_pages)
    dst_pages = alloc_b.ensure(2, n)
    b.set_block_table(2, dst_pages)
    b.import_pages(dst_pages, parked)
    b.set_position(n, seq=2)
    # second copy inside cache A through a device buffer, on a stream
    stream = torch.cuda.Stream()
    dev_buf = torch.empty(parked.nbytes, dtype=torch.uint8, device="cuda")
    twin_pages = alloc_a.ensure(1, n)
    a.set_block_table(1, twin_pages)
    a.export_pages(src_pages, dev_buf, stream=stream)
    a.import_pages(twin_pages, dev_buf, stream=stream)
    stream.synchronize()
    a.set_position(n, seq=1)
    a.set_position(n, seq=0)

    def rows(c, l, seq):
        if precision == "float16":
            k, v = c.retrieve(l, np.float16, seq=seq)
            return [k.view(np.uint16), v.view(np.uint16)]
        if precision == "q8_0":
            return list(c.retrieve_q8_0_rows(l, seq=seq))
        (kc, _, _, km), (vc, _, _, vm) = c.retrieve_turboquant_runtime_rows(l, seq=seq)
        return [kc, km.view(np.uint32), vc, vm.view(np.uint32)]

    for l in range(L):
        want = rows(a, l, 0)
        for c, seq in ((b, 2), (a, 1)):
            got = rows(c, l, seq)
            assert all(np.array_equal(x, y) for x, y in zip(want, got)), (l, seq)
    # one decode step with the same q / k / v on all three sequences: identical outputs
    q1 = rng.standard_normal((L, 1, Hq, D), dtype=np.float32)
    k1 = rng.standard_normal((L, 1, Hkv, D), dtype=np.float32)
    v1 = rng.standard_normal((L, 1, Hkv, D), dtype=np.float32)
    q, k, v = (torch.as_tensor(np.repeat(x, B, axis=1)).cuda() for x in (q1, k1, v1))
    for c, al, seqs in ((a, alloc_a, (2,)), (b, alloc_b, (0, 1))):   # the idle sequences get a page for their one new row
        for s_ in seqs:
            c.set_block_table(s_, al.ensure(s_, 1))
    out_a = torch.empty((L, B, Hq, D), device="cuda")
    out_b = torch.empty((L, B, Hq, D), device="cuda")
    a.decode_step(q, k, v, out_a, Hq, sp)
    b.decode_step(q, k, v, out_b, Hq, sp)
    torch.cuda.synchronize()
    assert a.device_status() == 0 and b.device_status() == 0
    # same rows, same query: equal up to the summation order (the sequences fall on different CTA boundaries)
    assert torch.isfinite(out_a).all()
    tol = 2e-5 * float(out_a[:, 0].abs().max())
    assert float((out_a[:, 0] - out_a[:, 1]).abs().max()) < tol and float((out_a[:, 0] - out_b[:, 2]).abs().max()) < tol
    with pytest.raises(er.EdgeRunnerCUDAError):
        a.export_pages([pages])                                # beyond the pool
    tm = er.KVCache(32, 1, Hkv, D, er.Precision.float16, layout=er.Layout.token_major)
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        tm.page_bytes()
    assert e.value.name == "unsupported"


def test_heterogeneous_layers_and_shared_kv(er, torch, oracle):
    """KVCache.init(... headDimByLayer:kvSourceLayers: ...) (KVCache.swift:276-392): per-layer head sizes, a layer that
    aliases an earlier layer's buffers, the initializer's refusals; attention over a 256-wide layer through the windowed
    raw-buffer operator on the buffers the cache hands out, against the CPU routine."""
    Hkv, T = 2, 32
    dims, src = [256, 512, 256, 256, 512], [0, 1, 2, 0, 1]
    c = er.HeterogeneousKVCache(T, Hkv, dims, src, er.Precision.float16)
    assert c.head_dim == 256 and c.head_dim_for_layer(1) == 512 and not c.owns_buffers(3) and c.owns_buffers(2)
    rng = np.random.Generator(np.random.PCG64(9))
    rows = {l: [] for l in (0, 1, 2)}
    for t in range(5):
        for l in (0, 1, 2):
            k = rng.standard_normal(Hkv * dims[l]).astype(np.float16)
            v = rng.standard_normal(Hkv * dims[l]).astype(np.float16)
            c.append_f16(l, k, v)
            rows[l].append((k, v))
    for l, s_ in enumerate(src):                          # a shared layer reads its source's rows
        k, v = c.retrieve(l, np.float16)
        assert np.array_equal(k.view(np.uint16), np.concatenate([r[0] for r in rows[s_]]).view(np.uint16))
        assert np.array_equal(v.view(np.uint16), np.concatenate([r[1] for r in rows[s_]]).view(np.uint16))
    assert c.metal_buffers(3) == c.metal_buffers(0) and c.metal_buffers(2) != c.metal_buffers(0)
    assert c.cache_params(4).currentLen == 5 and c.current_length == 5
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        c.retrieve(5, np.float16)
    assert e.value.name == "invalidLayer"
    for bad in (([256, 256], [1, 1]), ([256, 512], [0, 0]), ([256, 256, 256], [0, 0, 1]), ([256], [0, 0]), ([], [])):
        with pytest.raises(er.EdgeRunnerCUDAError) as e:
            er.HeterogeneousKVCache(T, Hkv, bad[0], bad[1], er.Precision.float16)
        assert e.value.name == "unsupportedStorage"
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        er.HeterogeneousKVCache(T, Hkv, [128], [0], er.Precision.turboquantV2)
    assert e.value.name == "unsupportedStorage"
    # attention of 8 query heads over layer 3 (= layer 0's rows, head size 256) with the windowed operator
    H, D = 8, 256
    q = rng.standard_normal((H, D)).astype(np.float32)
    kbuf, vbuf = c.metal_buffers(3)
    qd = torch.as_tensor(q).cuda()
    out = torch.empty((H, D), device="cuda")
    er.Gemma4DecodeKernels().encode_decode_gqa_f16kv_windowed(qd, kbuf, vbuf, out, H, Hkv, D, 0, 5, T)
    torch.cuda.synchronize()
    k16 = np.zeros((T, Hkv, D), np.float16)
    v16 = np.zeros((T, Hkv, D), np.float16)
    for t, (k, v) in enumerate(rows[0]):
        k16[t], v16[t] = k.reshape(Hkv, D), v.reshape(Hkv, D)
    want = oracle.gqa_f16kv_windowed(q, k16.view(np.uint16), v16.view(np.uint16), 0, 5)
    got = out.cpu().numpy()
    floor = 1e-3 * np.abs(want).max()
    assert float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor))) < 2e-3
    c.close()


def test_policy_cache_follows_the_layer_contract(er, torch):
    """A 10-layer stack under TurboQuantV2Contract with turbo4 keys / turbo3 values and the firstLast4Q8 adaptive mode: layers
    0-3 and 6-9 keep q8_0 rows, layers 4-5 TurboQuant rows; every layer's step through PolicyKVCache equals the step of a
    uniform cache of that layer's formats.  (Modes that put turbo2 values next to turbo4 ones resolve too, but decode attention
    is built for 3- and 4-bit rows.)"""
    L, Hq, Hkv, D, ctx = 10, 8, 2, 128, 90
    contract = er.TurboQuantLayerContract(key_type="turbo4", adaptive_mode=1)
    pc = er.PolicyKVCache(128, L, Hkv, D, contract)
    assert pc.layer_types[0] == ("q8_0", "q8_0") and pc.layer_types[3] == ("q8_0", "q8_0") and pc.layer_types[6] == ("q8_0", "q8_0")
    assert pc.layer_types[4] == ("turbo4", "turbo3") and pc.layer_types[5] == ("turbo4", "turbo3")
    assert sorted(len(pc.layers_of(p)) for p in pc.caches) == [2, 8]
    mixed = er.TurboQuantLayerContract(key_type="turbo4", early_q8_layers=2, adaptive_mode=5)      # boundaryTurbo4
    assert [mixed.value_cache_type_for(l, L) for l in (0, 1, 2, 8, 9)] == ["q8_0", "q8_0", "turbo2", "turbo4", "turbo4"]
    rng = np.random.Generator(np.random.PCG64(77))
    sp = er.step_params(rope_theta=1e6)
    from edgerunner_b200.layer_contract import cache_arguments
    for layer in (0, 4, 5, 9):
        K = torch.as_tensor(rng.standard_normal((ctx, Hkv, D), dtype=np.float32)).cuda()
        V = torch.as_tensor(rng.standard_normal((ctx, Hkv, D), dtype=np.float32)).cuda()
        q = torch.as_tensor(rng.standard_normal((1, Hq, D), dtype=np.float32)).cuda()
        k = torch.as_tensor(rng.standard_normal((1, Hkv, D), dtype=np.float32)).cuda()
        v = torch.as_tensor(rng.standard_normal((1, Hkv, D), dtype=np.float32)).cuda()
        (cache,), local = pc.at(layer)
        cache.write_rows(local, 0, 0, ctx, K, V, sp)
        precision, extra = cache_arguments(*pc.layer_types[layer])
        ref = er.KVCache(128, 1, Hkv, D, precision, **extra)
        ref.write_rows(0, 0, 0, ctx, K, V, sp)
        got, want = torch.empty((1, Hq, D), device="cuda"), torch.empty((1, Hq, D), device="cuda")
        pc.decode_step(layer, q, k, v, got, Hq, sp)
        ref.decode_step(q, k, v, want, Hq, sp)
        torch.cuda.synchronize()
        assert torch.equal(got, want), layer
        assert cache.total_written(local, 0) == ctx + 1
        ref.close()
    pc.close()


def _decoded_rows(cache, layer, which, np_):
    """A cache's K (which = 0) or V (1) rows of sequence 0 as float32 [tokens, kv heads, 128], through its own decoded retrieve."""
    if cache.precision.name == "float16":
        return cache.retrieve(layer, np_.float16)[which].astype(np_.float32).reshape(-1, cache.num_kv_heads, 128)
    if cache.precision.name == "q8_0":
        return np_.asarray(cache.retrieve_decoded_q8_0(layer)[which]).reshape(-1, cache.num_kv_heads, 128)
    return np_.asarray(cache.retrieve_decoded_turboquant(layer)[which]).reshape(-1, cache.num_kv_heads, 128)


@pytest.mark.parametrize("contract_kw,layer_pair", [
    (dict(early_q8_key_layers=2), ("q8_0", "turbo3")),                       # gqa_attention_q8k_turboquant(_decode)
    (dict(key_type="turbo4", value_cache_type="dense"), ("turbo4", "dense")),  # gqa_attention_turboquant_decode_f16v
    (dict(key_cache_type="dense", value_type="turbo4", adaptive_mode=0), ("dense", "turbo4")),
    (dict(key_type="turbo3", value_cache_type="q8_0"), ("turbo3", "q8_0")),
])
def test_mixed_family_layers_through_pair_caches(er, torch, oracle, contract_kw, layer_pair):
    """Layers whose keys and values use different cache types (the reference's hybrid layers, chosen per layer by
    TurboQuantV2Contract): the two sides live in two caches; decode steps and a prefill chunk through PolicyKVCache equal plain
    fp32 attention over the rows each side decodes to (the transforms are orthonormal, so scores in the keys' rotated space and
    outputs transformed back from the values' space are attention over the decoded rows)."""
    L, Hq, Hkv, D, ctx, steps = 3, 8, 2, 128, 75, 2
    theta = 1e6
    pc = er.PolicyKVCache(128, L, Hkv, D, er.TurboQuantLayerContract(**contract_kw))
    assert pc.layer_types[0] == layer_pair and pc.is_mixed(0)
    (kc, vc), local = pc.at(0)
    rng = np.random.Generator(np.random.PCG64(31))
    sp = er.step_params(rope_theta=theta)
    K = torch.as_tensor(rng.standard_normal((ctx, Hkv, D), dtype=np.float32).astype(np.float16).astype(np.float32)).cuda()
    V = torch.as_tensor(rng.standard_normal((ctx, Hkv, D), dtype=np.float32).astype(np.float16).astype(np.float32)).cuda()
    pc.write_rows(0, 0, 0, ctx, K, V, sp)
    worst = 0.0
    for s_ in range(steps):
        q = rng.standard_normal((1, Hq, D), dtype=np.float32)
        k = torch.as_tensor(rng.standard_normal((1, Hkv, D), dtype=np.float32)).cuda()
        v = torch.as_tensor(rng.standard_normal((1, Hkv, D), dtype=np.float32)).cuda()
        out = torch.full((1, Hq, D), float("nan"), device="cuda")
        pc.decode_step(0, torch.as_tensor(q).cuda(), k, v, out, Hq, sp)
        torch.cuda.synchronize()
        n = ctx + s_ + 1
        assert kc.total_written(local, 0) == n and vc.total_written(local, 0) == n
        Kd, Vd = _decoded_rows(kc, local, 0, np), _decoded_rows(vc, local, 1, np)
        assert Kd.shape[0] == n and Vd.shape[0] == n
        qr = oracle.rope_neox(q, n - 1, theta)
        want = oracle.gqa_f32(qr, Kd, Vd, causal=False)[0]
        got = out.cpu().numpy()[0]
        floor = 1e-3 * np.abs(want).max()
        worst = max(worst, float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor))))
    # a chunk of 16 query rows at the end of the sequence
    S, n = 16, ctx + steps
    qc = rng.standard_normal((S, Hq, D), dtype=np.float32)
    outp = torch.full((S, Hq, D), float("nan"), device="cuda")
    pc.attention_prefill(0, 0, torch.as_tensor(qc).cuda(), outp, Hq, S, sp, q_offset=n - S)
    torch.cuda.synchronize()
    gp = outp.cpu().numpy()
    for r in range(S):
        qr = oracle.rope_neox(qc[r][None], n - S + r, theta)
        want = oracle.gqa_f32(qr, Kd[:n - S + r + 1], Vd[:n - S + r + 1], causal=False)[0]
        floor = 1e-3 * np.abs(want).max()
        worst = max(worst, float(np.max(np.abs(gp[r] - want) / np.maximum(np.abs(want), floor))))
    # the same rows as a chunk in the middle of the sequence (positions 20 .. 35): later rows stay invisible
    off = 20
    outm = torch.full((S, Hq, D), float("nan"), device="cuda")
    pc.attention_prefill(0, 0, torch.as_tensor(qc).cuda(), outm, Hq, S, sp, q_offset=off)
    torch.cuda.synchronize()
    gm = outm.cpu().numpy()
    for r in range(S):
        qr = oracle.rope_neox(qc[r][None], off + r, theta)
        want = oracle.gqa_f32(qr, Kd[:off + r + 1], Vd[:off + r + 1], causal=False)[0]
        floor = 1e-3 * np.abs(want).max()
        worst = max(worst, float(np.max(np.abs(gm[r] - want) / np.maximum(np.abs(want), floor))))
    print("%s keys / %s values: worst element-wise relative error %.2e" % (layer_pair[0], layer_pair[1], worst))
    assert worst < 2e-3
    assert kc.device_status() == 0 and vc.device_status() == 0
    pc.close()
