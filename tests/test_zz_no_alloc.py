"""The allocation-free attention entry point (er_gqa_attention_f16kv_static) against the regular one.

Some hosts of this library may not let it allocate device memory (a serving process whose own pool already holds all
free HBM, or a thread that must stay off the driver's allocation path), so this operator keeps its split-K workspace
in an array built into the library.  The test drives both entry points through the C ABI on the same inputs, twice
in a row (the second call finds the first call's leftovers in the shared workspace), and expects outputs within the
attention tolerance of the other GPU tests -- bit-identical for single query rows, where both run the same kernel
(multi-row calls of the regular entry point use the tensor-core prefill kernel instead) -- and against the CPU oracle;
one case is a multi-row call long enough that every row's launch is split over many CTAs and merged through the shared
workspace.  The workspace's status word is read back at the end (no bounded wait may have given up)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _rel(got, ref):
    floor = 1e-3 * np.abs(ref).max() + 1e-30
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), floor)))


def test_static_workspace_entry_point_matches_regular_one(oracle):
    import torch
    import edgerunner_b200 as er

    rng = np.random.Generator(np.random.PCG64(77))
    gk = er.GQAKernel()
    cases = [  # (query rows, kv rows, q heads, kv heads, causal, q offset)
        (1, 700, 16, 8, True, 699),
        (3, 150, 8, 2, True, 147),
        (1, 33, 4, 4, False, 0),
        (4, 6000, 8, 2, True, 5996),          # four rows, each launch split over all SMs (partials merged through the workspace)
    ]
    for call in range(2):                      # two calls in a row share the built-in workspace
        for S, T, H, Hkv, causal, off in cases:
            q = torch.as_tensor(rng.standard_normal((S, H, 128), dtype=np.float32)).cuda()
            k = torch.as_tensor(rng.standard_normal((T, Hkv, 128), dtype=np.float32).astype(np.float16)).cuda()
            v = torch.as_tensor(rng.standard_normal((T, Hkv, 128), dtype=np.float32).astype(np.float16)).cuda()
            want = torch.full((S, H, 128), float("nan"), device="cuda")
            got = torch.full((S, H, 128), float("nan"), device="cuda")
            gk.encode(q, k, v, want, S, 128, H, Hkv, causal, kv_seq_len=T, q_offset=off)
            gk.encode_static_workspace(q, k, v, got, S, 128, H, Hkv, causal, kv_seq_len=T, q_offset=off)
            torch.cuda.synchronize()
            w, g = want.cpu().numpy(), got.cpu().numpy()
            assert np.isfinite(g).all()
            assert _rel(g, w) < TOL, (call, S, T, H, Hkv)
            if S == 1:
                assert np.array_equal(g, w)
            ref = oracle.gqa_f16kv(q.cpu().numpy(), k.cpu().numpy().view(np.uint16), v.cpu().numpy().view(np.uint16), causal=causal,
                                   q_offset=off, threads=8)
            assert _rel(g, ref) < TOL, ("oracle", call, S, T, H, Hkv)
    assert er.lib().er_gqa_attention_f16kv_static_status() == 0      # no bounded wait gave up in any of those launches


def test_static_workspace_rejects_shapes_beyond_its_limits():
    import torch
    import edgerunner_b200 as er

    gk = er.GQAKernel()
    q = torch.zeros((1, 32, 128), device="cuda")
    kv = torch.zeros((4, 32, 128), dtype=torch.float16, device="cuda")
    out = torch.zeros_like(q)
    with pytest.raises(er.EdgeRunnerCUDAError) as e:       # 32 kv heads > 16
        gk.encode_static_workspace(q, kv, kv, out, 1, 128, 32, 32, False, kv_seq_len=4)
    assert e.value.name == "unsupported" and "at most 16 kv heads" in str(e.value)
    kv2 = torch.zeros((4, 2, 128), dtype=torch.float16, device="cuda")
    q2 = torch.zeros((1, 16, 128), device="cuda")
    with pytest.raises(er.EdgeRunnerCUDAError) as e:       # 8 query heads per kv head > 4
        gk.encode_static_workspace(q2, kv2, kv2, torch.zeros_like(q2), 1, 128, 16, 2, False, kv_seq_len=4)
    assert e.value.name == "unsupported"
