"""kv-head sharding on GPUs (all through the C ABI):

* one GPU: G in {2, 4, 8} caches that each hold Hkv / G heads of a Llama-3.1-8B-shaped ragged batch in 16-token pages
  with a random block table; their outputs, concatenated by head, against the CPU oracle (element-wise 2e-3) and against
  the unsharded run; the kernel's peer-store epilogue exercised with a second buffer on the same GPU;
* two GPUs (skipped below two): both exchanges (fused peer stores, NCCL all-gather + re-layout) under torchrun with the
  NCCL backend, each rank checking the exchanged [layers, batch, heads, 128] tensor bit for bit against the shards
  computed on its own GPU.  NVLS is switched off for the test processes (plain NCCL rings / peer stores only).
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import attention_err, max_rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = 2e-3


@pytest.fixture(scope="module")
def er():
    import edgerunner_b200 as er
    assert er.lib().er_device_count() > 0
    return er


def test_head_shards_on_one_gpu_match_oracle_and_unsharded(er, oracle):
    import torch
    from edgerunner_b200.sharding import HeadShard, head_sharded_reference, small_paged_case
    case = small_paged_case(er)
    L, B, H, Hkv, S = case["layers"], case["batch"], case["num_heads"], case["num_kv_heads"], case["steps"]
    runs = {G: head_sharded_reference(er, case["make_cache"], case["fill_cache"], case["q"], case["k"], case["v"], case["params"],
                                      G, steps=S).cpu().numpy() for G in (1, 2, 4, 8)}
    # oracle: per (layer, sequence) the fp16 rows the cache holds (RoPE'd keys) followed by the appended rows
    q, k, v = case["q"].cpu().numpy(), case["k"].cpu().numpy(), case["v"].cpu().numpy()
    worst = 0.0
    for l in range(L):
        for b, n in enumerate(case["lens"]):
            kc = [oracle.rope_neox_to_f16(case["k0"][l][b], 0, case["theta"])]
            vc = [oracle.f32_to_f16_bits(case["v0"][l][b])]
            for s in range(S):
                kc.append(oracle.rope_neox_to_f16(k[s, l, b][None], n + s, case["theta"]))
                vc.append(oracle.f32_to_f16_bits(v[s, l, b][None]))
                qr = oracle.rope_neox(q[s, l, b][None], n + s, case["theta"])
                want = oracle.gqa_f16kv(qr, np.concatenate(kc), np.concatenate(vc), causal=False)[0]
                for G, got in runs.items():
                    e = max_rel_err(got[s, l, b], want)
                    worst = max(worst, e)
                    assert e < TOL, (G, s, l, b, e)
    print("kv-head shards vs oracle: worst element-wise relative error %.2e" % worst)
    for G in (2, 4, 8):       # a different CTA split of the same rows: fp32 merge order only
        assert attention_err(runs[G], runs[1]) < 1e-5, G


def test_peer_store_epilogue_on_one_gpu(er):
    """The decode kernel writes its rows at a head offset of a full-width buffer and mirrors them into `peer` buffers; here
    the peers are two more buffers on the same GPU.  Every precision's kernel family is covered."""
    import torch
    from edgerunner_b200.sharding import HeadShard
    rng = np.random.Generator(np.random.PCG64(17))
    L, B, H, Hkv, T = 2, 3, 16, 4, 150
    for precision, kw in (("float16", {}), ("q8_0", {}), ("turboquantV2", dict(key_type=4, value_type=3))):
        sp = er.step_params(rope_theta=1e4)
        full = [torch.full((L, B, H, 128), float("nan"), device="cuda") for _ in range(3)]
        plain = torch.empty((L, B, H, 128), device="cuda")
        q = torch.as_tensor(rng.standard_normal((L, B, H, 128), dtype=np.float32)).cuda()
        for r in range(2):
            shard = HeadShard(H, Hkv, 2, r)
            # decode_kernel=1: the sharded output layout exists in the persistent kernel, so the plain run uses it too (bitwise)
            c = er.KVCache(256, L, shard.local_kv_heads, 128, getattr(er.Precision, precision), max_batch=B, decode_kernel=1, **kw)
            for l in range(L):
                for b in range(B):
                    kk = torch.as_tensor(rng.standard_normal((T, shard.local_kv_heads, 128), dtype=np.float32)).cuda()
                    c.write_rows(l, b, 0, T - 10 * b, kk[:T - 10 * b], kk.flip(0)[:T - 10 * b].contiguous(), sp)
            ql = shard.slice_q(q).contiguous()
            o = torch.empty((L, B, shard.local_heads, 128), device="cuda")
            c.attention_decode(ql, o, shard.local_heads, sp)
            plain[:, :, shard.q_begin:shard.q_end] = o
            c.set_output_sharding(H, shard.q_begin, [full[1].data_ptr(), full[2].data_ptr()])
            c.attention_decode(ql, full[0], shard.local_heads, sp)
            torch.cuda.synchronize()
            assert c.device_status() == 0
            c.close()
        for f in full:
            assert torch.equal(f, plain), precision


_WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
import edgerunner_b200 as er
from edgerunner_b200.sharding import verify_exchange
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
used = [verify_exchange(er, world, rank, x) for x in ("nccl", "p2p")]
dist.destroy_process_group()
print("rank %d ok %s" % (rank, ",".join(used)))
'''


def test_exchange_on_two_gpus_nccl(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + os.getpid() % 300), str(script), ROOT]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
    print(r.stdout.strip().splitlines()[-2:])
