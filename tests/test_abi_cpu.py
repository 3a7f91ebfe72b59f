"""CPU-side checks of the product: the C-ABI library builds/loads and exports every symbol include/er_kv.h
declares, error paths that need no device, the host-side block-table allocator and sharding arithmetic.
No compute entry point is called here (there is no GPU in this environment and no CPU fallback in the library)."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def er():
    import edgerunner_b200 as er
    from edgerunner_b200 import build
    build.build()
    return er


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "er_kv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(er_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(er):
    from edgerunner_b200 import _lib
    declared = _declared_functions()
    assert len(declared) >= 30
    L = er.lib()
    for name in declared:
        assert hasattr(L, name), name
    assert sorted(_lib.SYMBOLS) == declared          # the Python binding covers the whole header
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    exported = set(re.findall(r" T (er_[a-z0-9_]+)", out))
    assert exported == set(declared)                 # and nothing else leaks out of the library


def test_param_struct_layouts_match_reference_headers(er):
    import ctypes as C
    from edgerunner_b200 import _lib
    # Sources/EdgeRunnerSharedTypes/include/{KVCacheParams,AttentionParams,RoPEParams}.h: plain uint32/float fields
    assert C.sizeof(_lib.ERKVCacheParams) == 24 and C.sizeof(_lib.ERGQAParams) == 44 and C.sizeof(_lib.ERRoPEParams) == 28
    assert [f[0] for f in _lib.ERGQAParams._fields_] == ["seqLen", "headDim", "numHeads", "numKVHeads", "groupSize", "scale",
                                                         "causal", "kvBlockSize", "qBlockSize", "kvSeqLen", "qOffset"]
    assert C.sizeof(_lib.er_kv_config) == 64


def test_no_device_fails_loudly(er):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    assert er.lib().er_device_count() == 0
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        er.KVCache(16, 1, 2, 4, er.Precision.float32)
    assert e.value.name == "cuda" and "no CPU fallback" in str(e.value)
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        er.KVCache(16, 1, 2, 128, er.Precision.float8)
    assert e.value.name == "unsupportedStorage"
    with pytest.raises(er.EdgeRunnerCUDAError) as e:
        er.KVCache(0, 1, 2, 128, er.Precision.float16)
    assert e.value.name == "shape"
    assert er.lib().er_status_string(-6) == b"compressedBufferAccessRequiresTurboQuantAPI"


def test_tables_identical_in_oracle_and_product():
    a = open(os.path.join(ROOT, "oracle", "er_tq_tables.h")).read().replace("ER_ORACLE_TQ_TABLES_H", "X")
    b = open(os.path.join(ROOT, "edgerunner_b200", "csrc", "tq_tables.h")).read().replace("ER_CSRC_TQ_TABLES_H", "X")
    assert a == b


def test_product_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "edgerunner_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "er_oracle" not in text and "liber_oracle" not in text, f
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), f


def test_block_table_allocator(er):
    a = er.BlockTableAllocator(10, 16, free_order=[3, 1, 4, 0, 5, 9, 2, 6, 8, 7])
    assert a.pages_for(0) == 0 and a.pages_for(1) == 1 and a.pages_for(16) == 1 and a.pages_for(17) == 2
    assert a.ensure("s0", 33) == [3, 1, 4]
    assert a.ensure("s1", 16) == [0]
    assert a.ensure("s0", 40) == [3, 1, 4] and a.ensure("s0", 49) == [3, 1, 4, 5]
    assert a.free_pages == 5
    with pytest.raises(er.OutOfPages):
        a.ensure("s2", 16 * 6)
    assert a.free_pages == 5 and a.block_table("s2") == []
    a.release("s0")
    assert a.free_pages == 9 and a.ensure("s2", 16 * 6) == [3, 1, 4, 5, 9, 2]
    with pytest.raises(ValueError):
        er.BlockTableAllocator(4, 24)
    with pytest.raises(ValueError):
        er.BlockTableAllocator(4, 16, free_order=[0, 1, 1, 2])


def test_head_and_sequence_shards():
    from edgerunner_b200.sharding import HeadShard, split_range
    covered = []
    for r in range(4):
        s = HeadShard(32, 8, 4, r)
        assert s.group == 4 and s.local_kv_heads == 2 and s.local_heads == 8
        covered += list(range(s.q_begin, s.q_end))
        assert s.q_begin == s.kv_begin * 4
    assert covered == list(range(32))
    with pytest.raises(ValueError):
        HeadShard(32, 8, 3, 0)
    parts = [split_range(10, 4, r) for r in range(4)]
    assert parts == [(0, 3), (3, 6), (6, 8), (8, 10)]


_GLOO_WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
from edgerunner_b200.sharding import HeadShard, all_gather_heads, max_over_ranks, split_range
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%s" % sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
B, H, Hkv, D = 3, 8, 4, 128
shard = HeadShard(H, Hkv, 2, rank)
full = torch.arange(B * H * D, dtype=torch.float32).reshape(B, H, D)
local = shard.slice_q(full).clone()              # stands in for this rank's attention output slice
out = all_gather_heads(local)
assert out.shape == full.shape and torch.equal(out, full), "gathered heads differ"
assert max_over_ranks(1.0 + rank) == 2.0
b0, b1 = split_range(5, 2, rank)                 # sequence sharding: disjoint cover, no exchange
cover = [torch.zeros(5) for _ in range(2)]
mine = torch.zeros(5); mine[b0:b1] = 1
dist.all_gather(cover, mine)
assert torch.equal(cover[0] + cover[1], torch.ones(5))
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_all_gather_of_head_slices_gloo_world2(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o
        assert "rank %d ok" % r in o


def test_heterogeneous_cache_refusals_need_no_device():
    """The share-map checks of the heterogeneous initializer (KVCache.swift:297-333) run before anything touches a device."""
    import edgerunner_b200 as er
    for dims, src, prec in (([256, 256], [1, 1], er.Precision.float16),          # shares a later layer
                            ([256, 512], [0, 0], er.Precision.float16),          # head sizes differ
                            ([256, 256, 256], [0, 0, 1], er.Precision.float16),  # source does not own its buffers
                            ([256], [0, 0], er.Precision.float16),               # lengths differ
                            ([256, 256], [0, 7], er.Precision.float16),          # out of range
                            ([128], [0], er.Precision.q8_0)):                    # dense only
        with pytest.raises(er.EdgeRunnerCUDAError) as e:
            er.HeterogeneousKVCache(32, 2, dims, src, prec)
        assert e.value.name == "unsupportedStorage"


def test_layer_contract_matches_the_reference_tests():
    """TurboQuantV2Contract's per-layer resolution, pinned to the literals of the reference's own test
    (Tests/EdgeRunnerMetalTests/TurboQuantAttentionTests.swift:23-140, which sets the same variables)."""
    from edgerunner_b200 import TurboQuantLayerContract as C_
    c = C_.from_environment({})
    assert (c.key_type, c.value_type) == ("turbo3", "turbo3")
    assert c.key_cache_type_for(0, 28) == "turbo3" and c.value_cache_type_for(0, 28) == "turbo3"
    assert c.key_preset_for(0, 28) == "turbo3" and c.value_preset_for(0, 28) == "turbo3"
    c = C_.from_environment({"EDGERUNNER_TURBOQUANT_KEY_TYPE": "turbo4"})
    assert c.key_type == "turbo4" and c.key_preset_for(0, 1) == "turbo4"
    assert C_.from_environment({"EDGERUNNER_TURBOQUANT_VALUE_POLICY": "boundaryTurbo4"}).value_policy == "boundaryTurbo4"
    c = C_.from_environment({"EDGERUNNER_TURBOQUANT_EARLY_Q8_LAYERS": "1"})
    assert [c.key_cache_type_for(l, 28) for l in (0, 1)] == ["q8_0", "turbo3"]
    assert [c.value_cache_type_for(l, 28) for l in (0, 1)] == ["q8_0", "turbo3"]
    assert c.key_preset_for(0, 28) is None and c.value_preset_for(0, 28) is None
    assert c.key_preset_for(1, 28) == "turbo3" and c.value_preset_for(1, 28) == "turbo3"
    c = C_.from_environment({"EDGERUNNER_TURBOQUANT_EARLY_Q8_KEY_LAYERS": "1"})
    assert [c.key_cache_type_for(l, 28) for l in (0, 1)] == ["q8_0", "turbo3"]
    assert [c.value_cache_type_for(l, 28) for l in (0, 1)] == ["turbo3", "turbo3"]
    assert c.key_preset_for(0, 28) is None and c.value_preset_for(0, 28) == "turbo3"
    c = C_.from_environment({"EDGERUNNER_TURBOQUANT_KEY_PRESET": "planar3", "EDGERUNNER_TURBOQUANT_VALUE_CACHE_TYPE": "dense"})
    assert c.key_cache_type_for(0, 28) == "turbo3" and c.value_cache_type_for(0, 28) == "dense"
    assert c.key_preset_for(0, 28) == "planar3" and c.value_preset_for(0, 28) is None
    # forkAdaptiveModeSevenMapsBoundaryVToQ8 (:127-140)
    c = C_.from_environment({"EDGERUNNER_TURBOQUANT_VALUE_TYPE": "turbo2", "TURBO_LAYER_ADAPTIVE": "7"})
    assert [c.value_cache_type_for(l, 28) for l in (0, 1, 2, 25, 26, 27)] == ["q8_0", "q8_0", "turbo2", "turbo2", "q8_0", "q8_0"]
    # the mode inferred from turbo2 values is the same one (TurboQuant.swift:656-658); short stacks stay uniform
    c = C_(value_type="turbo2")
    assert c.value_cache_type_for(0, 28) == "q8_0" and c.value_cache_type_for(0, 6) == "turbo2"
    assert C_.residual_scale("balanced") == 0.0


def test_policy_cache_pairs_for_mixed_family_layers():
    import edgerunner_b200 as er
    from edgerunner_b200.layer_contract import cache_arguments
    assert cache_arguments("turbo4", "turbo3")[0] == er.Precision.turboquantV2
    assert cache_arguments("q8_0", "turbo3") is None and cache_arguments("turbo3", "dense") is None      # two caches, one per side
    c = er.TurboQuantLayerContract(early_q8_key_layers=1)
    assert (c.key_cache_type_for(0, 4), c.value_cache_type_for(0, 4)) == ("q8_0", "turbo3")


def test_bench_workload_table_is_consistent():
    """Every workload of bench.py names a format the script can build and account bytes for (no GPU involved: the table only)."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.DEFAULT_WORKLOAD in bench.WORKLOADS
    for name, w in bench.WORKLOADS.items():
        assert w["name"] and w["heads"] % w["kv_heads"] == 0, name
        if "keys" in w:                                    # cache pairs
            assert w["keys"] in bench.PAIR_SIDES and w["values"] in bench.PAIR_SIDES and w["keys"] != w["values"], name
            continue
        assert w["precision"] in ("float16", "q8_0", "turboquant", "balanced", "aggressive"), name
        if w["precision"] == "turboquant":
            assert w["kbits"] in (2, 3, 4) and w["vbits"] in (2, 3, 4), name
        assert bench.row_bytes(w) in (512, 272, 192, 160) or w["precision"] == "turboquant", name
        if w.get("layout") == "paged":
            assert w["page_size"] % 16 == 0, name
