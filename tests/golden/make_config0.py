"""Generates tests/golden/config0_expected.npz: the CPU oracle's result for benchmark configuration 0.

Configuration 0 of the benchmark contract: single Qwen3-0.6B-shaped layer, batch 1, 16 query heads, 8 kv heads (group 2),
head_dim 128; contiguous fp16 cache pre-filled with 512 tokens, append 1 token; Q/K/V i.i.d. N(0,1) from seed 0
(numpy PCG64, float32 draws in the order Q, K, V) cast to fp16; NeoX RoPE theta 1e6 at positions 0..512; softmax
scale 1/sqrt(128); fp32 accumulate; output fp32 [16,128].

The reference (Swift + Metal) cannot run in this environment, so this fixture pins the oracle's own output
(regression guard for oracle and kernels alike), not an output of the reference.

    python tests/golden/make_config0.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROWS = [0, 1, 255, 511, 512]


def config0_inputs():
    rng = np.random.Generator(np.random.PCG64(0))
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(np.float16).astype(np.float32)
    Q = draw((16, 128))
    K = draw((513, 8, 128))
    V = draw((513, 8, 128))
    return Q, K, V


def main():
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import er_oracle as oracle
    oracle.build()
    Q, K, V = config0_inputs()
    theta = 1.0e6
    kc = np.zeros((513, 8, 128), np.uint16)
    for t in range(512):
        kc[t] = oracle.rope_neox_to_f16(K[t:t + 1], t, theta)[0]
    vc = np.zeros((513, 8, 128), np.uint16)
    vc[:512] = oracle.f32_to_f16_bits(V[:512])
    out, q_rot = oracle.decode_step_f16(Q, K[512], V[512], kc, vc, 512, theta)
    np.savez_compressed(os.path.join(HERE, "config0_expected.npz"), out=out, q_rot=q_rot, k_rows=kc[ROWS], v_rows=vc[ROWS])
    print("wrote config0_expected.npz; out[0,:4] =", out[0, :4])


if __name__ == "__main__":
    main()
