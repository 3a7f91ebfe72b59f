"""Shared test helpers: seeded inputs in the shapes of the benchmark configurations and error metrics."""
import numpy as np

THETA_QWEN3 = 1.0e6          # Qwen3 rope_theta
THETA_LLAMA3 = 5.0e5


def normal_f16(rng, shape):
    """N(0,1) drawn from the generator, cast to fp16 and widened back (the configurations' "cast to fp16")."""
    return rng.standard_normal(shape, dtype=np.float32).astype(np.float16).astype(np.float32)


def rng_for(seed):
    return np.random.Generator(np.random.PCG64(seed))


def max_rel_err(got, ref):
    """max |got-ref| / max(|ref|, 1e-3 * max|ref|): relative error with a floor so near-zero outputs do not
    dominate (attention outputs cross zero)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    floor = 1e-3 * np.max(np.abs(ref)) + 1e-30
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), floor)))


def attention_err(got, ref):
    """Error metric of the 2e-3 bound: |got-ref| relative to the largest output magnitude of the same head row
    (the reference's own f16-KV test bounds the absolute error of O(0.1)-sized outputs by 2e-3,
    Tests/EdgeRunnerMetalTests/GQATests.swift:431-433)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    scale = np.max(np.abs(ref), axis=-1, keepdims=True) + 1e-30
    return float(np.max(np.abs(got - ref) / scale))


def outlier_channels(rng, shape_channels, frac=0.01, factor=20.0):
    """Per-channel scale vector: Bernoulli(frac) channels multiplied by `factor` (configuration 2)."""
    mask = rng.random(shape_channels) < frac
    return np.where(mask, factor, 1.0).astype(np.float32)
