"""edgerunner_b200: B200 (sm_100a) backend for EdgeRunner's decode-time KV-cache path.

Hand-written CUDA kernels behind a C ABI (include/er_kv.h, built into edgerunner_b200/lib/liber_kv.so) plus
this thin host-side mirror of the reference's KVCache / kernel-holder classes.  Nothing here computes on
the CPU: if the shared library is missing, `lib()` raises.
"""
from ._lib import EdgeRunnerCUDAError, lib  # noqa: F401
from .block_table import BlockTableAllocator, OutOfPages  # noqa: F401
from .layered_cache import HeterogeneousKVCache  # noqa: F401
from .layer_contract import PolicyKVCache, TurboQuantLayerContract  # noqa: F401
from .kernels import Gemma4DecodeKernels, GQAKernel, RoPEKernel, TurboQuantKernel, Q8Kernel  # noqa: F401
from .kv_cache import (ALL_SEQUENCES, KVCache, Layout, NormFormat, OutlierSelection, Precision, TurboQuantFixedType,  # noqa: F401
                       step_params)
