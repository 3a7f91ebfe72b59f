"""Per-layer head sizes and KV-shared layers over the CUDA backend: the host-side mirror of the reference's heterogeneous
initializer, KVCache.init(device:maxSeqLen:numKVHeads:headDimByLayer:kvSourceLayers:precision:)
(Sources/EdgeRunnerMetal/KVCache.swift:276-392), which Gemma-4-style models use: layers differ in head_dim, and a layer may
alias the K/V buffers of an earlier layer that owns them.

An `er_kv` cache holds layers of one shape, so this class keeps one token-major cache (the reference's [slot][kvHead][dim]
ring) per distinct head_dim, holding the OWNING layers of that size, and maps every layer to (cache, local layer); a shared
layer maps to its source's slot -- the same bytes, as in the reference, where the alias shares the MTLBuffer.  Validation and
error cases follow the Swift initializer (every violation is KVCacheError.unsupportedStorage).  Attention over such layers
goes through the raw-buffer operators (GQAKernel / Gemma4DecodeKernels), which take any even head size up to 512, on the
device buffers this class hands out -- the division of labour the reference has between KVCache and its kernel holders."""
import numpy as np

from . import _lib
from ._lib import EdgeRunnerCUDAError
from .kv_cache import KVCache, Layout, Precision


class HeterogeneousKVCache:
    def __init__(self, max_seq_len, num_kv_heads, head_dim_by_layer, kv_source_layers, precision):
        head_dim_by_layer, kv_source_layers = [int(d) for d in head_dim_by_layer], [int(s) for s in kv_source_layers]
        n = len(head_dim_by_layer)

        def refuse(why):
            raise EdgeRunnerCUDAError(_lib.ER_ERR_UNSUPPORTED_STORAGE, why)

        if n == 0 or len(kv_source_layers) != n:
            refuse("headDimByLayer and kvSourceLayers must be non-empty and of equal length")
        for layer, source in enumerate(kv_source_layers):
            if not 0 <= source < n:
                refuse("source layer %d of layer %d is out of range" % (source, layer))
            if source != layer:
                if source > layer:
                    refuse("layer %d shares a later layer (%d)" % (layer, source))
                if kv_source_layers[source] != source:
                    refuse("layer %d shares layer %d, which does not own its buffers" % (layer, source))
                if head_dim_by_layer[layer] != head_dim_by_layer[source]:
                    refuse("layer %d and its source %d differ in head_dim" % (layer, source))
        precision = Precision(precision)
        if precision not in (Precision.float32, Precision.float16):
            refuse("heterogeneous layouts are dense (float32 / float16) only")
        self.max_seq_len, self.num_layers, self.num_kv_heads = max_seq_len, n, num_kv_heads
        self.head_dim_by_layer, self.kv_source_layers, self.precision = head_dim_by_layer, kv_source_layers, precision
        # headDim = the most common per-layer size, the first one on ties (dominantHeadDim, KVCache.swift:394-408)
        counts = {}
        for d in head_dim_by_layer:
            counts[d] = counts.get(d, 0) + 1
        best = max(counts.values())
        self.head_dim = next(d for d in head_dim_by_layer if counts[d] == best)
        owners = {}                                   # head_dim -> owning layers, in layer order
        for layer, source in enumerate(kv_source_layers):
            if source == layer:
                owners.setdefault(head_dim_by_layer[layer], []).append(layer)
        self._caches = {d: KVCache(max_seq_len, len(ls), num_kv_heads, d, precision, layout=Layout.token_major) for d, ls in owners.items()}
        self._slot = {}
        for d, ls in owners.items():
            for local, layer in enumerate(ls):
                self._slot[layer] = (self._caches[d], local)
        for layer, source in enumerate(kv_source_layers):
            self._slot[layer] = self._slot[source]

    def close(self):
        for c in self._caches.values():
            c.close()

    def _at(self, layer):
        if not 0 <= layer < self.num_layers:
            raise EdgeRunnerCUDAError(_lib.ER_ERR_INVALID_LAYER, "layer %d" % layer)
        return self._slot[layer]

    def head_dim_for_layer(self, layer):              # headDim(forLayer:)
        self._at(layer)
        return self.head_dim_by_layer[layer]

    def owns_buffers(self, layer):
        self._at(layer)
        return self.kv_source_layers[layer] == layer

    def elements_per_token(self, layer):
        return self.num_kv_heads * self.head_dim_for_layer(layer)

    @property
    def current_length(self):
        return max(c.current_length for c in self._caches.values())

    def append(self, layer, keys, values):
        cache, local = self._at(layer)
        cache.append(local, keys, values)

    def append_f16(self, layer, keys, values):
        cache, local = self._at(layer)
        cache.append_f16(local, keys, values)

    def retrieve(self, layer, as_type):
        cache, local = self._at(layer)
        return cache.retrieve(local, as_type)

    def metal_buffers(self, layer):
        """(key, value) device addresses of the layer's ring -- a shared layer returns its source's."""
        cache, local = self._at(layer)
        return cache.metal_buffers(local)

    def cache_params(self, layer):
        cache, local = self._at(layer)
        return cache.cache_params(local)

    def reset(self):
        for c in self._caches.values():
            c.reset()

    def set_position(self, position):
        for c in self._caches.values():
            c.set_position(position)

    def advance_write_position(self, layer, count):
        cache, local = self._at(layer)
        cache.advance_write_position(local, count)
