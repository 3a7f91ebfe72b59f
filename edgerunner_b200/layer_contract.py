"""The per-layer KV format contract of the reference (TurboQuantV2Contract, Sources/EdgeRunnerMetal/TurboQuant.swift:343-536)
as host logic over the CUDA backend: which cache type -- dense (fp16), q8_0, turbo2 / turbo3 / turbo4 -- and which preset
the keys and the values of layer i of n use, and a cache object that follows it.

The reference resolves the contract from process environment variables at every call.  Here it is a value
(`TurboQuantLayerContract`), so the library itself reads no environment; `from_environment(mapping)` builds one from a
mapping with the reference's variable names for callers that want the same knobs.

`PolicyKVCache` keeps one `er_kv` cache per distinct (key type, value type) pair of the model's layers and maps every
layer to (cache, local layer).  Pairs whose two sides belong to different families (q8_0 keys with TurboQuant values,
TurboQuant keys with dense values, ...: the reference's hybrid layers) keep TWO caches of the same geometry, one in the
keys' format and one in the values' -- each stores both of its slabs, so such layers cost one unused slab per side --
and run attention through er_kv_attention_decode_pair (the keys' cache supplies K, the values' cache V)."""
from dataclasses import dataclass
from typing import Mapping, Optional

from . import _lib
from ._lib import EdgeRunnerCUDAError
from .kv_cache import KVCache, Layout, NormFormat, Precision

CACHE_TYPES = ("dense", "q8_0", "turbo2", "turbo3", "turbo4")           # TurboQuantLayerCacheType (:194-229)
FIXED_TYPES = ("turbo2", "turbo3", "turbo4")                             # TurboQuantFixedType (:172-190)
PRESETS = ("turbo2", "turbo3", "turbo4", "planar3", "balanced", "balanced64", "balanced96", "fiveBit", "sixBit", "sevenBit",
           "aggressive", "aggressive64")                                 # TurboQuantPreset raw values
# TurboQuantAdaptiveMode raw values (:232-239)
UNIFORM, FIRST_LAST4_Q8, LAST8_Q8, BOUNDARY_TURBO4, LAST8_TURBO4, BOUNDARY_Q8 = 0, 1, 2, 5, 6, 7


def _is_turbo(cache_type):
    return cache_type in FIXED_TYPES


@dataclass(frozen=True)
class TurboQuantLayerContract:
    key_type: str = "turbo3"                       # keyType / valueType: the fixed types behind the defaults (:344-356)
    value_type: str = "turbo3"
    key_cache_type: Optional[str] = None           # base cache types; None = the fixed type above
    value_cache_type: Optional[str] = None
    early_q8_layers: int = 0                       # the first n layers keep K and V as q8_0
    early_q8_key_layers: int = 0                   # the first n layers keep K as q8_0
    adaptive_mode: Optional[int] = None            # None = inferred: boundaryQ8 when the values are turbo2, else uniform (:656-658)
    key_policy: str = "uniform"                    # uniform | boundaryPromoted | last8Promoted
    value_policy: str = "uniform"                  # uniform | boundaryTurbo4 | last8Turbo4
    key_preset: Optional[str] = None               # preset overrides (None = the fixed type's preset)
    value_preset: Optional[str] = None
    promoted_key_preset: str = "turbo4"

    # ---- resolution ----
    @property
    def resolved_adaptive_mode(self):
        if self.adaptive_mode is not None:
            return self.adaptive_mode
        return BOUNDARY_Q8 if self.value_type == "turbo2" else UNIFORM

    def key_cache_type_for(self, layer, layer_count):
        """keyCacheType(forLayer:layerCount:), :432-457."""
        base = self.key_cache_type or self.key_type
        if self.early_q8_layers > 0 and layer < min(self.early_q8_layers, layer_count) and _is_turbo(base):
            return "q8_0"
        if self.early_q8_key_layers > 0 and layer < min(self.early_q8_key_layers, layer_count) and _is_turbo(base):
            return "q8_0"
        mode = self.resolved_adaptive_mode
        if mode == FIRST_LAST4_Q8 and _is_turbo(base) and layer_count >= 8:
            return "q8_0" if (layer < 4 or layer >= layer_count - 4) else base
        if mode == LAST8_Q8 and _is_turbo(base) and layer_count >= 8:
            return "q8_0" if layer >= layer_count - 8 else base
        return base

    def value_cache_type_for(self, layer, layer_count):
        """valueCacheType(forLayer:layerCount:), :459-488."""
        base = self.value_cache_type or self.value_type
        if self.early_q8_layers > 0 and layer < min(self.early_q8_layers, layer_count) and _is_turbo(base):
            return "q8_0"
        mode = self.resolved_adaptive_mode
        if mode == UNIFORM or not _is_turbo(base) or layer_count < 8:
            return base
        first2_last2 = layer < 2 or layer >= layer_count - 2
        if mode == FIRST_LAST4_Q8:
            return "q8_0" if (layer < 4 or layer >= layer_count - 4) else base
        if mode == LAST8_Q8:
            return "q8_0" if layer >= layer_count - 8 else base
        if mode == BOUNDARY_TURBO4:
            return "turbo4" if first2_last2 else "turbo2"
        if mode == LAST8_TURBO4:
            return "turbo4" if layer >= layer_count - 8 else "turbo2"
        if mode == BOUNDARY_Q8:
            return "q8_0" if first2_last2 else "turbo2"
        return base

    def key_preset_for(self, layer, layer_count):
        """keyPreset(forLayer:layerCount:), :490-506: None for layers whose keys are not TurboQuant rows."""
        cache_type = self.key_cache_type_for(layer, layer_count)
        if not _is_turbo(cache_type):
            return None
        base = self.key_preset or cache_type
        if self.key_policy == "boundaryPromoted" and layer_count >= 8:
            return self.promoted_key_preset if (layer < 2 or layer >= layer_count - 2) else base
        if self.key_policy == "last8Promoted" and layer_count >= 8:
            return self.promoted_key_preset if layer >= layer_count - 8 else base
        return base

    def value_preset_for(self, layer, layer_count):
        """valuePreset(forLayer:layerCount:), :508-530."""
        cache_type = self.value_cache_type_for(layer, layer_count)
        if not _is_turbo(cache_type):
            return None
        if self.resolved_adaptive_mode in (BOUNDARY_TURBO4, LAST8_TURBO4):
            return cache_type
        base = self.value_preset or cache_type
        whole = self.value_preset or self.value_type            # TurboQuantV2Contract.valuePreset, the fallback of short stacks
        if self.value_policy == "boundaryTurbo4":
            if layer_count < 8:
                return whole
            return "turbo4" if (layer < 2 or layer >= layer_count - 2) else base
        if self.value_policy == "last8Turbo4":
            if layer_count < 8:
                return whole
            return "turbo4" if layer >= layer_count - 8 else base
        return base

    @staticmethod
    def residual_scale(preset):
        """residualScale(for:fallbackType:), :670-684: 0 for every preset of the contract."""
        return 0.0

    @classmethod
    def from_environment(cls, env: Mapping[str, str]):
        """The contract the reference would resolve from these variables (TurboQuantEnvOverrides, :3-24); unknown values fall
        back to the defaults as there."""
        def pick(name, allowed, default):
            v = env.get(name)
            return v if v in allowed else default

        def cache_type(name):
            v = env.get(name)
            if v is None:
                return None
            v = v.lower()
            return {"dense": "dense", "f16": "dense", "q8_0": "q8_0", "turbo2": "turbo2", "turbo3": "turbo3", "turbo4": "turbo4"}.get(v)

        def integer(name):
            try:
                return int(env.get(name, "0"))
            except ValueError:
                return 0

        mode = None
        raw = env.get("TURBO_LAYER_ADAPTIVE", env.get("EDGERUNNER_TURBOQUANT_LAYER_ADAPTIVE"))
        if raw is not None:
            try:
                if int(raw) in (UNIFORM, FIRST_LAST4_Q8, LAST8_Q8, BOUNDARY_TURBO4, LAST8_TURBO4, BOUNDARY_Q8):
                    mode = int(raw)
            except ValueError:
                pass
        return cls(key_type=pick("EDGERUNNER_TURBOQUANT_KEY_TYPE", FIXED_TYPES, "turbo3"),
                   value_type=pick("EDGERUNNER_TURBOQUANT_VALUE_TYPE", FIXED_TYPES, "turbo3"),
                   key_cache_type=cache_type("EDGERUNNER_TURBOQUANT_KEY_CACHE_TYPE"),
                   value_cache_type=cache_type("EDGERUNNER_TURBOQUANT_VALUE_CACHE_TYPE"),
                   early_q8_layers=integer("EDGERUNNER_TURBOQUANT_EARLY_Q8_LAYERS"),
                   early_q8_key_layers=integer("EDGERUNNER_TURBOQUANT_EARLY_Q8_KEY_LAYERS"),
                   adaptive_mode=mode,
                   key_policy=pick("EDGERUNNER_TURBOQUANT_KEY_POLICY", ("uniform", "boundaryPromoted", "last8Promoted"), "uniform"),
                   value_policy=pick("EDGERUNNER_TURBOQUANT_VALUE_POLICY", ("uniform", "boundaryTurbo4", "last8Turbo4"), "uniform"),
                   key_preset=pick("EDGERUNNER_TURBOQUANT_KEY_PRESET", PRESETS, None),
                   value_preset=pick("EDGERUNNER_TURBOQUANT_VALUE_PRESET", PRESETS, None),
                   promoted_key_preset=pick("EDGERUNNER_TURBOQUANT_PROMOTED_KEY_PRESET", PRESETS, "turbo4"))


_BITS = {"turbo2": 2, "turbo3": 3, "turbo4": 4}


def cache_arguments(key_type, value_type):
    """(Precision, extra KVCache arguments) of a layer whose keys / values use these cache types, or None when the pair has
    no kernel here (its sides belong to different families)."""
    if key_type == "dense" and value_type == "dense":
        return Precision.float16, {}
    if key_type == "q8_0" and value_type == "q8_0":
        return Precision.q8_0, {}
    if key_type in _BITS and value_type in _BITS:
        return Precision.turboquantV2, dict(key_type=_BITS[key_type], value_type=_BITS[value_type])
    return None


def _side_arguments(cache_type):
    """A cache whose rows of BOTH sides use `cache_type` (one side of a mixed-family layer reads only its own slab)."""
    return cache_arguments(cache_type, cache_type)


class PolicyKVCache:
    """One cache (or, for mixed-family layers, one pair of caches) per (key type, value type) pair of a layer stack that
    follows a TurboQuantLayerContract."""

    def __init__(self, max_seq_len, num_layers, num_kv_heads, head_dim, contract=None, *, max_batch=1, layout=Layout.head_major,
                 norm_format=NormFormat.float32, page_size=0, num_pages=0):
        self.contract = contract or TurboQuantLayerContract()
        self.num_layers = num_layers
        self.layer_types = [(self.contract.key_cache_type_for(l, num_layers), self.contract.value_cache_type_for(l, num_layers))
                            for l in range(num_layers)]
        groups = {}
        for layer, pair in enumerate(self.layer_types):
            groups.setdefault(pair, []).append(layer)

        def make(precision, extra, count):
            return KVCache(max_seq_len, count, num_kv_heads, head_dim, precision, max_batch=max_batch, layout=layout,
                           norm_format=norm_format, page_size=page_size, num_pages=num_pages, **extra)

        self._caches, self._slot = {}, {}
        for pair, layers in groups.items():
            whole = cache_arguments(*pair)
            if whole is not None:
                caches = (make(whole[0], whole[1], len(layers)),)
            else:
                caches = tuple(make(*_side_arguments(t), len(layers)) for t in pair)     # (keys' cache, values' cache)
            self._caches[pair] = caches
            for local, layer in enumerate(layers):
                self._slot[layer] = (caches, local)

    def close(self):
        for caches in self._caches.values():
            for c in caches:
                c.close()

    @property
    def caches(self):
        """{(key type, value type): (cache,) or (keys' cache, values' cache)}."""
        return dict(self._caches)

    def layers_of(self, pair):
        return [l for l, p in enumerate(self.layer_types) if p == pair]

    def is_mixed(self, layer):
        return len(self.at(layer)[0]) == 2

    def at(self, layer):
        """((cache,) or (keys' cache, values' cache), local layer index) of a model layer."""
        if not 0 <= layer < self.num_layers:
            raise EdgeRunnerCUDAError(_lib.ER_ERR_INVALID_LAYER, "layer %d" % layer)
        return self._slot[layer]

    def write_rows(self, layer, seq, start, count, k, v, params, stream=None):
        caches, local = self.at(layer)
        for c in caches:
            c.write_rows(local, seq, start, count, k, v, params, stream=stream)

    def decode_step(self, layer, q, k, v, out, num_heads, params, stream=None):
        """One layer's step (the per-layer dispatch of fusedDecodePass): q [batch, heads, 128], k / v [batch, kv heads, 128]."""
        caches, local = self.at(layer)
        if len(caches) == 1:
            caches[0].decode_step(q, k, v, out, num_heads, params, layer_begin=local, layer_end=local + 1, stream=stream)
            return
        kc, vc = caches
        for c in caches:           # each side quantises the step's rows into its own format
            c.append_rope_kv(k, v, params, layer_begin=local, layer_end=local + 1, stream=stream)
        kc.attention_decode_with_values_of(vc, q, out, num_heads, params, pending=1, layer_begin=local, layer_end=local + 1, stream=stream)
        for c in caches:
            c.advance(1, layer_begin=local, layer_end=local + 1, stream=stream)

    def attention_prefill(self, layer, seq, q, out, num_heads, seq_len, params, q_offset=None, stream=None):
        caches, local = self.at(layer)
        if len(caches) == 1:
            caches[0].attention_prefill(local, seq, q, out, num_heads, seq_len, params, q_offset=q_offset, stream=stream)
        else:
            caches[0].attention_prefill_with_values_of(caches[1], local, seq, q, out, num_heads, seq_len, params, q_offset=q_offset, stream=stream)

    def set_block_table(self, seq, pages):
        for caches in self._caches.values():
            for c in caches:
                c.set_block_table(seq, pages)

    def reset(self):
        for caches in self._caches.values():
            for c in caches:
                c.reset()
