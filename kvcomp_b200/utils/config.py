"""The reference's configuration object (utils/config.py:21-140) and its global holder
(models/cache/kvcomp_quant.py:10-12), with the same fields, str()/from_str() round trip, equality and
hash.  Two optional fields are added; left at None, each cache class follows the reference class it
replaces (KVCompCtx: the CUDA path's batch-spanning units and int8 min_ints; KVCompCache: the model
path's per-sequence units and un-narrowed min_ints)."""
from .compute import QuantMode


class ExtractCacheConfig:       # utils/config.py:3-19
    def __init__(self, collect_round):
        self.collect_round = collect_round
        self.key_caches = {}
        self.value_caches = {}

    def size(self):
        total = 0
        for per_round in list(self.key_caches.values()) + list(self.value_caches.values()):
            for t in per_round.values():
                total += t.numel() * 16
        return total


class KVCompCacheConfig:
    _FIELDS = ("enable_quant", "model_name", "enable_pre_rope", "k_quant_mode", "v_quant_mode", "k_block_size",
               "v_block_size", "k_recent_size", "v_recent_size", "k_quant_scale_rel", "v_quant_scale_rel")

    def __init__(self, model_name, k_quant_mode, v_quant_mode, k_block_size, v_block_size, k_recent_size,
                 v_recent_size, k_quant_scale_rel, v_quant_scale_rel, enable_quant=True, enable_pre_rope=False,
                 quant_per_sequence=None, wide_min_ints=None):
        self.enable_quant = enable_quant
        self.model_name = model_name
        self.enable_pre_rope = enable_pre_rope
        self.k_quant_mode = k_quant_mode
        self.v_quant_mode = v_quant_mode
        self.k_block_size = k_block_size
        self.v_block_size = v_block_size
        self.k_recent_size = k_recent_size
        self.v_recent_size = v_recent_size
        self.k_quant_scale_rel = k_quant_scale_rel
        self.v_quant_scale_rel = v_quant_scale_rel
        # additions (None = the default of the cache class in use): quant units per sequence
        # (utils/compute.py:138-143) or spanning the batch (models/cache/kvcomp_encode.py:10-13);
        # int16 or int8 (kvcomp_encode.py:97) min_ints
        self.quant_per_sequence = quant_per_sequence
        self.wide_min_ints = wide_min_ints

    def __str__(self):
        d = {"enable_quant": self.enable_quant, "enable_pre_rope": self.enable_pre_rope, "model_name": self.model_name}
        if self.enable_quant:
            d.update(k_quant_mode=self.k_quant_mode.value, v_quant_mode=self.v_quant_mode.value,
                     k_block_size=self.k_block_size, v_block_size=self.v_block_size,
                     k_recent_size=self.k_recent_size, v_recent_size=self.v_recent_size,
                     k_quant_scale_rel=self.k_quant_scale_rel, v_quant_scale_rel=self.v_quant_scale_rel)
        return str(d)

    __repr__ = __str__

    @staticmethod
    def from_str(text):
        import ast
        d = ast.literal_eval(text)
        on = d["enable_quant"]
        return KVCompCacheConfig(
            model_name=d["model_name"], enable_quant=on, enable_pre_rope=d["enable_pre_rope"],
            k_quant_mode=QuantMode(d["k_quant_mode"]) if on else None,
            v_quant_mode=QuantMode(d["v_quant_mode"]) if on else None,
            k_block_size=d["k_block_size"] if on else None, v_block_size=d["v_block_size"] if on else None,
            k_recent_size=d["k_recent_size"] if on else None, v_recent_size=d["v_recent_size"] if on else None,
            k_quant_scale_rel=d["k_quant_scale_rel"] if on else None,
            v_quant_scale_rel=d["v_quant_scale_rel"] if on else None)

    def _key(self):
        return tuple(getattr(self, f) for f in self._FIELDS)

    def __eq__(self, other):
        return isinstance(other, KVCompCacheConfig) and self._key() == other._key()

    def __hash__(self):
        return hash(self._key())


class KVCompCacheConfigStatic:  # models/cache/kvcomp_quant.py:10-12
    config = None
    extract_cache = None
