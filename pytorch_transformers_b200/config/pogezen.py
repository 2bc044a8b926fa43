"""Configuration of the Pogezen design: a decoder whose layers are listed one by one, each with a mixer (a matrix
memory with exponential gates, or an attention with rotated and normed queries and keys, a sliding window that
keeps a sequence's first tokens, softmax weights mixed across heads and values mixed across layers) behind a short
convolution on the mixer's input, and an optional dense feed-forward; all norms are Dynamic Tanh.

config.json keys: ``architecture`` ("Pogezen"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``canon.taps``
and ``layers``: a list of ``{"type", "mixer": {...}, "mlp": {...} | null}``. An ``mlstm`` mixer gives ``heads, dim,
vdim, gate_cap``; an ``attention`` mixer gives ``heads, kv_heads, dim, vdim, scale, mask: {size, keep_first},
rot: {base, dims, scaling: {factor, original, fast, slow}}, v_mix``; an ``mlp`` of kind ``dense`` gives ``ff``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, List

from .base import ModelConfig, _require
from .pafevik import _positive_int

MIXERS = ("mlstm", "attention")


@dataclasses.dataclass
class PogezenConfig(ModelConfig):
    model_type: ClassVar[str] = "pogezen"

    architecture: str = "Pogezen"
    vocab: int = 0
    width: int = 0
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    norm: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    embedding: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"scale": 1.0})
    canon: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"taps": 1})
    tie_word_embeddings: bool = True         # the logits are products with the embedding table itself

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _require(isinstance(self.layers, list) and len(self.layers) > 0, "layers must be a non-empty list")
        _require(isinstance(self.norm, dict) and float(self.norm.get("eps", 0)) > 0, "norm.eps must be positive")
        _require(isinstance(self.embedding, dict) and float(self.embedding.get("scale", 1.0)) != 0, "embedding.scale must not be 0")
        _require(isinstance(self.canon, dict), "canon must be an object")
        taps = self.canon.get("taps", 1)
        _require(isinstance(taps, int) and not isinstance(taps, bool) and 1 <= taps <= 8, f"canon.taps must be 1 to 8, got {taps!r}")
        first_mix = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _require(isinstance(layer, dict) and layer.get("type") in MIXERS,
                     f"{where}.type must be one of {', '.join(MIXERS)}, got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            _require(isinstance(m, dict), f"{where}.mixer must be an object")
            if layer["type"] == "mlstm":
                for key in ("heads", "dim", "vdim"):
                    _positive_int(m.get(key), f"{where}.mixer.{key}")
                _require(float(m.get("gate_cap", 0)) > 0, f"{where}.mixer.gate_cap must be positive")
            else:
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(m.get(key), f"{where}.mixer.{key}")
                _require(m["heads"] % m["kv_heads"] == 0, f"{where}.mixer.heads must be a multiple of kv_heads")
                _require(float(m.get("scale", 0)) > 0, f"{where}.mixer.scale must be positive")
                mask = m.get("mask") or {}
                _require(isinstance(mask, dict), f"{where}.mixer.mask must be an object")
                size, keep = mask.get("size", 0), mask.get("keep_first", 0)
                _require(isinstance(size, int) and size >= 0 and isinstance(keep, int) and keep >= 0,
                         f"{where}.mixer.mask.size and keep_first must be integers >= 0")
                rot = m.get("rot") or {}
                dims = rot.get("dims", 0)
                _require(isinstance(dims, int) and 0 <= dims <= m["dim"] and dims % 2 == 0,
                         f"{where}.mixer.rot.dims must be even and at most dim")
                _require(dims == 0 or float(rot.get("base", 0)) > 0, f"{where}.mixer.rot.base must be positive")
                sc = rot.get("scaling")
                if sc is not None:
                    _require(isinstance(sc, dict) and all(float(sc.get(key, 0)) > 0 for key in ("factor", "original", "fast", "slow")),
                             f"{where}.mixer.rot.scaling must give positive factor, original, fast and slow")
                if m.get("v_mix"):
                    if first_mix is None:
                        first_mix = i
                    else:
                        f = self.layers[first_mix]["mixer"]
                        _require(f["kv_heads"] == m["kv_heads"] and f["vdim"] == m["vdim"],
                                 f"{where}.mixer: kv_heads and vdim must equal those of layer {first_mix}, whose values it mixes in")
            mlp = layer.get("mlp")
            if mlp is not None:
                _require(isinstance(mlp, dict) and mlp.get("kind", "dense") == "dense", f"{where}.mlp.kind must be 'dense'")
                _positive_int(mlp.get("ff"), f"{where}.mlp.ff")

    # the names that the rest of the library uses for the sizes every decoder has
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)
