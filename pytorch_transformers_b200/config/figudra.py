"""Configuration of the Figudra design: a decoder whose layers are listed one by one. Every layer is a parallel block
(one RMS norm; the mixer and the feed-forward both read its output) with one of three mixers: ``gla`` (a gated linear
attention whose decay is computed per key channel from the layer's input), ``attention`` (grouped heads, no rotation, a
query temperature that grows with the position, soft-capped scores, a sigmoid gate on the heads) and ``attention_2``
(normed queries and keys, a rotation of part of each head with linearly scaled frequencies, a sliding window that keeps a
sequence's first tokens, a softmax with one added to its denominator). The feed-forward is a dense gated unit or a mixture
of gated experts with a group-limited sigmoid router and a gated shared expert; a layer may have none. A layer with
``weights_of: j`` runs layer j's weights on a cache and state of its own.

config.json keys: ``architecture`` ("Figudra"), ``vocab``, ``width``, ``norm.eps`` and ``layers``: a list of
``{"type", "mixer": {...}, "mlp": {...} | null[, "weights_of": j]}``. A ``gla`` mixer gives ``heads, dim, vdim, tau``; an
``attention`` mixer ``heads, kv_heads, dim, vdim, scale[, softcap][, q_temp: {coef, every}]``; an ``attention_2`` mixer
``heads, kv_heads, dim, vdim, scale[, mask: {size, keep_first}][, rot: {base, dims[, scaling: {factor}]}]``. An ``mlp`` of
kind ``dense`` gives ``ff``; of kind ``moe`` ``expert: {ff}``, ``router: {experts, top, scale, groups: {count, keep}}`` and
optionally ``shared: {ff}``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, List

from .base import ModelConfig, _require
from .pafevik import _positive_int

MIXERS = ("gla", "attention", "attention_2")


def _whole(v: Any) -> bool:
    """An integer, also one that JSON wrote as 64.0."""
    return (isinstance(v, int) and not isinstance(v, bool)) or (isinstance(v, float) and v.is_integer())


def _check_mixer(kind: str, m: Dict[str, Any], where: str) -> None:
    _require(isinstance(m, dict), f"{where}.mixer must be an object")
    for key in ("heads", "dim", "vdim"):
        _positive_int(m.get(key), f"{where}.mixer.{key}")
    if kind == "gla":
        _require(float(m.get("tau", 0)) > 0, f"{where}.mixer.tau must be positive")
        return
    _positive_int(m.get("kv_heads"), f"{where}.mixer.kv_heads")
    _require(m["heads"] % m["kv_heads"] == 0, f"{where}.mixer.heads must be a multiple of kv_heads")
    _require(float(m.get("scale", 0)) > 0, f"{where}.mixer.scale must be positive")
    if kind == "attention":
        _require(float(m.get("softcap") or 0) >= 0, f"{where}.mixer.softcap must not be negative")
        temp = m.get("q_temp")
        if temp is not None:
            _require(isinstance(temp, dict) and _whole(temp.get("every")) and temp["every"] > 0
                     and isinstance(temp.get("coef"), (int, float)),
                     f"{where}.mixer.q_temp must give a number coef and a positive integer every")
        return
    mask = m.get("mask") or {}
    _require(isinstance(mask, dict), f"{where}.mixer.mask must be an object")
    size, keep = mask.get("size", 0), mask.get("keep_first", 0)
    _require(_whole(size) and size >= 0 and _whole(keep) and keep >= 0,
             f"{where}.mixer.mask.size and keep_first must be integers >= 0")
    rot = m.get("rot") or {}
    dims = rot.get("dims", 0)
    _require(_whole(dims) and 0 <= dims <= m["dim"] and dims % 2 == 0,
             f"{where}.mixer.rot.dims must be even and at most dim")
    _require(dims == 0 or float(rot.get("base", 0)) > 0, f"{where}.mixer.rot.base must be positive")
    sc = rot.get("scaling")
    _require(sc is None or (isinstance(sc, dict) and float(sc.get("factor", 0)) > 0),
             f"{where}.mixer.rot.scaling.factor must be positive")


def _check_mlp(mlp: Dict[str, Any], where: str) -> None:
    _require(isinstance(mlp, dict) and mlp.get("kind") in ("dense", "moe"), f"{where}.mlp.kind must be 'dense' or 'moe'")
    if mlp["kind"] == "dense":
        _positive_int(mlp.get("ff"), f"{where}.mlp.ff")
        return
    _require(isinstance(mlp.get("expert"), dict), f"{where}.mlp.expert must be an object")
    _positive_int(mlp["expert"].get("ff"), f"{where}.mlp.expert.ff")
    r = mlp.get("router")
    _require(isinstance(r, dict), f"{where}.mlp.router must be an object")
    _positive_int(r.get("experts"), f"{where}.mlp.router.experts")
    _positive_int(r.get("top"), f"{where}.mlp.router.top")
    groups = r.get("groups") or {"count": 1, "keep": 1}
    _require(isinstance(groups, dict), f"{where}.mlp.router.groups must be an object")
    count, keep = groups.get("count", 1), groups.get("keep", 1)
    _positive_int(count, f"{where}.mlp.router.groups.count")
    _positive_int(keep, f"{where}.mlp.router.groups.keep")
    _require(r["experts"] % count == 0 and keep <= count and r["top"] <= r["experts"] // count * keep,
             f"{where}.mlp.router: cannot choose {r['top']} of {r['experts']} experts in {keep} of {count} groups")
    if mlp.get("shared") is not None:
        _require(isinstance(mlp["shared"], dict), f"{where}.mlp.shared must be an object")
        _positive_int(mlp["shared"].get("ff"), f"{where}.mlp.shared.ff")


@dataclasses.dataclass
class FigudraConfig(ModelConfig):
    model_type: ClassVar[str] = "figudra"

    architecture: str = "Figudra"
    vocab: int = 0
    width: int = 0
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    norm: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    tie_word_embeddings: bool = False        # the head is a tensor of its own

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _require(isinstance(self.layers, list) and len(self.layers) > 0, "layers must be a non-empty list")
        _require(isinstance(self.norm, dict) and float(self.norm.get("eps", 0)) > 0, "norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _require(isinstance(layer, dict) and layer.get("type") in MIXERS,
                     f"{where}.type must be one of {', '.join(MIXERS)}, got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            _check_mixer(layer["type"], layer.get("mixer"), where)
            if layer.get("mlp") is not None:
                _check_mlp(layer["mlp"], where)
            j = layer.get("weights_of")
            if j is not None:
                _require(isinstance(j, int) and not isinstance(j, bool) and 0 <= j < len(self.layers) and j != i
                         and isinstance(self.layers[j], dict) and self.layers[j].get("weights_of") is None,
                         f"{where}.weights_of must name another layer that has weights of its own, got {j!r}")
                same = all(layer.get(k) == self.layers[j].get(k) for k in ("type", "mixer", "mlp"))
                _require(same, f"{where} uses the weights of layer {j} and must equal it in type, mixer and mlp")

    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer ``i`` runs."""
        j = self.layers[i].get("weights_of")
        return i if j is None else int(j)

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
