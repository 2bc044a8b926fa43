"""Pogezen as an assembly of parts: PogezenConfig -> ModelSpec, with the checkpoint's tensor names.

Every layer is a pre-norm ``sequential`` block of Dynamic Tanh norms around a mixer and, unless its ``mlp`` is
null, a ``dense`` feed-forward with a squared relu. The mixer is an ``input_conv`` (the short convolution that is
added to the mixer's input, ``l<i>.canon1``) around an ``mlstm`` or around a ``sink_attention`` with biases, a YaRN
rotation on part of each head, queries and keys divided by their root mean square after the rotation, a window
that keeps the first tokens, softmax weights mixed across heads and, in layers that say ``v_mix``, values mixed
with those of the first such layer. The embeddings are scaled; the residual stream is float32; the head is the
embedding table. Tensor names: ``embed``, ``l<i>.norm1|norm2`` (+ ``.b``, ``.alpha``), ``l<i>.canon1``,
``l<i>.mix.*``, ``l<i>.mlp.up|down``, ``final.norm`` (+ ``.b``, ``.alpha``).
"""
from __future__ import annotations

from ..config.pogezen import PogezenConfig
from ..parts.base import ModelSpec, PartSpec


def _norm(cfg: PogezenConfig, name: str) -> PartSpec:
    return PartSpec("norm", "dyt", {"size": cfg.width}, names={"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})


def _mixer(cfg: PogezenConfig, i: int, first_mix) -> PartSpec:
    layer = cfg.layers[i]
    m, p, eps = layer["mixer"], f"l{i}.mix.", float(cfg.norm["eps"])
    if layer["type"] == "mlstm":
        names = {n: p + n for n in ("q", "k", "v", "g", "o", "norm", "i", "f")}
        names.update({"i_b": p + "i.b", "f_b": p + "f.b"})
        return PartSpec("mixer", "mlstm", {"hidden": cfg.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                           "gate_cap": float(m["gate_cap"]), "eps": eps}, names=names)
    mask, rot = m.get("mask") or {}, m.get("rot") or {}
    children = {}
    if int(rot.get("dims", 0)) > 0:
        # without a scaling the frequencies are the plain ones: a factor of 1 leaves them as they are
        sc = rot.get("scaling") or {"factor": 1.0, "original": 1.0, "fast": 1.0, "slow": 1.0}
        children["position"] = PartSpec("position", "rotary",
                                        {"head_dim": m["dim"], "theta": float(rot["base"]), "rotary_dim": int(rot["dims"]),
                                         "yarn": {key: float(sc[key]) for key in ("factor", "original", "fast", "slow")}})
    value_mix = "none" if not m.get("v_mix") else ("source" if i == first_mix else "mix")
    names = {n: p + n for n in ("q", "k", "v", "o", "talk")}
    names.update({n + "_b": p + n + ".b" for n in ("q", "k", "v", "o")})
    if value_mix != "none":
        names["vmix"] = p + "vmix"
    return PartSpec("mixer", "sink_attention",
                    {"hidden": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                     "scale": float(m["scale"]), "window": int(mask.get("size", 0)), "eps": eps, "qk_norm": True,
                     "qk_gain": False, "sink": False, "gate": False, "bias": True,
                     "keep_first": int(mask.get("keep_first", 0)) if int(mask.get("size", 0)) > 0 else 0, "talk": True,
                     "value_mix": value_mix}, children=children, names=names)


def pogezen_block(cfg: PogezenConfig, i: int, first_mix) -> PartSpec:
    mixer = PartSpec("mixer", "input_conv", {"hidden": cfg.width, "taps": int(cfg.canon.get("taps", 1))},
                     children={"inner": _mixer(cfg, i, first_mix)}, names={"conv": f"l{i}.canon1"})
    children = {"norm_mixer": _norm(cfg, f"l{i}.norm1"), "mixer": mixer}
    mlp = cfg.layers[i].get("mlp")
    if mlp is not None:
        children["norm_ff"] = _norm(cfg, f"l{i}.norm2")
        children["feed_forward"] = PartSpec("feed_forward", "dense", {"hidden": cfg.width, "inner": mlp["ff"], "activation": "relu2"},
                                            names={"up.weight": f"l{i}.mlp.up", "down.weight": f"l{i}.mlp.down"})
    return PartSpec("block", "sequential", children=children)


def pogezen_spec(cfg: PogezenConfig) -> ModelSpec:
    mixing = [i for i, layer in enumerate(cfg.layers) if layer["type"] == "attention" and layer["mixer"].get("v_mix")]
    first_mix = mixing[0] if mixing else None
    return ModelSpec(vocab_size=cfg.vocab, hidden_size=cfg.width, embedding_name="embed",
                     blocks=[pogezen_block(cfg, i, first_mix) for i in range(len(cfg.layers))],
                     final_norm=_norm(cfg, "final.norm"), head_name=None,
                     embedding_scale=float(cfg.embedding.get("scale", 1.0)), stream_float32=True)
