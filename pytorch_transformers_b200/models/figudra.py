"""Figudra as an assembly of parts: FigudraConfig -> ModelSpec, with the checkpoint's tensor names.

Every layer is a ``parallel`` block with one RMS norm whose output both the mixer and the feed-forward read. The mixer
is a ``gla`` (gated linear attention with a decay per key channel) or a ``sink_attention`` in one of two settings:
``attention`` (no rotation, query temperature, soft-capped scores, a sigmoid gate per entry of the heads) and
``attention_2`` (normed queries and keys with gains before a rotation of part of each head with linearly scaled
frequencies, a window that keeps the first tokens, a sink of value 0). The feed-forward is a ``gated`` unit with the tanh
form of GELU or ``routed_experts`` with sigmoid scores, groups scored by their two best, normalised weights and a gated
shared expert; a layer may have none. A layer with ``weights_of: j`` is one more schedule entry of block j with a cache
entry of its own. The embeddings are normed; the residual stream is float32; the head is a tensor of its own.
Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.figudra import FigudraConfig
from ..parts.base import ModelSpec, PartSpec, ScheduleEntry

SINK_VALUE = 0.0        # attention_2's softmax has one added to its denominator: a sink whose score is 0


def _norm(cfg: FigudraConfig, name: str) -> PartSpec:
    return PartSpec("norm", "rmsnorm", {"size": cfg.width, "eps": float(cfg.norm["eps"])}, names={"weight": name})


def _mixer(cfg: FigudraConfig, i: int) -> PartSpec:
    layer = cfg.layers[i]
    m, p, eps = layer["mixer"], f"l{i}.mix.", float(cfg.norm["eps"])
    if layer["type"] == "gla":
        names = {n: p + n for n in ("q", "k", "v", "g", "o", "norm", "a1", "a2")}
        names["a2_b"] = p + "a2.b"
        # the decay's low rank is the size of a tensor; a configuration may name it (`rank`) for weights drawn at random
        return PartSpec("mixer", "gla", {"hidden": cfg.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                         "tau": float(m["tau"]), "eps": eps, "rank": m.get("rank")}, names=names)
    common = {"hidden": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
              "scale": float(m["scale"]), "eps": eps, "sink": False}
    if layer["type"] == "attention":
        temp = m.get("q_temp")
        return PartSpec("mixer", "sink_attention",
                        dict(common, qk_norm=False, gate=True, gate_wide=True, softcap=float(m.get("softcap") or 0.0),
                             q_temp=(float(temp["coef"]), int(temp["every"])) if temp else None),
                        names={n: p + n for n in ("q", "k", "v", "g", "o")})
    mask, rot = m.get("mask") or {}, m.get("rot") or {}
    children = {}
    if int(rot.get("dims", 0)) > 0:
        children["position"] = PartSpec("position", "rotary",
                                        {"head_dim": m["dim"], "theta": float(rot["base"]), "rotary_dim": int(rot["dims"]),
                                         "factor": float((rot.get("scaling") or {}).get("factor", 1.0))})
    window = int(mask.get("size", 0))
    names = {n: p + n for n in ("q", "k", "v", "o")}
    names.update({"q_norm": p + "q.norm", "k_norm": p + "k.norm"})
    return PartSpec("mixer", "sink_attention",
                    dict(common, qk_norm=True, qk_gain=True, norm_first=True, gate=False, sink_value=SINK_VALUE, window=window,
                         keep_first=int(mask.get("keep_first", 0)) if window > 0 else 0), children=children, names=names)


def _gated(cfg: FigudraConfig, prefix: str, inner: int, activation: str) -> PartSpec:
    return PartSpec("feed_forward", "gated", {"hidden": cfg.width, "inner": inner, "activation": activation, "wide_out": True},
                    names={n: prefix + n for n in ("gate", "up", "down")})


def _feed_forward(cfg: FigudraConfig, i: int) -> PartSpec:
    mlp, p = cfg.layers[i]["mlp"], f"l{i}.mlp."
    if mlp["kind"] == "dense":
        return _gated(cfg, p, mlp["ff"], "gelu_pytorch_tanh")
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    names = {"router": p + "router"}
    for e in range(r["experts"]):
        for t in ("gate", "up", "down"):
            names[f"e{e}.{t}"] = f"{p}e{e}.{t}"
    children = {}
    if mlp.get("shared") is not None:
        children["shared"] = _gated(cfg, p + "shared.", mlp["shared"]["ff"], "silu")
        names["shared_gate"] = p + "shared.sg"
    return PartSpec("feed_forward", "routed_experts",
                    {"hidden": cfg.width, "inner": mlp["expert"]["ff"], "experts": r["experts"], "top": r["top"],
                     "groups": int(groups.get("count", 1)), "keep": int(groups.get("keep", 1)), "scale": float(r.get("scale", 1.0)),
                     "score": "sigmoid", "correction": False, "group_score": "top2_sum", "normalize": True,
                     "shared_gate": "shared" in children}, children=children, names=names)


def figudra_block(cfg: FigudraConfig, i: int) -> PartSpec:
    children = {"norm_mixer": _norm(cfg, f"l{i}.norm1"), "mixer": _mixer(cfg, i)}
    if cfg.layers[i].get("mlp") is not None:
        children["feed_forward"] = _feed_forward(cfg, i)
    return PartSpec("block", "parallel", children=children)


def figudra_spec(cfg: FigudraConfig) -> ModelSpec:
    own = [i for i in range(len(cfg.layers)) if cfg.weights_layer(i) == i]      # layers with tensors of their own
    block_of = {layer: b for b, layer in enumerate(own)}
    # every layer is a run with a cache entry (pages or state) of its own, also where it runs another layer's weights
    schedule = [ScheduleEntry(block=block_of[cfg.weights_layer(i)], cache_entry=i) for i in range(len(cfg.layers))]
    return ModelSpec(vocab_size=cfg.vocab, hidden_size=cfg.width, embedding_name="embed",
                     blocks=[figudra_block(cfg, i) for i in own], final_norm=_norm(cfg, "final.norm"), head_name="head",
                     schedule=schedule, embedding_norm=_norm(cfg, "embed.norm"), stream_float32=True)
