"""Small Figudra configurations and seeded weights for the tests (test-side code only).

The configurations differ from one another in every size: head counts and groupings, key and value sizes that differ
from each other and are no multiple of 8, windows shorter than a page, longer than a page and longer than any prompt,
kept first tokens from none to more than a page, rotations over a part of a head, over all of it and none, with and
without scaling, soft caps and query temperatures present and absent, decays through ranks of 1 to 32 and exponents
1 / tau from 1 to 1 / 16, routers with one group and with several, with and without a shared expert, dense and routed
feed-forwards and none, layers that run another layer's weights, and every order of the three mixers. "ones" sets to 1
what can be 1. Weights are drawn so that every tensor matters: norm gains away from 1, decay biases that spread the
decays over (0, 1), router rows large enough that the choice differs from token to token and small enough that the
scores stay apart.
"""
from __future__ import annotations

import os

import numpy as np
import torch

import tiny_models as tm


def gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}}


def att(heads, kv_heads, dim, vdim, scale, softcap=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m}


def att2(heads, kv_heads, dim, vdim, scale, window=0, keep=0, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    if rot is not None:
        r = {"base": rot[1], "dims": rot[0]}
        if len(rot) > 2:
            r["scaling"] = {"factor": rot[2]}
        m["rot"] = r
    return {"type": "attention_2", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, count=1, keep=1, scale=1.0, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _cfg(vocab, width, eps, layers):
    out = []
    for layer in layers:
        if isinstance(layer, int):          # this layer runs the weights of that one
            out.append(dict(out[layer], weights_of=layer))
        else:
            mixer, mlp = layer
            out.append(dict(mixer, mlp=mlp))
    return {"architecture": "Figudra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out}


CONFIGS = {
    # the capped attention first; layers that run again with the weights of another; a layer without feed-forward; windows
    # shorter and longer than a page; rotation over a part and over all of a head
    "mixed": _cfg(211, 96, 1e-5, [
        (att(6, 2, 24, 20, 0.6, softcap=4.0, q_temp=(0.7, 16)), moe(6, 2, 40, count=3, keep=2, scale=1.5, shared=24)),
        (gla(3, 16, 40, 4.0, 8), dense(80)),
        (att2(4, 2, 16, 20, 0.25, 33, 5, rot=(8, 10000.0, 4.0)), None),
        1,
        (att2(2, 1, 32, 8, 0.2, 70, 0, rot=(32, 500.0)), moe(4, 3, 24)),
        0,
    ]),
    # sizes that are no multiple of 8 or of a warp; the linear attention first; more kept tokens than a page holds;
    # an attention without cap and temperature; a router with one group
    "odd": _cfg(97, 52, 1e-6, [
        (gla(2, 6, 10, 1.0, 3), dense(30)),
        (att2(5, 5, 10, 14, 0.3, 129, 70, rot=(6, 10000.0, 2.0)), moe(5, 2, 18, shared=10)),
        (att(3, 1, 18, 6, 0.3), None),
    ]),
    # whatever can be 1 is 1: one head, a window of one, one kept token, one expert of which one is chosen, rank 1, tau 1,
    # scale 1, a temperature that changes with every position
    "ones": _cfg(64, 32, 1e-6, [
        (att2(1, 1, 16, 16, 1.0 / 16, 1, 1, rot=(2, 10.0)), dense(16)),
        (gla(1, 8, 8, 1.0, 1), moe(1, 1, 16, shared=8)),
        (att(1, 1, 8, 16, 1.0, softcap=1.0, q_temp=(1.0, 1)), None),
    ]),
    # head sizes of the tensor cores; a window longer than every prompt and one of 130; wide linear attentions
    "wide": _cfg(300, 128, 1e-5, [
        (att2(8, 2, 64, 64, 0.1, 130, 4, rot=(32, 100000.0, 8.0)), moe(16, 4, 64, count=4, keep=2, scale=2.5, shared=96)),
        (gla(4, 64, 64, 8.0, 16), dense(200)),
        (att(4, 2, 128, 128, 0.15, softcap=20.0, q_temp=(0.3, 50)), moe(8, 2, 48, count=2, keep=1)),
        (gla(2, 128, 96, 16.0, 32), dense(48)),
        (att2(4, 2, 64, 64, 0.125, 1000, 6, rot=(64, 10000.0)), None),
        2,
    ]),
}


def steady(cfg):
    """The configuration with routers that choose every expert (all groups kept, ``top`` = all): the weights still
    come from the scores, but no choice can fall the other way. A bfloat16 model's stream differs from the plain
    implementation's by about a hundredth, which moves a token's scores by as much; among six to sixteen scores some
    pair at the edge of the choice is that close in one token out of ten, the token then runs other experts, and the
    recurrent layers carry the difference to every later token. Whole models in bfloat16 are compared under these
    routers; the choice itself is compared in float32 whole models and, in both dtypes, on the parts alone, where
    the plain implementation reads the same input rows."""
    import copy
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "moe":
            r = mlp["router"]
            r["top"] = r["experts"]
            r["groups"] = dict(r.get("groups") or {"count": 1}, keep=(r.get("groups") or {"count": 1})["count"])
    return cfg


def tensor_shapes(cfg):
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "embed.norm": (W,), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        H, d, vd = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "gla":
            r = m["rank"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * vd, W), p + "mix.g": (H * vd, W),
                           p + "mix.o": (W, H * vd), p + "mix.norm": (vd,), p + "mix.a1": (r, W), p + "mix.a2": (H * d, r),
                           p + "mix.a2.b": (H * d,)})
        else:
            G = m["kv_heads"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * vd, W), p + "mix.o": (W, H * vd)})
            if layer["type"] == "attention":
                shapes[p + "mix.g"] = (H * vd, W)
            else:
                shapes.update({p + "mix.q.norm": (d,), p + "mix.k.norm": (d,)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            continue
        F = mlp["expert"]["ff"]
        shapes[p + "mlp.router"] = (mlp["router"]["experts"], W)
        for e in range(mlp["router"]["experts"]):
            shapes.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
        if mlp.get("shared") is not None:
            S = mlp["shared"]["ff"]
            shapes.update({p + "mlp.shared.gate": (S, W), p + "mlp.shared.up": (S, W), p + "mlp.shared.down": (W, S),
                           p + "mlp.shared.sg": (1, W)})
    return shapes


def bf16_exact(w):
    """float32 values that a bfloat16 file holds exactly (so both dtypes see one model)."""
    w = np.asarray(w, dtype=np.float32)
    return (tm.to_bf16_bits(w).astype(np.uint32) << 16).view(np.float32).reshape(w.shape)


def make_weights(cfg, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        z = rng.standard_normal(shape).astype(np.float32)
        last = name.split(".")[-1]
        if last in ("norm1", "norm") or name in ("final.norm", "embed.norm"):
            w = 1.0 + 0.2 * z
        elif name.endswith("a2.b"):
            w = 1.0 + 2.0 * z                # decays from nearly closed to nearly open
        elif last == "a2":
            w = 2.0 * z / np.sqrt(shape[-1])
        elif last in ("router", "sg"):
            w = 1.5 * z / np.sqrt(shape[-1])       # sigmoids that do not saturate: few choices within rounding of each other
        elif name == "embed":
            w = 0.7 * z
        else:
            w = 1.2 * z / np.sqrt(shape[-1])
        out[name] = bf16_exact(w)
    return out


def write_folder(tmp, name, seed=0, bf16=False, cfg=None):
    cfg = cfg or CONFIGS[name]
    folder = os.path.join(str(tmp), f"figudra_{name}")
    return tm.write_model_folder(folder, cfg, make_weights(cfg, seed), bf16=bf16)


def torch_weights(cfg, seed, dtype=torch.float64):
    return {k: torch.from_numpy(np.asarray(v)).to(dtype) for k, v in make_weights(cfg, seed).items()}


def prompts(cfg, lengths, seed=0):
    rng = np.random.Generator(np.random.PCG64(700 + seed))
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
