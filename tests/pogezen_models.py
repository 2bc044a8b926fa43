"""Small Pogezen configurations and seeded weights for the tests (test-side code only).

The configurations differ from one another in every size: head counts and groupings, key and value sizes that
differ from each other and are no multiple of 8, values wider than 32 (several stretches of the matrix memory's
columns), windows shorter than a page, longer than a page and longer than any prompt, kept first tokens from none
to more than a page, rotations over a part of a head, over all of it and none, with and without scaling, filters of
one to four taps, layer order (either mixer first), layers with and without feed-forward, value mixing in all, in
some and in a single layer. "ones" sets to 1 what can be 1. Weights are drawn so that every tensor matters: norm
gains and biases away from 1 and 0, the heads' mixing matrix away from the identity, a mixing weight near a third.
"""
from __future__ import annotations

import os

import numpy as np
import torch

import tiny_models as tm


def att(heads, kv_heads, dim, vdim, window, keep, rot=None, scale=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window, "keep_first": keep},
         "scale": scale if scale is not None else 3.0 / dim, "v_mix": v_mix}
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m}


def rot(dims, base=10000.0, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def mem(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _cfg(vocab, width, taps, emb_scale, eps, layers):
    return {"architecture": "Pogezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb_scale},
            "canon": {"taps": taps},
            "layers": [dict(layer, mlp=(None if ff is None else {"kind": "dense", "ff": ff})) for layer, ff in layers]}


CONFIGS = {
    # attention first; windows shorter and longer than a page; rotation over a part and over all of a head; a layer of each
    # kind with and without feed-forward; the last attention mixes no values and rotates nothing
    "mixed": _cfg(211, 96, 3, 2.5, 1e-5, [
        (att(6, 2, 24, 20, 33, 5, rot(8, 10000.0, (4.0, 64, 8.0, 1.0)), v_mix=True), 80),
        (mem(3, 16, 40, 10.0), None),
        (att(4, 2, 16, 20, 70, 1, rot(16, 500.0), v_mix=True), 56),
        (mem(2, 24, 8, 6.0), 64),
        (att(2, 1, 32, 8, 5, 0), None),
    ]),
    # sizes that are no multiple of 8 or of a warp; four taps; the memory first; more kept tokens than a page holds;
    # one layer alone says v_mix (a source without a user)
    "odd": _cfg(97, 52, 4, 1.7, 1e-6, [
        (mem(2, 6, 10, 5.0), 30),
        (att(5, 5, 10, 14, 129, 70, rot(6, 10000.0, (2.0, 32, 4.0, 0.5))), 18),
        (att(3, 1, 18, 6, 7, 3, rot(2, 100.0), v_mix=True), None),
    ]),
    # whatever can be 1 is 1: one head, one tap (no filter state), a window of one, one kept token, scale 1
    "ones": _cfg(64, 32, 1, 1.0, 1e-6, [
        (att(1, 1, 16, 16, 1, 1, rot(2, 10.0), scale=1.0, v_mix=True), 16),
        (mem(1, 8, 8, 1.0), 16),
        (att(1, 1, 8, 16, 2, 0, v_mix=True), None),
    ]),
    # head sizes of the tensor cores; a window longer than every prompt and one of 130; two taps; wide memories
    "wide": _cfg(300, 128, 2, 3.0, 1e-5, [
        (att(8, 2, 64, 64, 130, 4, rot(32, 10000.0, (8.0, 128, 16.0, 2.0)), v_mix=True), 200),
        (mem(4, 64, 64, 15.0), None),
        (att(4, 2, 64, 64, 1000, 6, rot(64, 10000.0), v_mix=True), 96),
        (mem(2, 128, 96, 8.0), 48),
    ]),
}


def tensor_shapes(cfg):
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W)}
    norm = lambda name: {name: (W,), name + ".b": (W,), name + ".alpha": ()}
    shapes.update(norm("final.norm"))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes.update(norm(p + "norm1"))
        shapes[p + "canon1"] = (W, cfg["canon"]["taps"])
        if layer["type"] == "mlstm":
            H, d, vd = m["heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * vd, W), p + "mix.g": (H * vd, W),
                           p + "mix.o": (W, H * vd), p + "mix.norm": (H * vd,), p + "mix.i": (H, W), p + "mix.i.b": (H,),
                           p + "mix.f": (H, W), p + "mix.f.b": (H,)})
        else:
            H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,),
                           p + "mix.v": (G * vd, W), p + "mix.v.b": (G * vd,), p + "mix.talk": (H, H),
                           p + "mix.o": (W, H * vd), p + "mix.o.b": (W,)})
            if m.get("v_mix"):
                shapes[p + "mix.vmix"] = ()
        if layer.get("mlp") is not None:
            shapes.update(norm(p + "norm2"))
            shapes.update({p + "mlp.up": (layer["mlp"]["ff"], W), p + "mlp.down": (W, layer["mlp"]["ff"])})
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
        if last == "alpha":
            w = 0.6 + 0.2 * np.abs(z)
        elif last == "vmix":
            w = 0.35 + 0.1 * z
        elif name.endswith(".b") and ("norm" in name):
            w = 0.2 * z
        elif last in ("norm1", "norm2", "norm") or name == "final.norm":
            w = 1.0 + 0.2 * z
        elif last == "canon1":
            w = 0.4 * z
        elif last == "talk":
            w = np.eye(shape[0], dtype=np.float32) + 0.3 * z
        elif name.endswith("f.b"):
            w = 2.0 + z                     # forget gates mostly open
        elif name.endswith("i.b"):
            w = z
        elif name.endswith(".b"):
            w = 0.3 * z
        elif name == "embed":
            w = 0.7 * z
        elif last in ("i", "f"):
            w = 3.0 * z / np.sqrt(shape[-1])
        else:
            w = 1.2 * z / np.sqrt(shape[-1])
        out[name] = bf16_exact(w)
    return out


def write_folder(tmp, name, seed=0, bf16=False, cfg=None):
    cfg = cfg or CONFIGS[name]
    folder = os.path.join(str(tmp), f"pogezen_{name}")
    return tm.write_model_folder(folder, cfg, make_weights(cfg, seed), bf16=bf16)


def torch_weights(cfg, seed, dtype=torch.float64):
    return {k: torch.from_numpy(np.asarray(v)).to(dtype) for k, v in make_weights(cfg, seed).items()}


def prompts(cfg, lengths, seed=0):
    rng = np.random.Generator(np.random.PCG64(900 + seed))
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
