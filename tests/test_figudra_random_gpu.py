"""Random Figudra configurations under random cuttings of the work, against the plain implementation.

The fixed configurations of tests/figudra_models.py pin known corners; this draws others: widths, any order of the
three mixers, layers that run the weights of an earlier or a later layer, head counts and groupings, key and value sizes
(also those of the compiled-in and tensor-core kernels and ones that are no multiple of 8), decay exponents and ranks,
soft caps and query temperatures present and absent, windows from one token to longer than every prompt, kept first
tokens from none to more than a page, rotation over none, a part or all of a head with and without scaling, dense and
routed feed-forwards and none, routers with one group and several, with and without a shared expert, in float32 and
bfloat16. Every request is fed as a prompt of a random length (in one step, or in two or three portions), then token by
token in a batch whose members end at different times, and every logit row is compared.
"""
import os
import random

import numpy as np
import pytest
import torch

import figudra_models as fm
import plain_figudra as plain
import tiny_models as tm

pytestmark = pytest.mark.gpu


def random_mlp(r: random.Random):
    kind = r.choice(["none", "dense", "moe", "moe"])
    if kind == "none":
        return None
    if kind == "dense":
        return fm.dense(r.choice([24, 56, 200]))
    count, per = r.choice([1, 1, 2, 3, 4]), r.choice([1, 2, 3, 5])
    keep = r.randint(1, count)
    top = r.randint(1, min(per * keep, 6))
    return fm.moe(count * per, top, r.choice([16, 40, 72]), count=count, keep=keep, scale=r.choice([1.0, 0.5, 2.5]),
                  shared=r.choice([None, 8, 48]))


def random_layer(r: random.Random, kind: str):
    if kind == "gla":
        d, vd = r.choice([(4, 12), (12, 4), (20, 36), (32, 32), (64, 64), (64, 128), (128, 64), (48, 80), (256, 16), (96, 32),
                          (128, 128)])
        return fm.gla(r.choice([1, 2, 3, 5]), d, vd, r.choice([1.0, 2.5, 16.0, 64.0]), r.choice([1, 4, 16, 24])), random_mlp(r)
    d, vd = r.choice([(8, 8), (12, 20), (24, 12), (40, 40), (64, 64), (64, 32), (128, 128), (96, 48), (128, 64), (32, 32)])
    kv = r.choice([1, 2, 3])
    heads = kv * r.choice([1, 2, 4])
    scale = r.choice([d ** -0.5, 1.0 / d, 0.3, 0.15])
    if kind == "attention":
        return fm.att(heads, kv, d, vd, scale, softcap=r.choice([None, 1.5, 30.0, 50.0]),
                      q_temp=r.choice([None, (0.4, 32), (1.3, 1), (0.1, 7), (0.25, 100)])), random_mlp(r)
    rot = None
    if r.random() < 0.85:
        dims = r.choice([2, d // 2 // 2 * 2, d])
        rot = (dims, r.choice([50.0, 10000.0, 1e6])) + r.choice([(), (2.0,), (8.0,), (1.0,)])
    window = r.choice([0, 1, 2, 9, 31, 64, 65, 100, 128, 140, 500])
    return fm.att2(heads, kv, d, vd, scale, window, r.choice([0, 1, 3, 5, 8, 64, 70]) if window else 0, rot=rot), random_mlp(r)


KINDS = ["gla", "attention", "attention_2"]


def random_config(r: random.Random) -> dict:
    kinds = [r.choice(KINDS) for _ in range(r.choice([1, 2, 3, 4, 5, 6]))]
    if r.random() < 0.5 and len(kinds) > 2:        # every kind at least once
        kinds[:3] = KINDS
        r.shuffle(kinds)
    own = [random_layer(r, kind) for kind in kinds]
    # runs of another layer's weights, before or after the layer that has them
    order = [("own", j) for j in range(len(own))]
    for _ in range(r.choice([0, 0, 1, 2])):
        order.insert(r.randint(0, len(order)), ("again", r.randrange(len(own))))
    place = {j: i for i, (what, j) in enumerate(order) if what == "own"}
    layers = []
    for what, j in order:
        mixer, mlp = own[j]
        layers.append(dict(mixer, mlp=mlp) if what == "own" else dict(mixer, mlp=mlp, weights_of=place[j]))
    return {"architecture": "Figudra", "vocab": r.choice([61, 200, 515]), "width": r.choice([40, 64, 72, 136, 256]),
            "norm": {"eps": r.choice([1e-5, 1e-6, 1e-3])}, "layers": layers}


def row_errors(got, ref):
    got, ref = got.double().cpu().reshape(-1, got.shape[-1]), ref.double().cpu().reshape(-1, ref.shape[-1])
    return (got - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-30)


@pytest.mark.parametrize("first_seed", range(0, 48, 8))
def test_random_configurations_and_cuttings(tmp_path, first_seed):
    import pytorch_transformers_b200 as ptb
    for seed in range(first_seed, first_seed + 8):
        r = random.Random(9000 + seed)
        cfg = random_config(r)
        dtype = r.choice(["float32", "float32", "bfloat16"])
        if dtype == "bfloat16":
            cfg = fm.steady(cfg)        # no choice of experts within a bfloat16 rounding of another
        folder = tm.write_model_folder(os.path.join(str(tmp_path), f"m{seed}"), cfg, fm.make_weights(cfg, seed),
                                       bf16=(dtype == "bfloat16"))
        model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
        w = fm.torch_weights(cfg, seed)
        g = np.random.Generator(np.random.PCG64(seed))
        lengths = [int(g.integers(2, r.choice([40, 150, 400]))) for _ in range(r.choice([1, 2, 3, 5]))]
        reqs = [g.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
        refs = [plain.forward(cfg, w, q) for q in reqs]
        what = f"seed {seed} {dtype} {cfg}"
        errors = []

        def compare(got, want):
            errors.append(row_errors(got, want))

        cache = model.new_cache(sum((n + 63) // 64 * 64 for n in lengths) + 64)
        slots = [cache.open() for _ in reqs]
        heads = [int(g.integers(1, n + 1)) for n in lengths]
        cuts = r.choice([1, 2, 3])
        marks = [sorted({0, h} | {int(g.integers(1, h + 1)) for _ in range(cuts - 1)}) for h in heads]
        for step in range(cuts):
            part = [(i, marks[i][step], marks[i][step + 1]) for i in range(len(reqs)) if step + 1 < len(marks[i])]
            if not part:
                break
            out, at = model.step(cache, [slots[i] for i, _, _ in part], [reqs[i][a:b] for i, a, b in part], want="all"), 0
            for i, a, b in part:
                compare(out[at:at + b - a], refs[i][a:b])
                at += b - a
        pos = list(heads)
        for i in [i for i in range(len(reqs)) if pos[i] >= lengths[i]]:
            cache.close(slots[i])
        live = [i for i in range(len(reqs)) if pos[i] < lengths[i]]
        for _ in range(80):
            if not live:
                break
            out = model.step(cache, [slots[i] for i in live], [[reqs[i][pos[i]]] for i in live], want="last")
            for row, i in enumerate(live):
                compare(out[row:row + 1], refs[i][pos[i]:pos[i] + 1])
                pos[i] += 1
            for i in [i for i in live if pos[i] >= lengths[i]]:
                cache.close(slots[i])
            live = [i for i in live if pos[i] < lengths[i]]
        model.check_errors()
        cache.check()
        e = torch.cat(errors)
        if dtype == "float32":
            assert e.max() < 2e-4 and e.median() < 2e-5, f"{what}: worst row error {e.max():.3g}, median {e.median():.3g}"
        else:
            assert e.median() < 3e-2 and (e < 6e-2).double().mean() >= 0.9, \
                f"{what}: median row error {e.median():.3g}, worst {e.max():.3g}"
