"""Random Pogezen configurations under random cuttings of the work, against the plain implementation.

The fixed configurations of tests/pogezen_models.py pin known corners; this draws others: widths, head counts and
groupings, key and value sizes (also those of the tensor-core kernels), windows from a few tokens to longer than
every prompt, kept first tokens from none to more than a page, rotation over none, a part or all of a head with and
without stretched frequencies, one to four taps, either mixer first, runs of one kind of layer, layers with and
without feed-forward, value mixing in none, one, some or all attention layers, in float32 and bfloat16. Every request
is fed as a prompt of a random length (in one step, or in two or three portions), then token by token in a batch
whose members end at different times, and every logit row is compared.
"""
import os
import random

import numpy as np
import pytest
import torch

import plain_pogezen as plain
import pogezen_models as pm
import tiny_models as tm

pytestmark = pytest.mark.gpu


def random_config(r: random.Random) -> dict:
    width = r.choice([40, 64, 72, 136, 256])
    layers, kinds = [], [r.choice(["mlstm", "attention"]) for _ in range(r.choice([1, 2, 3, 4, 5]))]
    if r.random() < 0.5 and len(kinds) > 1:        # both kinds at least once
        kinds[0], kinds[1] = "attention", "mlstm"
        r.shuffle(kinds)
    mix = r.choice(["none", "all", "some"])
    shared_kv, shared_vd = r.choice([1, 2, 3]), r.choice([8, 20, 40, 64])     # layers that mix values have the same values
    for kind in kinds:
        ff = r.choice([None, 24, 56, 200])
        if kind == "mlstm":
            d, vd = r.choice([(4, 12), (12, 4), (20, 36), (32, 32), (64, 64), (64, 128), (128, 64), (48, 80)])
            layers.append((pm.mem(r.choice([1, 2, 3, 5]), d, vd, r.choice([1.0, 4.0, 15.0, 30.0])), ff))
            continue
        d, vd = r.choice([(8, 8), (12, 20), (24, 12), (40, 40), (64, 64), (64, 32), (128, 128), (96, 48), (128, 64)])
        kv = r.choice([1, 2, 3])
        heads = kv * r.choice([1, 2, 4])
        rot = None
        if r.random() < 0.85:
            dims = r.choice([2, d // 2 // 2 * 2, d])
            scaling = None
            if r.random() < 0.6:
                scaling = (r.choice([1.5, 2.0, 8.0, 40.0]), r.choice([16, 64, 4096]), r.choice([4.0, 32.0]), r.choice([0.5, 1.0, 2.0]))
            rot = pm.rot(dims, r.choice([50.0, 10000.0, 1e6]), scaling)
        v_mix = mix == "all" or (mix == "some" and r.random() < 0.6)
        if v_mix:
            kv, vd = shared_kv, shared_vd
            heads = kv * r.choice([1, 2, 4])
        layers.append((pm.att(heads, kv, d, vd, r.choice([1, 2, 9, 31, 64, 65, 100, 128, 500]), r.choice([0, 1, 3, 8, 64, 70]),
                              rot, scale=r.choice([None, d ** -0.5, 1.0 / d, 0.3]), v_mix=v_mix), ff))
    return pm._cfg(r.choice([61, 200, 515]), width, r.choice([1, 2, 3, 4]), r.choice([1.0, 0.5, 4.0]), r.choice([1e-5, 1e-6, 1e-3]),
                   layers)


def row_errors(got, ref):
    got, ref = got.double().cpu().reshape(-1, got.shape[-1]), ref.double().cpu().reshape(-1, ref.shape[-1])
    return (got - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-30)


@pytest.mark.parametrize("first_seed", range(0, 48, 8))
def test_random_configurations_and_cuttings(tmp_path, first_seed):
    import pytorch_transformers_b200 as ptb
    for seed in range(first_seed, first_seed + 8):
        r = random.Random(7000 + seed)
        cfg = random_config(r)
        dtype = r.choice(["float32", "float32", "bfloat16"])
        folder = tm.write_model_folder(os.path.join(str(tmp_path), f"m{seed}"), cfg, pm.make_weights(cfg, seed),
                                       bf16=(dtype == "bfloat16"))
        model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
        w = pm.torch_weights(cfg, seed)
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
