"""Pogezen on the GPU against the plain implementation (tests/plain_pogezen.py), in float32 and bfloat16.

First every mechanism alone: the Dynamic Tanh norm with and without the input filter (whole, in portions, token by
token, a slot that is used again), the matrix memory as a part (whole, in portions, token by token, two sequences,
a key far back that an open forget gate still carries and a closed one has dropped), the attention as a part (one
key that a query is aligned with, placed just inside and just outside the window and the kept first tokens, at a
page's border, in prompts and in single tokens; the heads' mixing matrix; rotation, norm and mixed values as the
cache holds them). Then whole models of several shapes: each request alone, the stream after every layer, a prompt
and then single tokens, portions down to two tokens, batches of unequal requests on a small cache whose slots and
pages are used again, long decoding through replayed graphs, greedy generation through ``generate``, and the trace
runner as a child process.
"""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_pogezen as plain
import pogezen_models as pm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]


def K():
    from pytorch_transformers_b200 import kernels
    return kernels


def tdtype(name):
    return getattr(torch, name)


def row_errors(got, ref):
    got, ref = got.double().cpu().reshape(-1, got.shape[-1]), ref.double().cpu().reshape(-1, ref.shape[-1])
    return (got - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-30)


def close(got, ref, dtype, what="", f32=1e-4, bf16=3e-2):
    """float32: every row within rounding of float32 sums, and the rows' median well within (a row whose normaliser
    n . q nearly cancels carries more of it than the others). bfloat16: the rows' median within a bfloat16 model's
    rounding and 9 rows in 10 within twice that."""
    e = row_errors(got, ref)
    if dtype == "float32":
        assert e.max() < f32 and e.median() < f32 / 10, f"{what}: worst row error {e.max():.3g}, median {e.median():.3g}"
    else:
        assert e.median() < bf16 and (e < 2 * bf16).double().mean() >= 0.9, \
            f"{what}: median row error {e.median():.3g}, worst {e.max():.3g}"


class Mixer:
    """A mixer part alone on a cache of its own, fed rows directly."""

    def __init__(self, spec, weights, dtype):
        from pytorch_transformers_b200.parts.base import BuildContext, make_part
        self.k, self.dt = K(), tdtype(dtype)
        self.part = make_part(BuildContext(torch.device("cuda"), self.dt, self.k), spec)
        for part in self.part.walk():
            decls = part.param_decls()
            if decls:
                part.bind({n: weights[part.spec.names[n]].to(device="cuda", dtype=torch.float32 if d.role == "vector" else self.dt)
                           for n, d in decls.items()})
        planners = self.part.planner()
        self.planners = [p for p in (list(planners) if isinstance(planners, (list, tuple)) else [planners]) if p is not None]

    def cache(self, max_tokens, max_slots=None):
        from pytorch_transformers_b200.cache.paged import Cache
        return Cache([(0, self.part.cache_need(), self.part.state_need())], max_tokens, self.dt, "cuda", max_slots=max_slots)

    def step(self, cache, slots, rows):
        from pytorch_transformers_b200.engine.batch import StepContext
        from pytorch_transformers_b200.parts.base import ScheduleEntry
        ctx = StepContext(cache, slots, [[0] * r.shape[0] for r in rows], 1, [[] for _ in rows], self.planners)
        x = torch.cat(rows).to(self.dt).cuda().contiguous()
        y = self.part.forward(x, ctx, ScheduleEntry(0, 0))
        ctx.commit()
        return list(y.double().cpu().split([r.shape[0] for r in rows]))


def bf16_exact(t):
    return t.bfloat16().double()


# ------------------------------------------------------------------------------------------------ the norm and the filter
@pytest.mark.parametrize("out", DTYPES)
@pytest.mark.parametrize("width,taps", [(52, 4), (96, 1), (300, 3), (2048, 2)])
def test_dynamic_tanh_and_input_filter_whole_in_portions_and_token_by_token(width, taps, out):
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.base import StateNeed
    k = K()
    g = torch.Generator().manual_seed(width + taps)
    w = {"n": 1 + 0.2 * torch.randn(width, generator=g), "n.b": 0.2 * torch.randn(width, generator=g), "n.alpha": torch.tensor(0.7)}
    filt = 0.4 * torch.randn(width, taps, generator=g)
    xs = [torch.randn(n, width, generator=g) * 2 for n in (37, 5)]
    wd = {kk: v.double() for kk, v in w.items()}
    alone = k.dyt(xs[0].cuda(), w["n.alpha"].cuda(), w["n"].cuda(), w["n.b"].cuda(), tdtype(out))
    close(alone, plain.dyt(xs[0].double(), wd, "n"), out, "norm alone", f32=2e-6, bf16=5e-3)
    refs = [plain.input_conv(plain.dyt(x.double(), wd, "n"), filt.double()) for x in xs]
    cache = Cache([(0, None, StateNeed((taps - 1) * width + 3))], 64, torch.float32, "cuda", max_slots=2)
    for cuts in ([(37, 5)], [(20, 2), (17, 3)], [(1, 1)] * 5 + [(30, 0)] + [(1, 0)] * 2, [(3, 5), (2, 0), (32, 0)]):
        slots = [cache.open(), cache.open()]            # the second round uses the first one's slots again
        at, got = [0, 0], [[], []]
        for cut in cuts:
            live = [b for b in (0, 1) if cut[b] > 0]
            rows = [xs[b][at[b]:at[b] + cut[b]] for b in live]
            ctx = StepContext(cache, [slots[b] for b in live], [[0] * r.shape[0] for r in rows], 1, [[] for _ in rows])
            state = cache.entry_state(0)[:, :(taps - 1) * width] if taps > 1 else None
            y = k.dyt(torch.cat(rows).cuda(), w["n.alpha"].cuda(), w["n"].cuda(), w["n.b"].cuda(), tdtype(out), conv=filt.cuda(),
                      state=state, slots=ctx.dev["slots"], batch=ctx.batch_c[0], single_tokens=ctx.is_decode)
            ctx.commit()
            for b, part in zip(live, y.split([r.shape[0] for r in rows])):
                got[b].append(part)
                at[b] += cut[b]
        for b in (0, 1):
            n = at[b]
            close(torch.cat(got[b]), refs[b][:n], out, f"filter, cuts {cuts}", f32=2e-6, bf16=5e-3)
        for s in slots:
            cache.close(s)
    assert float(cache.entry_state(0)[:, (taps - 1) * width:].abs().max()) == 0        # nothing written past its stretch


# ------------------------------------------------------------------------------------------------ the matrix memory
def memory_spec(m, width, eps=1e-5, p="mix."):
    from pytorch_transformers_b200.parts.base import PartSpec
    names = {n: p + n for n in ("q", "k", "v", "g", "o", "norm", "i", "f")}
    names.update({"i_b": p + "i.b", "f_b": p + "f.b"})
    return PartSpec("mixer", "mlstm", {"hidden": width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                       "gate_cap": m["gate_cap"], "eps": eps}, names=names)


def memory_weights(m, width, seed, f_bias=2.0):
    g = torch.Generator().manual_seed(seed)
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    r = lambda *s: torch.randn(*s, generator=g)
    w = {"mix.q": 1.2 * r(H * d, width) / math.sqrt(width), "mix.k": 1.2 * r(H * d, width) / math.sqrt(width),
         "mix.v": 1.2 * r(H * vd, width) / math.sqrt(width), "mix.g": r(H * vd, width) / math.sqrt(width),
         "mix.o": r(width, H * vd) / math.sqrt(H * vd), "mix.norm": 1 + 0.2 * r(H * vd),
         "mix.i": 3 * r(H, width) / math.sqrt(width), "mix.i.b": r(H), "mix.f": 3 * r(H, width) / math.sqrt(width), "mix.f.b": f_bias + r(H)}
    return {kk: bf16_exact(v) for kk, v in w.items()}


MEMORIES = [dict(heads=3, dim=16, vdim=40, gate_cap=10.0), dict(heads=2, dim=6, vdim=10, gate_cap=5.0),
            dict(heads=1, dim=8, vdim=8, gate_cap=1.0), dict(heads=2, dim=128, vdim=96, gate_cap=8.0),
            dict(heads=1, dim=200, vdim=33, gate_cap=12.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", MEMORIES, ids=lambda m: f"{m['heads']}x{m['dim']}x{m['vdim']}")
def test_matrix_memory_whole_in_portions_and_token_by_token(dtype, m):
    width = 48
    w = memory_weights(m, width, seed=m["dim"])
    mixer = Mixer(memory_spec(m, width), {kk: v.float() for kk, v in w.items()}, dtype)
    g = torch.Generator().manual_seed(1)
    xs = [bf16_exact(torch.randn(n, width, generator=g)) for n in (150, 9)]
    refs = [plain.mlstm(x, w, "mix.", m, 1e-5) for x in xs]
    cache = mixer.cache(64, max_slots=2)
    for cuts in ([(150, 9)], [(64, 2), (7, 7), (79, 0)], [(1, 1)] * 9 + [(100, 0)] + [(1, 0)] * 5):
        slots = [cache.open(), cache.open()]
        at, got = [0, 0], [[], []]
        for cut in cuts:
            live = [b for b in (0, 1) if cut[b] > 0]
            outs = mixer.step(cache, [slots[b] for b in live], [xs[b][at[b]:at[b] + cut[b]] for b in live])
            for b, o in zip(live, outs):
                got[b].append(o)
                at[b] += cut[b]
        for b in (0, 1):
            close(torch.cat(got[b]), refs[b][:at[b]], dtype, f"memory, cuts {cuts[:3]}", f32=3e-5, bf16=2.5e-2)
        for s in slots:
            cache.close(s)


CHUNKED = [dict(heads=2, dim=64, vdim=64, gate_cap=15.0), dict(heads=1, dim=128, vdim=64, gate_cap=6.0),
           dict(heads=3, dim=64, vdim=128, gate_cap=9.0), dict(heads=2, dim=128, vdim=128, gate_cap=12.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("f_bias", [3.0, -2.0])
@pytest.mark.parametrize("m", CHUNKED, ids=lambda m: f"{m['heads']}x{m['dim']}x{m['vdim']}")
def test_matrix_memory_long_prompts_in_chunks(dtype, m, f_bias):
    """Prompts long enough for the chunked form (bfloat16, sizes of the tensor cores) of unequal lengths, whole, cut at
    and off the chunks' edges, continued from a state that single tokens or an earlier portion left, with forget gates
    mostly open and mostly closed."""
    width = 40
    w = memory_weights(m, width, seed=m["dim"] + m["vdim"], f_bias=f_bias)
    mixer = Mixer(memory_spec(m, width), {kk: v.float() for kk, v in w.items()}, dtype)
    g = torch.Generator().manual_seed(2)
    xs = [bf16_exact(torch.randn(n, width, generator=g)) for n in (700, 333)]
    refs = [plain.mlstm(x, w, "mix.", m, 1e-5) for x in xs]
    cache = mixer.cache(64, max_slots=2)
    for cuts in ([(700, 333)], [(300, 0), (400, 333)], [(256, 5), (1, 1), (443, 327)], [(3, 0), (1, 0), (321, 257), (375, 76)]):
        slots = [cache.open(), cache.open()]
        at, got = [0, 0], [[], []]
        for cut in cuts:
            live = [b for b in (0, 1) if cut[b] > 0]
            outs = mixer.step(cache, [slots[b] for b in live], [xs[b][at[b]:at[b] + cut[b]] for b in live])
            for b, o in zip(live, outs):
                got[b].append(o)
                at[b] += cut[b]
        for b in (0, 1):
            close(torch.cat(got[b]), refs[b][:at[b]], dtype, f"memory in chunks, cuts {cuts[:3]}", bf16=2.5e-2)
        for s in slots:
            cache.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far,steps", [(0, "prompt"), (3, "tokens"), (63, "prompt"), (64, "tokens")])
@pytest.mark.parametrize("d,vd", [(16, 12), (64, 64)])
def test_matrix_memory_carries_a_far_key_only_while_the_forget_gate_is_open(dtype, far, steps, d, vd):
    """One token long ago has a wide-open input gate and a key that the last query is aligned with. The head whose
    forget gate stays open (bias +8) answers with that token's value; the head whose forget gate closes a little
    every step (bias -1) has lost it among the later tokens."""
    m, width, T = dict(heads=2, dim=d, vdim=vd, gate_cap=12.0), 40, 400
    w = memory_weights(m, width, seed=7)
    for name in ("mix.i", "mix.f"):
        w[name] = torch.zeros_like(w[name])
    w["mix.i.b"] = torch.zeros(2, dtype=torch.float64)
    w["mix.f.b"] = torch.tensor([8.0, -1.0], dtype=torch.float64)
    w["mix.i"][:, 0] = 6.0                         # channel 0 of the input opens the input gate
    w["mix.k"] = w["mix.q"].clone()                # so that one input gives a key and a query that point the same way
    w["mix.q"][:, 0] = w["mix.k"][:, 0] = 0.0      # the gates' channel does not move them
    g = torch.Generator().manual_seed(far)
    x = bf16_exact(0.3 * torch.randn(T, width, generator=g))
    x[:, 0] = -1.0
    direction = torch.randn(width - 1, generator=g)
    x[far, 1:] = bf16_exact(direction)
    x[far, 0] = 2.0
    x[T - 1, 1:] = bf16_exact(direction)
    mixer = Mixer(memory_spec(m, width), {kk: v.float() for kk, v in w.items()}, dtype)
    cache = mixer.cache(64, max_slots=1)
    s = cache.open()
    head = T - 1 if steps == "prompt" else T - 40
    outs = mixer.step(cache, [s], [x[:head]])
    for t in range(head, T):
        outs += mixer.step(cache, [s], [x[t:t + 1]])
    got = torch.cat(outs)
    ref = plain.mlstm(x, w, "mix.", m, 1e-5)
    close(got[-1:], ref[-1:], dtype, "last token", f32=3e-5, bf16=4e-2)
    # what the memory gave before the output projection, per head, against the far token's value
    H = 2
    k_far, q_last = (x[far] @ w["mix.k"].T).view(H, d), (x[T - 1] @ w["mix.q"].T).view(H, d)
    assert (k_far * q_last).sum(-1).abs().min() > 3          # aligned in both heads
    i, f = plain.log_gates(x, w, "mix.", 12.0)
    carried = (f[far + 1:].sum(0) + i[far]) - torch.logsumexp(torch.stack([f[j + 1:].sum(0) + i[j] for j in range(T)]), 0)
    assert carried[0] > -0.7 and carried[1] < -20            # the open head keeps at least half its weight on the far token


# ------------------------------------------------------------------------------------------------ the attention
def attention_spec(m, width, eps=1e-5, p="mix.", value_mix="none"):
    from pytorch_transformers_b200.parts.base import PartSpec
    children = {}
    rot = m.get("rot")
    if rot and rot.get("dims"):
        sc = rot.get("scaling") or {"factor": 1.0, "original": 1.0, "fast": 1.0, "slow": 1.0}
        children["position"] = PartSpec("position", "rotary", {"head_dim": m["dim"], "theta": rot["base"], "rotary_dim": rot["dims"],
                                                               "yarn": {kk: float(sc[kk]) for kk in ("factor", "original", "fast", "slow")}})
    names = {n: p + n for n in ("q", "k", "v", "o", "talk")}
    names.update({n + "_b": p + n + ".b" for n in ("q", "k", "v", "o")})
    if value_mix != "none":
        names["vmix"] = p + "vmix"
    return PartSpec("mixer", "sink_attention",
                    {"hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                     "scale": m["scale"], "window": m["mask"]["size"], "eps": eps, "qk_norm": True, "qk_gain": False, "sink": False,
                     "gate": False, "bias": True, "keep_first": m["mask"]["keep_first"], "talk": True, "value_mix": value_mix},
                    children=children, names=names)


def attention_weights(m, width, seed):
    g = torch.Generator().manual_seed(seed)
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    r = lambda *s: torch.randn(*s, generator=g)
    w = {"mix.q": r(H * d, width) / math.sqrt(width), "mix.q.b": 0.3 * r(H * d), "mix.k": r(G * d, width) / math.sqrt(width),
         "mix.k.b": 0.3 * r(G * d), "mix.v": r(G * vd, width) / math.sqrt(width), "mix.v.b": 0.3 * r(G * vd),
         "mix.talk": torch.eye(H) + 0.3 * r(H, H), "mix.o": r(width, H * vd) / math.sqrt(H * vd), "mix.o.b": 0.1 * r(width),
         "mix.vmix": torch.tensor(0.35)}
    return {kk: bf16_exact(v) for kk, v in w.items()}


def att_m(heads, kv_heads, dim, vdim, window, keep, rot=None, scale=None):
    return pm.att(heads, kv_heads, dim, vdim, window, keep, rot, scale)["mixer"]


ATTENTIONS = [att_m(6, 2, 24, 20, 33, 5, pm.rot(8, 10000.0, (4.0, 64, 8.0, 1.0))), att_m(5, 5, 10, 14, 129, 70, pm.rot(6)),
              att_m(1, 1, 16, 16, 1, 1, pm.rot(16, 10.0), scale=1.0), att_m(8, 2, 64, 64, 130, 4, pm.rot(32)),
              att_m(3, 1, 18, 6, 0, 0), att_m(4, 4, 32, 8, 64, 64)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", ATTENTIONS, ids=lambda m: f"{m['heads']}x{m['kv_heads']}x{m['dim']}x{m['vdim']}w{m['mask']['size']}k{m['mask']['keep_first']}")
def test_attention_with_rotation_kept_tokens_and_mixed_heads(dtype, m):
    width = 40
    w = attention_weights(m, width, seed=m["dim"])
    mixer = Mixer(attention_spec(m, width), {kk: v.float() for kk, v in w.items()}, dtype)
    g = torch.Generator().manual_seed(2)
    xs = [bf16_exact(torch.randn(n, width, generator=g)) for n in (300, 70)]
    refs = [plain.attention(x, w, "mix.", m, 1e-5, {}) for x in xs]
    cache = mixer.cache(64 * 8, max_slots=2)
    for cuts in ([(300, 70)], [(130, 64), (3, 1), (1, 1), (166, 4)], [(250, 60)] + [(1, 1)] * 10 + [(1, 0)] * 40):
        slots = [cache.open(), cache.open()]
        at, got = [0, 0], [[], []]
        for cut in cuts:
            live = [b for b in (0, 1) if cut[b] > 0]
            outs = mixer.step(cache, [slots[b] for b in live], [xs[b][at[b]:at[b] + cut[b]] for b in live])
            for b, o in zip(live, outs):
                got[b].append(o)
                at[b] += cut[b]
        for b in (0, 1):
            close(torch.cat(got[b]), refs[b][:at[b]], dtype, f"attention, cuts {cuts[:3]}", f32=3e-5, bf16=2.5e-2)
        for s in slots:
            cache.close(s)
        cache.check()


def needle_case(dtype, window, keep, query_pos, key_pos, past):
    """The query at ``query_pos`` and the key at ``key_pos`` point the same way in the entries that are not rotated;
    the value at ``key_pos`` is marked. Returns (what the attention gave for the query, the plain result)."""
    width, d, vd = 48, 32, 12
    m = att_m(1, 1, d, vd, window, keep, pm.rot(8), scale=1.5)
    w = attention_weights(m, width, seed=11)
    w["mix.talk"] = torch.ones(1, 1, dtype=torch.float64)
    g = torch.Generator().manual_seed(query_pos * 7 + key_pos)
    x = bf16_exact(0.05 * torch.randn(query_pos + 1, width, generator=g))
    direction = torch.randn(width, generator=g)
    # an input whose query and key both lie along one unrotated direction: solve for it through the projections' pseudo-inverse
    unit = torch.zeros(d, dtype=torch.float64)
    unit[8:] = 1.0
    xq = torch.linalg.lstsq(w["mix.q"], (6 * unit - w["mix.q.b"])[:, None]).solution[:, 0]
    xk = torch.linalg.lstsq(w["mix.k"], (6 * unit - w["mix.k.b"])[:, None]).solution[:, 0]
    x[query_pos], x[key_pos] = bf16_exact(xq), bf16_exact(xk)
    del direction
    mixer = Mixer(attention_spec(m, width), {kk: v.float() for kk, v in w.items()}, dtype)
    cache = mixer.cache(64 * 8, max_slots=1)
    s = cache.open()
    outs = mixer.step(cache, [s], [x[:past]]) if past else []
    if past <= query_pos:
        outs += mixer.step(cache, [s], [x[past:]])
    got = torch.cat(outs)[-1]
    ref = plain.attention(x, w, "mix.", m, 1e-5, {})[-1]
    # the weight that the plain form puts on the needle
    T = x.shape[0]
    pos = torch.arange(T)
    q = plain.rms(plain.rotate((x @ w["mix.q"].T + w["mix.q.b"]).view(T, 1, d), pos, m["rot"]), 1e-5)
    kk = plain.rms(plain.rotate((x @ w["mix.k"].T + w["mix.k.b"]).view(T, 1, d), pos, m["rot"]), 1e-5)
    sc = (q[-1, 0] * kk[:, 0]).sum(-1) * m["scale"]
    sc = sc.masked_fill(~plain.visible(T, window, keep)[-1], -math.inf)
    return got, ref, float(torch.softmax(sc, -1)[key_pos])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,keep,query_pos,past", [(33, 5, 200, 0), (33, 5, 200, 150), (33, 5, 200, 200), (64, 3, 191, 0),
                                                         (64, 3, 192, 192), (70, 64, 300, 0), (70, 65, 300, 300), (129, 1, 260, 256)])
def test_attention_sees_the_window_and_the_kept_tokens_and_not_one_key_more(dtype, window, keep, query_pos, past):
    for key_pos, seen in ((query_pos - window + 1, True), (query_pos - window, False), (keep - 1, True), (keep, False),
                          (0, True), (query_pos, True)):
        if key_pos == query_pos:
            continue
        got, ref, weight = needle_case(dtype, window, keep, query_pos, key_pos, past)
        assert (weight > 0.5) == seen, (key_pos, weight)
        e = float((got - ref).norm() / ref.norm())
        assert e < (3e-5 if dtype == "float32" else 3e-2), f"key {key_pos} (seen: {seen}): {e:.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_queries_keys_and_mixed_values_as_the_cache_holds_them(dtype):
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.base import CacheNeed
    from pytorch_transformers_b200.parts.position import yarn_frequencies
    k, dt = K(), tdtype(dtype)
    H, G, d, vd, T = 3, 1, 18, 6, 70
    rot = pm.rot(6, 100.0, (2.0, 32, 4.0, 0.5))
    g = torch.Generator().manual_seed(4)
    proj = bf16_exact(torch.randn(T, (H + G) * d + G * vd + 5, generator=g))        # rows wider than needed
    bias, first = bf16_exact(0.3 * torch.randn((H + G) * d + G * vd, generator=g)), bf16_exact(torch.randn(T, G * vd, generator=g))
    cache = Cache([(0, CacheNeed("full", G, d, v_head_dim=vd), None)], 128, dt, "cuda")
    s = cache.open()
    ctx = StepContext(cache, [s], [[0] * T], 1, [[]])
    f, mult = yarn_frequencies(6, 100.0, 2.0, 32, 4.0, 0.5)
    fp, mp = plain.rotary_frequencies(rot)
    torch.testing.assert_close(f, fp, atol=0, rtol=1e-15)
    assert mult == pytest.approx(mp)
    cos, sin = k.rope_table(ctx.dev["tok_pos"], f.float().cuda())
    k.scale_(cos, mult), k.scale_(sin, mult)
    k_pool, v_pool, _ = cache.entry_storage(0)
    lam = torch.tensor(0.35, device="cuda")
    q, kept = k.rope_norm_store(proj.to(dt).cuda(), bias.float().cuda(), k_pool, v_pool, ctx.batch_c[0], (cos, sin), H, G, d, vd, 1e-5,
                                unit_norm=True, v_first=first.to(dt).cuda(), lam=lam, keep_values=True)
    pos = torch.arange(T)
    qk = (proj[:, :(H + G) * d] + bias[:(H + G) * d]).view(T, H + G, d)
    want = plain.rms(plain.rotate(qk, pos, rot), 1e-5)
    close(q, want[:, :H], dtype, "queries", f32=2e-6, bf16=5e-3)
    pages = cache.pages(s, 0)
    keys = torch.cat([k_pool[p, 0] for p in pages])[:T]
    close(keys, want[:, H], dtype, "keys", f32=2e-6, bf16=5e-3)
    v = proj[:, (H + G) * d:(H + G) * d + G * vd] + bias[(H + G) * d:]
    close(kept, v, dtype, "own values", f32=1e-6, bf16=5e-3)
    vals = torch.cat([v_pool[p, 0] for p in pages])[:T]
    close(vals, 0.65 * v + 0.35 * first, dtype, "mixed values", f32=2e-6, bf16=8e-3)


# ------------------------------------------------------------------------------------------------ whole models
class Loaded:
    def __init__(self, tmp, name, dtype):
        import pytorch_transformers_b200 as ptb
        self.cfg = pm.CONFIGS[name]
        self.folder = pm.write_folder(tmp, name, seed=len(name), bf16=(dtype == "bfloat16"))
        self.model = ptb.AutoModelForCausalLM.from_pretrained(self.folder, dtype=dtype)
        self.w = pm.torch_weights(self.cfg, len(name))
        self._ref = {}

    def plain_logits(self, ids):
        key = tuple(ids)
        if key not in self._ref:
            self._ref[key] = plain.forward(self.cfg, self.w, ids)
        return self._ref[key]


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = Loaded(tmp_path_factory.mktemp(f"{name}_{dtype}"), name, dtype)
        return made[(name, dtype)]
    return get


NAMES = sorted(pm.CONFIGS)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(loaded, name, dtype):
    L = loaded(name, dtype)
    assert L.model.spec.stream_float32 and L.model.use_graphs
    cache = L.model.new_cache(320)
    for ids in pm.prompts(L.cfg, (1, 2, 5, 70, 129, 300), seed=1):
        s = cache.open()
        close(L.model.step(cache, [s], [ids], want="all"), L.plain_logits(ids), dtype, f"{name} {len(ids)} tokens")
        cache.close(s)
    L.model.check_errors()
    cache.check()


def test_residual_stream_after_every_layer(loaded):
    L = loaded("mixed", "float32")
    ids = pm.prompts(L.cfg, (50,), seed=2)[0]
    want, got = [], []
    plain.forward(L.cfg, L.w, ids, layers_out=want)
    blocks = L.model.blocks
    originals = [b.forward for b in blocks]
    try:
        for b, orig in zip(blocks, originals):
            b.forward = (lambda x, ctx, entry, orig=orig: (got.append(orig(x, ctx, entry)), got[-1])[1])
        cache = L.model.new_cache(64)
        L.model.step(cache, [cache.open()], [ids], want="last")
    finally:
        for b in blocks:
            del b.forward
    assert len(got) == len(want) == 5
    from pytorch_transformers_b200.parts.base import DeferredSum, resolve
    assert all(isinstance(a, DeferredSum) for a in got)      # no sum is a kernel of its own: the next norm forms it
    for i, (a, b) in enumerate(zip(got, want)):
        a = resolve(K(), a)
        assert a.dtype == torch.float32 and row_errors(a, b).max() < 1e-5, f"layer {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(256)
    for n, head in ((100, 60), (34, 1), (200, 62)):        # the single tokens cross a page's border and pass the windows
        ids = pm.prompts(L.cfg, (n,), seed=n)[0]
        s = cache.open()
        rows = [L.model.step(cache, [s], [ids[:head]], want="all")]
        rows += [L.model.step(cache, [s], [[t]], want="last") for t in ids[head:]]
        close(torch.cat(rows), L.plain_logits(ids), dtype, f"{name} prompt of {head} then {n - head} single tokens")
        cache.close(s)
    L.model.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("portion", [2, 3, 17, 64])
def test_prompts_in_portions(loaded, name, dtype, portion):
    L = loaded(name, dtype)
    cache = L.model.new_cache(192)
    ids = pm.prompts(L.cfg, (150,), seed=portion)[0]
    s = cache.open()
    rows = [L.model.step(cache, [s], [ids[i:i + portion]], want="all") for i in range(0, len(ids), portion)]
    close(torch.cat(rows), L.plain_logits(ids), dtype, f"{name} in portions of {portion}")
    cache.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_a_long_prompt_in_two_portions(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(64 * 9)
    ids = pm.prompts(L.cfg, (530,), seed=12)[0]
    s = cache.open()
    got = torch.cat([L.model.step(cache, [s], [ids[:400]], want="all"), L.model.step(cache, [s], [ids[400:]], want="all")])
    close(got, L.plain_logits(ids), dtype, f"{name} 400 + 130 tokens")
    cache.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_batches_of_unequal_requests_on_a_small_cache(loaded, name, dtype):
    """Two batches one after the other on a cache that holds just one of them: slots and pages of the first are
    used again by the second, whose sequences must start from empty state. Shorter requests end earlier."""
    L = loaded(name, dtype)
    cache = L.model.new_cache(64 * 5, max_slots=3)
    for seed, (lengths, heads) in enumerate([((130, 7, 66), (120, 2, 64)), ((3, 90, 65), (1, 64, 33))]):
        reqs = pm.prompts(L.cfg, lengths, seed=10 + seed)
        refs = [L.plain_logits(r) for r in reqs]
        slots = [cache.open() for _ in reqs]
        assert sorted(slots) == [0, 1, 2]
        out = L.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], want="last")
        live, t, got, want = [0, 1, 2], 0, [], []
        while True:
            for row, i in enumerate(live):
                got.append(out[row])
                want.append(refs[i][heads[i] + t - 1])
            for i in [i for i in live if heads[i] + t >= lengths[i]]:
                cache.close(slots[i])
            live = [i for i in live if heads[i] + t < lengths[i]]
            if not live:
                break
            out = L.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + t]] for i in live], want="last")
            t += 1
        close(torch.stack(got), torch.stack(want), dtype, f"{name} batch {seed}")
        cache.check()
        assert not cache.records
    L.model.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "ones", "wide"])
def test_long_decoding(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(64 * 12)
    reqs = pm.prompts(L.cfg, (330, 290), seed=5)
    refs = [L.plain_logits(r) for r in reqs]
    slots = [cache.open(), cache.open()]
    heads = (3, 1)
    out = [L.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], want="last")]
    L.model.record_steps(True)
    for t in range(289):
        out.append(L.model.step(cache, slots, [[reqs[0][3 + t]], [reqs[1][1 + t]]], want="last"))
    kinds = [r["kind"] for r in L.model.step_timings()]
    L.model.record_steps(False)
    assert kinds.count("graph") > 250            # the single-token steps were replayed graphs
    got = torch.stack(out)
    close(got[:, 0], refs[0][2:2 + 290], dtype, f"{name} long decoding, first")
    close(got[:, 1], refs[1][0:290], dtype, f"{name} long decoding, second")
    L.model.check_errors()
    cache.check()


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_generate(loaded, name):
    L = loaded(name, "float32")
    prompts = pm.prompts(L.cfg, (9, 1, 30), seed=3)
    out = L.model.generate(prompts, max_new_tokens=12, do_sample=False, eos_token_id=None)
    for p, seq in zip(prompts, out):
        assert seq[:len(p)] == p and len(seq) == len(p) + 12
        ids = list(p)
        for tok in seq[len(p):]:
            logits = L.plain_logits(ids)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) > 1e-4:          # no test on a tie within float32 rounding
                assert int(logits.argmax()) == tok
            ids.append(tok)


def test_generation_with_sampling_and_stop_tokens_runs(loaded):
    L = loaded("mixed", "bfloat16")
    prompts = pm.prompts(L.cfg, (5, 40), seed=8)
    out = L.model.generate(prompts, max_new_tokens=20, do_sample=True, top_k=20, temperature=0.8, seed=1, eos_token_id=7)
    assert all(len(o) <= len(p) + 20 for o, p in zip(out, prompts))
    again = L.model.generate(prompts, max_new_tokens=20, do_sample=True, top_k=20, temperature=0.8, seed=1, eos_token_id=7)
    assert out == again


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_model_from_config_and_from_folder_are_one_model(tmp_path, dtype):
    import pytorch_transformers_b200 as ptb
    cfg = ptb.PogezenConfig.from_dict(pm.CONFIGS["odd"])
    folder = ptb.write_random_model(cfg, seed=4, folder=str(tmp_path / "m"), dtype=tdtype(dtype))
    a = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    b = ptb.AutoModelForCausalLM.from_config(cfg, seed=4, dtype=dtype)
    ids = pm.prompts(pm.CONFIGS["odd"], (20,), seed=0)
    ca, cb = a.new_cache(64), b.new_cache(64)
    la, lb = a.step(ca, [ca.open()], ids, want="all"), b.step(cb, [cb.open()], ids, want="all")
    torch.testing.assert_close(la, lb, atol=0, rtol=0)
    assert torch.isfinite(la).all() and float(la.std()) > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_as_a_child_process(tmp_path, dtype):
    name = "mixed"
    cfg = pm.CONFIGS[name]
    folder = pm.write_folder(tmp_path, name, seed=2, bf16=(dtype == "bfloat16"))
    w = pm.torch_weights(cfg, 2)
    reqs = dict(zip("abc", pm.prompts(cfg, (70, 9, 40), seed=4)))
    refs = {kk: plain.forward(cfg, w, v) for kk, v in reqs.items()}
    heads = {"a": 64, "b": 6, "c": 40}
    steps = [{"step": 0, "entries": [{"id": i, "tokens": reqs[i][:heads[i]], "want": [0, heads[i] - 1]} for i in "abc"], "end": ["c"]}]
    expect = {0: [(i, p) for i in "abc" for p in (0, heads[i] - 1)]}
    for t in range(6):
        live = [i for i in "ab" if heads[i] + t < len(reqs[i])]
        steps.append({"step": t + 1, "entries": [{"id": i, "tokens": [reqs[i][heads[i] + t]], "want": [0]} for i in live],
                      "end": [i for i in live if heads[i] + t + 1 == len(reqs[i])]})
        expect[t + 1] = [(i, heads[i] + t) for i in live]
    out = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                           "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                          text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, want = [], []
    for step, rows in expect.items():
        arr = np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        assert arr.shape[0] == len(rows)
        got.append(torch.from_numpy(arr.copy()))
        want += [refs[i][p] for i, p in rows]
    close(torch.cat(got), torch.stack(want), dtype, "trace")
