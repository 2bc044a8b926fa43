"""Figudra on the GPU against the plain implementation (tests/plain_figudra.py), in float32 and bfloat16.

First every mechanism alone: the small kernels (the decay's logarithm, the gated unit, the heads' norm with a silu
gate, queries and keys normed with gains, rotated and given their temperature as the cache holds them), the gated
linear attention as a part (whole, in portions, token by token, in chunks, two sequences, a slot that is used again,
a key far back that an open channel still carries and a closed one has dropped), both attention settings as parts
(whole, in portions, single tokens; one key that a query is aligned with, placed far back, at a page's border, just
inside and just outside the window and the kept first tokens, in prompts and in single tokens; a soft cap that
binds; the added one of the softmax), the router against the plain one, the experts with their shared expert, the
gated feed-forward. Then whole models of several shapes: each request alone, the stream after every layer, a prompt
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

import plain_figudra as plain
import figudra_models as fm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
F64 = torch.float64


def K():
    from pytorch_transformers_b200 import kernels
    return kernels


def tdtype(name):
    return getattr(torch, name)


def row_errors(got, ref):
    got, ref = got.double().cpu().reshape(-1, got.shape[-1]), ref.double().cpu().reshape(-1, ref.shape[-1])
    return (got - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-30)


def close(got, ref, dtype, what="", f32=1e-4, bf16=3e-2):
    """float32: every row within rounding of float32 sums and the rows' median well within. bfloat16: the rows' median
    within a bfloat16 model's rounding and 9 rows in 10 within twice that."""
    e = row_errors(got, ref)
    if dtype == "float32":
        assert e.max() < f32 and e.median() < f32 / 10, f"{what}: worst row error {e.max():.3g}, median {e.median():.3g}"
    else:
        assert e.median() < bf16 and (e < 2 * bf16).double().mean() >= 0.9, \
            f"{what}: median row error {e.median():.3g}, worst {e.max():.3g}"


def bf16_exact(t):
    return t.bfloat16().double()


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

    def run_cut(self, cache, rows, cuts):
        """One sequence fed in portions of the given sizes; returns all its output rows."""
        s, at, got = cache.open(), 0, []
        for n in cuts:
            got.append(self.step(cache, [s], [rows[at:at + n]])[0])
            at += n
        cache.close(s)
        return torch.cat(got)


# ------------------------------------------------------------------------------------------------ small kernels
def test_decay_logarithm_gated_unit_and_silu_gate():
    k = K()
    g = torch.Generator().manual_seed(0)
    z, b = torch.randn(37, 24, generator=g) * 6, torch.randn(24, generator=g)
    got = k.gla_decay_(z.clone().cuda(), b.cuda(), 4.0).double().cpu()
    want = torch.nn.functional.logsigmoid(z.double() + b.double()) / 4.0
    torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-5)
    big = k.gla_decay_(torch.tensor([[60.0, -60.0, 0.0]]).cuda(), None, 1.0).cpu()
    assert float(big[0, 0]) > -1e-20 and abs(float(big[0, 1]) + 60) < 1e-4 and abs(float(big[0, 2]) + math.log(2)) < 1e-6
    for dtype in DTYPES:
        for f in (24, 13):
            gu = (torch.randn(50, 2 * f, generator=g) * 2).to(tdtype(dtype))
            for act, fn in (("silu", plain.silu), ("gelu_pytorch_tanh", plain.gelu_tanh)):
                want = fn(gu[:, :f].double()) * gu[:, f:].double()
                close(k.glu_act(gu.cuda(), act), want, dtype, f"gated unit {act}", f32=2e-6, bf16=5e-3)
        H, vd = 3, 10
        o, gain = torch.randn(20, H * vd, generator=g), 1 + 0.2 * torch.randn(vd, generator=g)
        gate = torch.randn(20, H * vd, generator=g).to(tdtype(dtype))
        got = k.head_norm_gate(o.cuda(), gain.repeat(H).cuda(), gate.cuda(), H, 1e-5, tdtype(dtype), gate_act="silu")
        want = (plain.rms_norm(o.double().reshape(20, H, vd), gain.double(), 1e-5).reshape(20, H * vd) * plain.silu(gate.double()))
        close(got, want, dtype, "heads' norm with a silu gate", f32=2e-6, bf16=5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,vd,dims", [(4, 2, 16, 20, 8), (3, 1, 10, 6, 6), (2, 2, 64, 64, 32), (1, 1, 200, 8, 0), (2, 1, 32, 8, 32)])
def test_queries_and_keys_normed_rotated_and_stored(dtype, H, G, d, vd, dims):
    """Norm with gains, then the rotation of a part of each head with scaled frequencies; keys in the cache, queries out.
    Without a norm: queries times the temperature of their position."""
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.base import CacheNeed
    k, dt = K(), tdtype(dtype)
    g = torch.Generator().manual_seed(d + dims)
    T, past = 70, 61
    cache = Cache([(0, CacheNeed("full", G, d, 0, v_head_dim=vd), None)], 384, dt, "cuda")
    s = cache.open()
    k_pool, v_pool, gi = cache.entry_storage(0)
    proj = torch.randn(past + T, (H + G) * d + G * vd, generator=g).to(dt)
    qg, kg = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
    inv = (100.0 ** (-2.0 * torch.arange(dims // 2).double() / max(dims, 1)) / 4.0).float().cuda()
    qs = []
    for lo, hi in ((0, past), (past, past + T)):
        ctx = StepContext(cache, [s], [[0] * (hi - lo)], 1, [[]])
        rope = k.rope_table(ctx.dev["tok_pos"], inv) if dims else None
        qs.append(k.rope_norm_store(proj[lo:hi].cuda().contiguous(), None, k_pool, v_pool, ctx.batch_c[gi], rope, H, G, d, vd, 1e-5,
                                    unit_norm=True, q_gain=qg.cuda(), k_gain=kg.cuda(), norm_first=True))
        ctx.commit()
    pos = torch.arange(past + T)
    p64 = proj.double()
    want_q = plain.rotate(plain.rms_norm(p64[:, :H * d].reshape(-1, H, d), qg.double(), 1e-5), pos, dims, 100.0, 4.0)
    want_k = plain.rotate(plain.rms_norm(p64[:, H * d:(H + G) * d].reshape(-1, G, d), kg.double(), 1e-5), pos, dims, 100.0, 4.0)
    close(torch.cat(qs).reshape(-1, H * d), want_q.reshape(-1, H * d), dtype, "queries", f32=3e-6, bf16=5e-3)
    keys = torch.cat([k_pool[p].permute(1, 0, 2) for p in cache.pages(s, gi)])[:past + T]
    close(keys.reshape(-1, G * d), want_k.reshape(-1, G * d), dtype, "keys", f32=3e-6, bf16=5e-3)
    # no norm, a temperature on the queries
    ctx = StepContext(cache, [cache.open()], [[0] * T], 1, [[]])
    q = k.rope_norm_store(proj[:T].cuda().contiguous(), None, k_pool, v_pool, ctx.batch_c[gi], None, H, G, d, vd, 1e-5,
                          unit_norm=False, q_temp=(0.7, 16))
    want = p64[:T, :H * d].reshape(T, H, d) * plain.query_temperature(torch.arange(T), 0.7, 16)[:, None, None]
    close(q.reshape(T, H * d), want.reshape(T, H * d), dtype, "queries with their temperature", f32=2e-6, bf16=5e-3)


# ------------------------------------------------------------------------------------------------ the gated linear attention
def gla_spec(m, width, eps=1e-5, p="mix."):
    from pytorch_transformers_b200.parts.base import PartSpec
    names = {n: p + n for n in ("q", "k", "v", "g", "o", "norm", "a1", "a2")}
    names["a2_b"] = p + "a2.b"
    return PartSpec("mixer", "gla", {"hidden": width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "tau": m["tau"],
                                     "eps": eps, "rank": m["rank"]}, names=names)


def gla_weights(m, width, seed, bias=1.0):
    g = torch.Generator().manual_seed(seed)
    H, d, vd, r = m["heads"], m["dim"], m["vdim"], m["rank"]
    rn = lambda *s: torch.randn(*s, generator=g)
    w = {"mix.q": 1.2 * rn(H * d, width) / math.sqrt(width), "mix.k": 1.2 * rn(H * d, width) / math.sqrt(width),
         "mix.v": 1.2 * rn(H * vd, width) / math.sqrt(width), "mix.g": 1.2 * rn(H * vd, width) / math.sqrt(width),
         "mix.o": 1.2 * rn(width, H * vd) / math.sqrt(H * vd), "mix.norm": 1 + 0.2 * rn(vd),
         "mix.a1": 1.2 * rn(r, width) / math.sqrt(width), "mix.a2": 2.0 * rn(H * d, r) / math.sqrt(r), "mix.a2.b": bias + 2.0 * rn(H * d)}
    return {kk: bf16_exact(v).float() for kk, v in w.items()}


GLA_SHAPES = [dict(heads=3, dim=16, vdim=40, tau=4.0, rank=8), dict(heads=2, dim=6, vdim=10, tau=1.0, rank=3),
              dict(heads=1, dim=8, vdim=8, tau=1.0, rank=1), dict(heads=2, dim=64, vdim=64, tau=8.0, rank=16),
              dict(heads=1, dim=128, vdim=96, tau=16.0, rank=32), dict(heads=1, dim=200, vdim=33, tau=2.0, rank=5)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", GLA_SHAPES, ids=lambda m: f"{m['heads']}x{m['dim']}x{m['vdim']}")
def test_gated_linear_attention_whole_in_portions_in_chunks_and_token_by_token(m, dtype):
    width = 48
    w = gla_weights(m, width, m["dim"])
    mixer = Mixer(gla_spec(m, width), w, dtype)
    g = torch.Generator().manual_seed(1)
    x = bf16_exact(torch.randn(330, width, generator=g)).float()
    ref = plain.gla_mixer(x.double(), plain.sub(w, "mix."), m, 1e-5)
    cache = mixer.cache(64, max_slots=2)
    # 330 tokens at once run in chunks of 64 (the last one short); 256 + 74 joins the chunked form and the walk
    for cuts in ([330], [256, 74], [100, 64, 2, 3, 17, 144], [1] * 40 + [290], [5] + [1] * 70 + [255]):
        close(mixer.run_cut(cache, x, cuts), ref, dtype, f"cuts {cuts[:6]}", f32=2e-5)
    # two sequences side by side, one ends early, and its slot is used again by a third
    y = bf16_exact(torch.randn(90, width, generator=g)).float()
    ref_y = plain.gla_mixer(y.double(), plain.sub(w, "mix."), m, 1e-5)
    a, b = cache.open(), cache.open()
    out = mixer.step(cache, [a, b], [x[:70], y[:20]])
    got_x, got_y = [out[0]], [out[1]]
    for t in range(20, 25):
        out = mixer.step(cache, [a, b], [x[50 + t:51 + t], y[t:t + 1]])
        got_x.append(out[0]); got_y.append(out[1])
    cache.close(b)
    c = cache.open()
    assert c == b
    out = mixer.step(cache, [c, a], [y[:90], x[75:80]])
    close(torch.cat(got_x + [out[1]]), ref[:80], dtype, "first of two", f32=2e-5)
    close(torch.cat(got_y), ref_y[:25], dtype, "second of two", f32=2e-5)
    close(out[0], ref_y, dtype, "a slot that is used again starts from nothing", f32=2e-5)


@pytest.mark.parametrize("n,back", [(700, 650), (300, 299), (130, 64), (65, 63), (40, 3), (1, 0)])
def test_a_far_key_on_an_open_channel_and_on_a_closed_one(n, back):
    """Kernel alone: channel 0 never decays (log 0), all others do. A key `back` tokens before the last query lies on
    channel 0 in head 0 and on channel 1 in head 1; the query asks both for it."""
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.base import StateNeed
    from pytorch_transformers_b200.parts.recurrent import RecurrenceChunks
    k = K()
    H, d, vd = 2, 8, 40
    g = torch.Generator().manual_seed(n)
    q, kk, v = 0.1 * torch.randn(n, H, d, generator=g), 0.1 * torch.randn(n, H, d, generator=g), torch.randn(n, H, vd, generator=g)
    la = torch.full((n, H, d), -0.05)
    la[:, :, 0] = 0.0
    at = n - 1 - back
    kk[:, :, :2] = 0.0
    kk[at, 0, 0] = kk[at, 1, 1] = 5.0
    q[n - 1, :, :2] = 5.0
    proj = torch.cat([q.reshape(n, -1), kk.reshape(n, -1), v.reshape(n, -1)], 1)
    ref, _ = plain.gla_recurrence(q.double(), kk.double(), v.double(), la.double().exp())
    for cuts in ([n], [n // 2, n - n // 2] if n > 1 else [1]):
        cache = Cache([(0, None, StateNeed(H * d * vd))], 64, torch.float32, "cuda")
        s, lo, outs = cache.open(), 0, []
        for c in cuts:
            ctx = StepContext(cache, [s], [[0] * c], 1, [[]], [RecurrenceChunks()])
            plan, chunks = ctx.plan(RecurrenceChunks.plan_key), None
            if plan.facts["n_chunks"]:
                chunks = (plan.dev["chunk_seq"], plan.dev["chunk_q0"], plan.dev["seq_chunk0"], plan.facts["n_chunks"])
            outs.append(k.gla(proj[lo:lo + c].cuda().contiguous(), la[lo:lo + c].reshape(c, -1).cuda().contiguous(),
                              ctx.state_of(type("E", (), {"cache_entry": 0, "state_offset": 0})(), H * d * vd), ctx.dev["slots"],
                              ctx.batch_c[0], H, d, vd, 1.0, chunks))
            ctx.commit()
            lo += c
        got = torch.cat(outs).double().cpu().reshape(n, H, vd)
        assert row_errors(got.reshape(n, -1), ref.reshape(n, -1)).max() < 2e-5
        last = got[n - 1]
        assert (last[0] - 25.0 * v[at, 0].double()).norm() < 0.05 * (25.0 * v[at, 0].double()).norm()       # carried whole
        faded = 25.0 * math.exp(-0.05 * back)
        assert (last[1] - faded * v[at, 1].double()).norm() < 0.05 * 25.0 * v[at, 1].double().norm() + 1.0


@pytest.mark.parametrize("d,vd", [(64, 64), (64, 128), (128, 64), (128, 128)])
def test_chunk_sums_on_the_tensor_cores(d, vd):
    """Kernel alone, bfloat16 projections with keys and values of 64 or 128 entries: a chunk's own sum is a product on the
    tensor cores whose float32 operand (the decayed keys) is split in two. Two sequences side by side with a short last
    chunk each; channels that stay open, that fade slowly and that close within a few tokens; compared with the plain
    recurrence on the same rounded projections far below bfloat16's rounding."""
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.base import StateNeed
    from pytorch_transformers_b200.parts.recurrent import RecurrenceChunks
    k = K()
    H, lengths = 3, [300, 449]
    g = torch.Generator().manual_seed(d + vd)
    n = sum(lengths)
    q, kk, v = (bf16_exact(torch.randn(n, H, x, generator=g)).float() for x in (d, d, vd))
    la = -torch.rand(n, H, d, generator=g) * 0.2
    la[:, :, 0] = 0.0                   # never decays
    la[:, :, 1] = -6.0                  # all but gone after one token
    la[:, 1, 2::3] *= 40.0              # a head with many fast channels
    proj = torch.cat([q.reshape(n, -1), kk.reshape(n, -1), v.reshape(n, -1)], 1).bfloat16().cuda()
    refs, lo = [], 0
    for L in lengths:
        refs.append(plain.gla_recurrence(q[lo:lo + L].double() * d ** -0.5, kk[lo:lo + L].double(), v[lo:lo + L].double(),
                                         la[lo:lo + L].double().exp()))
        lo += L
    cache = Cache([(0, None, StateNeed(H * d * vd))], 1024, torch.bfloat16, "cuda", max_slots=len(lengths))
    slots = [cache.open() for _ in lengths]
    ctx = StepContext(cache, slots, [[0] * L for L in lengths], 1, [[]] * len(lengths), [RecurrenceChunks()])
    plan = ctx.plan(RecurrenceChunks.plan_key)
    assert plan.facts["n_chunks"] == sum((L + 63) // 64 for L in lengths)
    chunks = (plan.dev["chunk_seq"], plan.dev["chunk_q0"], plan.dev["seq_chunk0"], plan.facts["n_chunks"])
    entry = type("E", (), {"cache_entry": 0, "state_offset": 0})()
    state = ctx.state_of(entry, H * d * vd)
    got = k.gla(proj, la.reshape(n, -1).cuda().contiguous(), state, ctx.dev["slots"], ctx.batch_c[0], H, d, vd, d ** -0.5, chunks)
    walked = k.gla(proj, la.reshape(n, -1).cuda().contiguous(), torch.zeros_like(state), ctx.dev["slots"], ctx.batch_c[0], H, d,
                   vd, d ** -0.5, None)
    ref = torch.cat([r[0].reshape(-1, H * vd) for r in refs])
    assert row_errors(got, ref).max() < 1e-4, row_errors(got, ref).max()
    assert row_errors(walked, ref).max() < 2e-5
    for i, slot in enumerate(slots):        # the state after the last chunk
        left = state[slot].double().cpu().reshape(H, d, vd)
        assert (left - refs[i][1]).norm() < 1e-5 * refs[i][1].norm()


# ------------------------------------------------------------------------------------------------ the attentions
def capped_spec(m, width, p="mix."):
    from pytorch_transformers_b200.parts.base import PartSpec
    t = m.get("q_temp")
    return PartSpec("mixer", "sink_attention",
                    {"hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                     "scale": m["scale"], "sink": False, "qk_norm": False, "gate": True, "gate_wide": True,
                     "softcap": m.get("softcap") or 0.0, "q_temp": (t["coef"], t["every"]) if t else None},
                    names={n: p + n for n in ("q", "k", "v", "g", "o")})


def windowed_spec(m, width, eps=1e-5, p="mix."):
    from pytorch_transformers_b200.parts.base import PartSpec
    children = {}
    rot, mask = m.get("rot") or {}, m.get("mask") or {}
    if rot.get("dims"):
        children["position"] = PartSpec("position", "rotary", {"head_dim": m["dim"], "theta": rot["base"], "rotary_dim": rot["dims"],
                                                               "factor": (rot.get("scaling") or {}).get("factor", 1.0)})
    names = {n: p + n for n in ("q", "k", "v", "o")}
    names.update({"q_norm": p + "q.norm", "k_norm": p + "k.norm"})
    return PartSpec("mixer", "sink_attention",
                    {"hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                     "scale": m["scale"], "sink": False, "sink_value": 0.0, "qk_norm": True, "qk_gain": True, "norm_first": True,
                     "gate": False, "eps": eps, "window": mask.get("size", 0), "keep_first": mask.get("keep_first", 0) if mask.get("size") else 0},
                    children=children, names=names)


def attention_weights(m, width, seed, gate=False, norms=False):
    g = torch.Generator().manual_seed(seed)
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rn = lambda *s: torch.randn(*s, generator=g)
    w = {"mix.q": 1.2 * rn(H * d, width) / math.sqrt(width), "mix.k": 1.2 * rn(G * d, width) / math.sqrt(width),
         "mix.v": 1.2 * rn(G * vd, width) / math.sqrt(width), "mix.o": 1.2 * rn(width, H * vd) / math.sqrt(H * vd)}
    if gate:
        w["mix.g"] = 1.5 * rn(H * vd, width) / math.sqrt(width)
    if norms:
        w["mix.q.norm"], w["mix.k.norm"] = 1 + 0.2 * rn(d), 1 + 0.2 * rn(d)
    return {kk: bf16_exact(v).float() for kk, v in w.items()}


def copying_weights(m, gate=False, norms=False):
    """Weights under which the mixer's input row is (q of every head | k of every K/V head | v | nothing ...): the test
    writes queries, keys and values directly. The output projection is the identity."""
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    width = (H + G) * d + G * vd
    eye = torch.eye(width)
    w = {"mix.q": eye[:H * d], "mix.k": eye[H * d:(H + G) * d], "mix.v": eye[(H + G) * d:], "mix.o": torch.eye(H * vd)}
    if gate:
        w["mix.g"] = torch.zeros(H * vd, width)
    if norms:
        w["mix.q.norm"], w["mix.k.norm"] = torch.ones(d), torch.ones(d)
    return w, width


CAPPED = [dict(heads=6, kv_heads=2, dim=24, vdim=20, scale=0.6, softcap=4.0, q_temp={"coef": 0.7, "every": 16}),
          dict(heads=3, kv_heads=1, dim=18, vdim=6, scale=0.3),
          dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.2, softcap=7.0, q_temp={"coef": 0.3, "every": 50}),
          dict(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.1, softcap=20.0),
          dict(heads=1, kv_heads=1, dim=8, vdim=16, scale=1.0, softcap=1.0, q_temp={"coef": 1.0, "every": 1})]

WINDOWED = [dict(heads=4, kv_heads=2, dim=16, vdim=20, scale=0.25, mask={"size": 33, "keep_first": 5}, rot={"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0}}),
            dict(heads=5, kv_heads=5, dim=10, vdim=14, scale=0.3, mask={"size": 129, "keep_first": 70}, rot={"base": 10000.0, "dims": 6}),
            dict(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.1, mask={"size": 130, "keep_first": 4}, rot={"base": 1e5, "dims": 32, "scaling": {"factor": 8.0}}),
            dict(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.05, rot={"base": 500.0, "dims": 128}),
            dict(heads=1, kv_heads=1, dim=16, vdim=16, scale=1.0 / 16, mask={"size": 1, "keep_first": 1}),
            dict(heads=2, kv_heads=1, dim=32, vdim=8, scale=0.2, mask={"size": 70, "keep_first": 0})]


def _id(m):
    return f"{m['heads']}h{m['kv_heads']}x{m['dim']}x{m['vdim']}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", CAPPED, ids=_id)
def test_capped_attention_whole_in_portions_and_single_tokens(m, dtype):
    width = 40
    w = attention_weights(m, width, m["dim"], gate=True)
    mixer = Mixer(capped_spec(m, width), w, dtype)
    g = torch.Generator().manual_seed(2)
    x = bf16_exact(torch.randn(200, width, generator=g)).float()
    ref = plain.capped_attention(x.double(), plain.sub(w, "mix."), m)
    cache = mixer.cache(256)
    for cuts in ([200], [130, 70], [64, 2, 3, 17, 114], [60] + [1] * 10 + [130], [1] * 70 + [130]):
        close(mixer.run_cut(cache, x, cuts), ref, dtype, f"cuts {cuts[:6]}", f32=2e-5)
    y = bf16_exact(torch.randn(70, width, generator=g)).float()
    ref_y = plain.capped_attention(y.double(), plain.sub(w, "mix."), m)
    a, b = cache.open(), cache.open()
    out = mixer.step(cache, [a, b], [x[:100], y[:62]])
    got_x, got_y = [out[0]], [out[1]]
    for t in range(8):
        out = mixer.step(cache, [a, b], [x[100 + t:101 + t], y[62 + t:63 + t]])
        got_x.append(out[0]); got_y.append(out[1])
    close(torch.cat(got_x), ref[:108], dtype, "first of two", f32=2e-5)
    close(torch.cat(got_y), ref_y, dtype, "second of two", f32=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", WINDOWED, ids=_id)
def test_windowed_attention_whole_in_portions_and_single_tokens(m, dtype):
    width = 40
    w = attention_weights(m, width, m["dim"] + 1, norms=True)
    mixer = Mixer(windowed_spec(m, width), w, dtype)
    g = torch.Generator().manual_seed(3)
    x = bf16_exact(torch.randn(300, width, generator=g)).float()
    ref = plain.windowed_attention(x.double(), plain.sub(w, "mix."), m, 1e-5)
    cache = mixer.cache(384)
    for cuts in ([300], [130, 170], [64, 2, 3, 17, 214], [120] + [1] * 100 + [80], [1] * 80 + [220]):
        close(mixer.run_cut(cache, x, cuts), ref, dtype, f"cuts {cuts[:6]}", f32=2e-5)
        cache.check()
    y = bf16_exact(torch.randn(150, width, generator=g)).float()
    ref_y = plain.windowed_attention(y.double(), plain.sub(w, "mix."), m, 1e-5)
    a, b = cache.open(), cache.open()
    out = mixer.step(cache, [a, b], [x[:100], y[:62]])
    got_x, got_y = [out[0]], [out[1]]
    for t in range(80):
        out = mixer.step(cache, [a, b], [x[100 + t:101 + t], y[62 + t:63 + t]])
        got_x.append(out[0]); got_y.append(out[1])
    close(torch.cat(got_x), ref[:180], dtype, "first of two", f32=2e-5)
    close(torch.cat(got_y), ref_y[:142], dtype, "second of two", f32=2e-5)


def _needle_rows(m, n, at, g, strength, norms):
    """Input rows for the copying weights: small random queries and keys, random values; the last query and the key at
    `at` lie along one direction (in the entries that are not rotated)."""
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    width = (H + G) * d + G * vd
    x = torch.zeros(n, width)
    x[:, :(H + G) * d] = (0.3 if not norms else 1.0) * torch.randn(n, (H + G) * d, generator=g)
    x[:, (H + G) * d:] = torch.randn(n, G * vd, generator=g)
    lo = (m.get("rot") or {}).get("dims", 0)
    direction = torch.zeros(d)
    direction[lo:] = torch.randn(d - lo, generator=g)
    direction = direction / direction.norm() * strength
    for h in range(H):
        x[n - 1, h * d:(h + 1) * d] = direction
    for c in range(G):
        x[at, (H + c) * d:(H + c + 1) * d] = direction
    return bf16_exact(x).float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [24, 64])
@pytest.mark.parametrize("n,at", [(700, 3), (700, 0), (300, 63), (300, 64), (130, 127), (129, 128), (65, 64), (2, 0)])
def test_capped_attention_finds_one_key_far_back_and_at_page_borders(n, at, d, dtype):
    """Full context: whatever the distance, the aligned key answers. The raw score of 200 is capped at 30."""
    m = dict(heads=2, kv_heads=1, dim=d, vdim=d, scale=0.5, softcap=30.0)
    w, width = copying_weights(m, gate=True)
    mixer = Mixer(capped_spec(m, width), w, dtype)
    g = torch.Generator().manual_seed(n + at)
    x = _needle_rows(m, n, at, g, 20.0, False)
    ref = plain.capped_attention(x.double(), plain.sub(w, "mix."), m)
    value = 0.5 * x[at, -d:].double()          # the gate's logit is 0 everywhere
    cache = mixer.cache(768)
    for cuts in ([n], [n - 1, 1], [max(1, n - 40)] + [1] * min(40, n - 1)):
        got = mixer.run_cut(cache, x, cuts)
        close(got, ref, dtype, f"cuts {cuts[:3]}", f32=2e-5)
        for h in range(2):
            assert (got[-1, h * d:(h + 1) * d] - value).norm() < 0.02 * value.norm()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,window,keep,dims", [(16, 33, 5, 8), (64, 130, 4, 32), (64, 64, 64, 0), (10, 129, 70, 6), (128, 70, 0, 64)])
def test_windowed_attention_sees_a_key_just_inside_and_not_just_outside(d, window, keep, dims, dtype):
    """One aligned key at the window's last place, one further, at the last kept position and the one after it, and at
    position 0; the query is the last token of a prompt, of a second portion, or a single token."""
    m = dict(heads=2, kv_heads=1, dim=d, vdim=d, scale=2.0 / math.sqrt(d), mask={"size": window, "keep_first": keep})
    if dims:
        m["rot"] = {"base": 10000.0, "dims": dims, "scaling": {"factor": 2.0}}
    w, width = copying_weights(m, norms=True)
    mixer = Mixer(windowed_spec(m, width), w, dtype)
    n = window + keep + 150
    cache = mixer.cache(64 * ((n + 63) // 64 + 1))
    places = [(n - window, True), (n - window - 1, keep > n - window - 1), (0, keep > 0), (n - 1, True), (n - 2, window > 1 or keep > n - 2)]
    if keep:
        places += [(keep - 1, True), (keep, keep > keep or n - 1 - keep < window)]
    for at, seen in places:
        g = torch.Generator().manual_seed(at + d)
        x = _needle_rows(m, n, at, g, 1.0, True)
        ref = plain.windowed_attention(x.double(), plain.sub(w, "mix."), m, 1e-5)
        value = x[at, -d:].double()
        for cuts in ([n], [n - 70, 70], [n - 30] + [1] * 30):
            got = mixer.run_cut(cache, x, cuts)
            close(got, ref, dtype, f"key at {at}, cuts {cuts[:2]}", f32=2e-5)
            cache.check()
            # aligned: score 2 sqrt(d) x (share of the unrotated entries); the others' scores are about +-2
            hit = (got[-1, :d] - value).norm() < 0.35 * value.norm()
            if d >= 64:
                assert hit == seen, f"key at {at} of {n}, window {window}, keep {keep}: seen {hit}, expected {seen}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_added_one_takes_weight_when_every_score_is_low(dtype):
    """Scores far below 0: the sink of value 0 holds nearly all the weight and the output shrinks to nearly nothing;
    scores far above 0: it holds nearly none."""
    m = dict(heads=1, kv_heads=1, dim=16, vdim=16, scale=1.0, mask={"size": 1000, "keep_first": 0})
    w, width = copying_weights(m, norms=True)
    mixer = Mixer(windowed_spec(m, width), w, dtype)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(40, width, generator=g)
    direction = torch.randn(16, generator=g)
    x[:, :16], x[:, 16:32] = direction, -direction           # every score = -16
    x = bf16_exact(x).float()
    cache = mixer.cache(64)
    low = mixer.run_cut(cache, x, [40])
    close(low, plain.windowed_attention(x.double(), plain.sub(w, "mix."), m, 1e-5), dtype, "low scores")
    assert float(low.abs().max()) < 1e-4
    x[:, 16:32] = x[:, :16]                                  # every score = +16
    high = mixer.run_cut(cache, x, [40])
    close(high, plain.windowed_attention(x.double(), plain.sub(w, "mix."), m, 1e-5), dtype, "high scores")
    assert float((high[0] - x[0, 32:].double()).abs().max()) < 1e-2


# ------------------------------------------------------------------------------------------------ the feed-forwards
@pytest.mark.parametrize("n,count,keep,top", [(12, 3, 2, 3), (16, 4, 2, 4), (5, 1, 1, 2), (1, 1, 1, 1), (6, 6, 3, 3), (64, 8, 3, 6)])
def test_router_against_the_plain_one(n, count, keep, top):
    k = K()
    g = torch.Generator().manual_seed(n)
    for tokens in (1, 7, 700):
        h = torch.randn(tokens, 24, generator=g)
        wr = torch.randn(n + 1, 24, generator=g)
        r = {"experts": n, "top": top, "scale": 1.5, "groups": {"count": count, "keep": keep}}
        ids, weights = plain.route(h.double(), wr[:n].double(), r)
        got_ids, got_w, logits = k.route(h.cuda(), wr.cuda(), None, count, keep, top, 1.5, "sigmoid", extra=1, group_top=2, normalize=True)
        torch.testing.assert_close(logits.double().cpu(), h.double() @ wr.double().T, atol=1e-5, rtol=1e-5)
        # a choice may differ where two scores are within float32 rounding of each other: compare the sets' scores
        s = torch.sigmoid(h.double() @ wr[:n].double().T)
        same = (got_ids.cpu().long().sort(1).values == ids.sort(1).values).all(1)
        assert same.double().mean() > 0.99
        torch.testing.assert_close(s.gather(1, got_ids.cpu().long()).sort(1).values[same], s.gather(1, ids).sort(1).values[same])
        rows = same.nonzero().flatten()
        order = got_ids.cpu().long()[rows].argsort(1)
        torch.testing.assert_close(got_w.double().cpu()[rows].gather(1, order), weights[rows].gather(1, ids[rows].argsort(1)),
                                   atol=1e-6, rtol=1e-5)


def ff_spec(mlp, width, p="mlp."):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.models.figudra import _feed_forward
    cfg = ptb.FigudraConfig.from_dict({"vocab": 8, "width": width, "layers": [
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.0}, "mlp": mlp}]})
    spec = _feed_forward(cfg, 0)

    def rename(s):
        s.names = {a: b.replace("l0.mlp.", p) for a, b in s.names.items()}
        for c in s.children.values():
            rename(c)
    rename(spec)
    return spec


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mlp,width", [(fm.dense(80), 96), (fm.dense(30), 52), (fm.moe(6, 2, 40, 3, 2, 1.5, shared=24), 96),
                                       (fm.moe(5, 2, 18, shared=10), 52), (fm.moe(1, 1, 16, shared=8), 32), (fm.moe(4, 3, 24), 96),
                                       (fm.moe(16, 4, 64, 4, 2, 2.5, shared=96), 128)])
def test_feed_forwards_against_the_plain_ones(mlp, width, dtype):
    from pytorch_transformers_b200.parts.base import BuildContext, make_part
    cfg = {"vocab": 8, "width": width, "norm": {"eps": 1e-5}, "layers": [dict(fm.att(1, 1, 8, 8, 1.0), mlp=mlp)]}
    w = {kk[3:]: torch.from_numpy(v) for kk, v in fm.make_weights(cfg, width).items() if kk.startswith("l0.mlp.")}
    dt = tdtype(dtype)
    part = make_part(BuildContext(torch.device("cuda"), dt, K()), ff_spec(mlp, width))
    for p in part.walk():
        decls = p.param_decls()
        p.bind({n: w[p.spec.names[n]].to(device="cuda", dtype=torch.float32 if d.role == "vector" else dt) for n, d in decls.items()})
    g = torch.Generator().manual_seed(5)
    for tokens in (1, 9, 300):
        h = bf16_exact(torch.randn(tokens, width, generator=g)).float()
        got = part.forward(h.to(dt).cuda(), None)
        assert got.dtype == torch.float32
        want = plain.feed_forward(h.double(), plain.sub(w, "mlp."), mlp)
        close(got, want, dtype, f"{mlp['kind']} {tokens} tokens", f32=2e-5)
        base = torch.randn(tokens, width, generator=g)
        close(part.forward(h.to(dt).cuda(), None, add=base.cuda()), want + base.double(), dtype, "with the stream", f32=2e-5)


# ------------------------------------------------------------------------------------------------ whole models
class Loaded:
    def __init__(self, tmp, name, dtype):
        import pytorch_transformers_b200 as ptb
        # bfloat16 models run routers that choose every expert (figudra_models.steady says why)
        self.cfg = fm.CONFIGS[name] if dtype == "float32" else fm.steady(fm.CONFIGS[name])
        self.folder = fm.write_folder(tmp, name, seed=len(name), bf16=(dtype == "bfloat16"), cfg=self.cfg)
        self.model = ptb.AutoModelForCausalLM.from_pretrained(self.folder, dtype=dtype)
        self.w = fm.torch_weights(self.cfg, len(name))
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


NAMES = sorted(fm.CONFIGS)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(loaded, name, dtype):
    L = loaded(name, dtype)
    assert L.model.spec.stream_float32 and L.model.use_graphs
    cache = L.model.new_cache(320)
    for ids in fm.prompts(L.cfg, (1, 2, 5, 70, 129, 300), seed=1):
        s = cache.open()
        close(L.model.step(cache, [s], [ids], want="all"), L.plain_logits(ids), dtype, f"{name} {len(ids)} tokens")
        cache.close(s)
    L.model.check_errors()
    cache.check()


def test_residual_stream_after_every_layer(loaded):
    L = loaded("mixed", "float32")
    ids = fm.prompts(L.cfg, (50,), seed=2)[0]
    want, got = [], []
    plain.forward(L.cfg, L.w, ids, streams=want)
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
    assert len(got) == len(want) == 6           # a layer that runs another's weights counts each time
    from pytorch_transformers_b200.parts.base import resolve
    for i, (a, b) in enumerate(zip(got, want)):
        a = resolve(K(), a)
        assert a.dtype == torch.float32 and row_errors(a, b).max() < 1e-5, f"layer {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(256)
    for n, head in ((100, 60), (34, 1), (200, 62)):        # the single tokens cross a page's border and pass the windows
        ids = fm.prompts(L.cfg, (n,), seed=n)[0]
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
    ids = fm.prompts(L.cfg, (150,), seed=portion)[0]
    s = cache.open()
    rows = [L.model.step(cache, [s], [ids[i:i + portion]], want="all") for i in range(0, len(ids), portion)]
    close(torch.cat(rows), L.plain_logits(ids), dtype, f"{name} in portions of {portion}")
    cache.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_a_long_prompt_in_two_portions(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(64 * 9)
    ids = fm.prompts(L.cfg, (530,), seed=12)[0]
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
        reqs = fm.prompts(L.cfg, lengths, seed=10 + seed)
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
    reqs = fm.prompts(L.cfg, (330, 290), seed=5)
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
    prompts = fm.prompts(L.cfg, (9, 1, 30), seed=3)
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
    prompts = fm.prompts(L.cfg, (5, 40), seed=8)
    out = L.model.generate(prompts, max_new_tokens=20, do_sample=True, top_k=20, temperature=0.8, seed=1, eos_token_id=7)
    assert all(len(o) <= len(p) + 20 for o, p in zip(out, prompts))
    again = L.model.generate(prompts, max_new_tokens=20, do_sample=True, top_k=20, temperature=0.8, seed=1, eos_token_id=7)
    assert out == again


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_model_from_config_and_from_folder_are_one_model(tmp_path, dtype):
    import pytorch_transformers_b200 as ptb
    cfg = ptb.FigudraConfig.from_dict(fm.CONFIGS["odd"])
    folder = ptb.write_random_model(cfg, seed=4, folder=str(tmp_path / "m"), dtype=tdtype(dtype))
    a = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    b = ptb.AutoModelForCausalLM.from_config(cfg, seed=4, dtype=dtype)
    ids = fm.prompts(fm.CONFIGS["odd"], (20,), seed=0)
    ca, cb = a.new_cache(64), b.new_cache(64)
    la, lb = a.step(ca, [ca.open()], ids, want="all"), b.step(cb, [cb.open()], ids, want="all")
    torch.testing.assert_close(la, lb, atol=0, rtol=0)
    assert torch.isfinite(la).all() and float(la.std()) > 0


def test_a_checkpoint_gives_the_decay_rank_that_the_configuration_leaves_out(tmp_path):
    import pytorch_transformers_b200 as ptb
    raw = json.loads(json.dumps(fm.CONFIGS["odd"]))
    weights = fm.make_weights(raw, 3)
    del raw["layers"][0]["mixer"]["rank"]
    import tiny_models as tm
    folder = tm.write_model_folder(str(tmp_path / "m"), raw, weights)
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype="float32")
    ids = fm.prompts(raw, (40,), seed=1)[0]
    cache = model.new_cache(64)
    want = plain.forward(fm.CONFIGS["odd"], {kk: torch.from_numpy(v) for kk, v in weights.items()}, ids)
    close(model.step(cache, [cache.open()], [ids], want="all"), want, "float32", "rank from the tensor")


def test_greedy_generation_from_the_command_line(tmp_path):
    """The library's command line on a Figudra folder, as a child process: the design is found by the folder's
    configuration, and the tokens are the plain implementation's."""
    cfg = fm.CONFIGS["odd"]
    folder = fm.write_folder(tmp_path, "odd", seed=6)
    w = fm.torch_weights(cfg, 6)
    prompts = fm.prompts(cfg, (7, 20), seed=9)
    script = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "ptb200-cli")
    args = [sys.executable, script, "run-generation", "--model_name_or_path", folder, "--fp32", "--greedy", "--length", "8"]
    for q in prompts:
        args += ["--prompt_ids", ",".join(map(str, q))]
    done = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    recs = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert [r["prompt_ids"] for r in recs] == prompts
    for q, r in zip(prompts, recs):
        ids = list(q)
        assert len(r["generated_ids"]) == 8
        for tok in r["generated_ids"]:
            logits = plain.forward(cfg, w, ids)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) > 1e-4:          # no test on a tie within float32 rounding
                assert int(logits.argmax()) == tok
            ids.append(tok)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_as_a_child_process(tmp_path, dtype):
    name = "mixed"
    cfg = fm.CONFIGS[name] if dtype == "float32" else fm.steady(fm.CONFIGS[name])
    folder = fm.write_folder(tmp_path, name, seed=2, bf16=(dtype == "bfloat16"), cfg=cfg)
    w = fm.torch_weights(cfg, 2)
    reqs = dict(zip("abc", fm.prompts(cfg, (70, 9, 40), seed=4)))
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
