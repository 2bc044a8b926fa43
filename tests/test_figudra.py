"""Figudra without a GPU: configuration and registry, the spec (tensor names and shapes, one cache entry a layer also
where a layer runs another's weights, pages for the attention layers with their windows and kept first tokens, state
for the gated linear attention), refused configurations and parts, and the plain implementation's own consistency
(the decaying sum carried by hand from one half of a sequence to the next and in closed form, what a window with kept
tokens sees, the added one of the softmax as one more entry, the soft cap's bound, the temperature's steps, the
router's groups)."""
import json
import math

import pytest
import torch

import plain_figudra as plain
import figudra_models as fm


def test_registry_finds_the_design_by_its_architecture_string(tmp_path):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.registry import lookup
    folder = fm.write_folder(tmp_path, "mixed")
    cfg = ptb.AutoConfig.from_pretrained(folder)
    assert isinstance(cfg, ptb.FigudraConfig) and cfg.vocab == 211 and cfg.width == 96 and len(cfg.layers) == 6
    assert cfg.vocab_size == 211 and cfg.hidden_size == 96 and cfg.num_hidden_layers == 6
    assert [cfg.weights_layer(i) for i in range(6)] == [0, 1, 2, 1, 4, 0]
    assert lookup({"architecture": "Figudra"}).model_type == "figudra"
    back = ptb.FigudraConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert back.layers == cfg.layers and back.norm == cfg.norm


@pytest.mark.parametrize("name", sorted(fm.CONFIGS))
def test_spec_names_every_tensor_and_states_every_need(name):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.models.figudra import figudra_spec
    raw = fm.CONFIGS[name]
    cfg = ptb.FigudraConfig.from_dict(raw)
    spec = figudra_spec(cfg)
    assert spec.stream_float32 and spec.head_name == "head" and spec.embedding_norm is not None
    model = ptb.CausalLM(spec, cfg, device="cpu", dtype=torch.float32)
    table, want = model.param_table(), fm.tensor_shapes(raw)
    assert set(table) == set(want)
    for tensor, (_, _, decl) in table.items():
        assert tuple(decl.shape) == tuple(want[tensor]), tensor
    own = [i for i, l in enumerate(raw["layers"]) if l.get("weights_of") is None]
    assert len(model.blocks) == len(own)
    assert [(e.block, e.cache_entry) for e in model.schedule] == \
        [(own.index(l.get("weights_of", i)), i) for i, l in enumerate(raw["layers"])]
    needs = model.cache_needs()
    assert [e for e, _, _ in needs] == list(range(len(raw["layers"])))       # a run of shared weights has its own entry
    for (entry, c, s), layer in zip(needs, raw["layers"]):
        m = layer["mixer"]
        if layer["type"] == "gla":
            assert c is None and s.numel == m["heads"] * m["dim"] * m["vdim"]
        elif layer["type"] == "attention":
            assert s is None and (c.kind, c.kv_heads, c.head_dim, c.v_head_dim) == ("full", m["kv_heads"], m["dim"], m["vdim"])
        else:
            mask = m.get("mask") or {}
            assert s is None and (c.kind, c.window, c.keep_first, c.kv_heads, c.head_dim, c.v_head_dim) == \
                ("window" if mask.get("size") else "full", mask.get("size", 0), mask.get("keep_first", 0), m["kv_heads"],
                 m["dim"], m["vdim"])
    assert model.use_graphs


def test_the_decay_rank_may_come_from_the_checkpoint_alone():
    """Without ``rank`` in the configuration the decay's two matrices are declared with an open size that the loader
    fills from the tensors; weights cannot be drawn at random then."""
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.models.figudra import figudra_spec
    from pytorch_transformers_b200.weights.loader import _fits
    from pytorch_transformers_b200.weights.random_init import random_tensor
    raw = json.loads(json.dumps(fm.CONFIGS["odd"]))
    del raw["layers"][0]["mixer"]["rank"]
    cfg = ptb.FigudraConfig.from_dict(raw)
    table = ptb.CausalLM(figudra_spec(cfg), cfg, device="cpu", dtype=torch.float32).param_table()
    assert tuple(table["l0.mix.a1"][2].shape) == (-1, 52) and tuple(table["l0.mix.a2"][2].shape) == (12, -1)
    assert _fits((3, 52), table["l0.mix.a1"][2].shape) and not _fits((3, 51), table["l0.mix.a1"][2].shape)
    assert not _fits((3,), table["l0.mix.a1"][2].shape)
    with pytest.raises(ValueError):
        random_tensor("l0.mix.a1", table["l0.mix.a1"][2], 0, "cpu", torch.float32)


def _with(name, **changes):
    cfg = json.loads(json.dumps(fm.CONFIGS[name]))
    for path, value in changes.items():
        at = cfg
        keys = path.split("__")
        for k in keys[:-1]:
            at = at[int(k)] if k.isdigit() else at[k]
        at[int(keys[-1]) if keys[-1].isdigit() else keys[-1]] = value
    return cfg


@pytest.mark.parametrize("bad", [
    dict(vocab=0), dict(width=-1), dict(layers=[]), dict(norm={"eps": 0}), dict(layers__0__type="conv"),
    dict(layers__0__mixer__heads=0), dict(layers__0__mixer__kv_heads=4), dict(layers__0__mixer__scale=0),
    dict(layers__0__mixer__softcap=-1.0), dict(layers__0__mixer__q_temp={"coef": 1.0, "every": 0}),
    dict(layers__1__mixer__tau=0), dict(layers__1__mixer__vdim=0), dict(layers__2__mixer__rot__dims=7),
    dict(layers__2__mixer__rot__dims=18), dict(layers__2__mixer__rot__scaling={"factor": 0}), dict(layers__2__mixer__mask__size=-1),
    dict(layers__0__mlp__router__top=5), dict(layers__0__mlp__router__groups={"count": 4, "keep": 2}),
    dict(layers__0__mlp__expert={}), dict(layers__0__mlp__shared={"ff": 0}), dict(layers__1__mlp={"kind": "dense"}),
    dict(layers__1__mlp={"kind": "glu", "ff": 8}), dict(layers__3__weights_of=3), dict(layers__3__weights_of=5),
    dict(layers__3__weights_of=9), dict(layers__3__mixer__tau=2.0),
])
def test_configurations_that_cannot_be_built_are_refused(bad):
    import pytorch_transformers_b200 as ptb
    with pytest.raises(ptb.ConfigError):
        ptb.FigudraConfig.from_dict(_with("mixed", **bad))


def test_keys_that_the_design_does_not_know_and_whole_numbers_written_as_floats_are_taken():
    """A configuration file may carry notes of its writer (a seed, a name), say ``weights_of: null`` for a layer with
    weights of its own and write a count as 16.0; the model is the same."""
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.models.figudra import figudra_spec
    plain_cfg = ptb.FigudraConfig.from_dict(_with("mixed"))
    temp = {"coef": 0.7, "every": 16.0}        # layer 5 runs layer 0's weights: their mixers stay equal
    noted = _with("mixed", seed=11, layers__1__weights_of=None, layers__0__note="first", layers__4__mixer__comment="x",
                  layers__0__mixer__q_temp=temp, layers__5__mixer__q_temp=temp,
                  layers__2__mixer__mask={"size": 33.0, "keep_first": 5.0}, layers__2__mixer__rot__dims=8.0)
    cfg = ptb.FigudraConfig.from_dict(noted)
    assert [cfg.weights_layer(i) for i in range(6)] == [plain_cfg.weights_layer(i) for i in range(6)]
    a, b = figudra_spec(cfg), figudra_spec(plain_cfg)
    assert [blk.children["mixer"].params for blk in a.blocks] == [blk.children["mixer"].params for blk in b.blocks]
    assert [(e.block, e.cache_entry) for e in a.schedule] == [(e.block, e.cache_entry) for e in b.schedule]


def test_parts_refuse_what_their_kernels_do_not_take():
    from pytorch_transformers_b200 import kernels
    from pytorch_transformers_b200.parts.base import BuildContext, PartSpec, make_part
    build = BuildContext(torch.device("cpu"), torch.float32, kernels)
    g = {"hidden": 8, "heads": 1, "dim": 8, "vdim": 8, "tau": 2.0}
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "gla", dict(g, dim=300)))
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "gla", dict(g, tau=0.0)))
    att = {"hidden": 8, "heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.0, "sink": False, "gate": False}
    for bad in (dict(softcap=-1.0), dict(q_temp=(1.0, 0)), dict(gate_wide=True), dict(sink=True, sink_value=0.0),
                dict(norm_first=True, qk_gain=False), dict(talk=True, sink_value=0.0), dict(talk=True, softcap=3.0)):
        with pytest.raises(ValueError):
            make_part(build, PartSpec("mixer", "sink_attention", dict(att, **bad)))
    ex = {"hidden": 8, "inner": 8, "experts": 4, "top": 2}
    with pytest.raises(ValueError):
        make_part(build, PartSpec("feed_forward", "routed_experts", dict(ex, group_score="mean")))
    with pytest.raises(ValueError):
        make_part(build, PartSpec("feed_forward", "routed_experts", dict(ex, shared_gate=True)))      # no shared expert to gate
    with pytest.raises(ValueError):
        make_part(build, PartSpec("feed_forward", "gated", {"hidden": 8, "inner": 8, "activation": "swish"}))


# ------------------------------------------------------------------------------------------------ the oracle with itself
def test_plain_decaying_sum_in_two_halves_and_in_closed_form():
    g = torch.Generator().manual_seed(1)
    T, H, d, dv = 11, 2, 3, 4
    q, k = torch.randn(T, H, d, generator=g, dtype=torch.float64), torch.randn(T, H, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    a = torch.rand(T, H, d, generator=g, dtype=torch.float64)
    whole, S = plain.gla_recurrence(q, k, v, a)
    first, S1 = plain.gla_recurrence(q[:6], k[:6], v[:6], a[:6])
    second, S2 = plain.gla_recurrence(q[6:], k[6:], v[6:], a[6:], S1)
    torch.testing.assert_close(torch.cat([first, second]), whole)
    torch.testing.assert_close(S2, S)
    # closed form: o_t = sum_{j <= t} (sum_c q_t[c] k_j[c] prod_{j < s <= t} a_s[c]) v_j
    t = 7
    o = torch.zeros(H, dv, dtype=torch.float64)
    for j in range(t + 1):
        w = (q[t] * k[j] * a[j + 1:t + 1].prod(0)).sum(-1)
        o += w[:, None] * v[j]
    torch.testing.assert_close(o, whole[t])


def test_plain_decay_is_the_sigmoid_to_the_power_one_over_tau():
    h = torch.randn(5, 6, dtype=torch.float64)
    w = {"a1": torch.randn(2, 6, dtype=torch.float64), "a2": torch.randn(8, 2, dtype=torch.float64),
         "a2.b": torch.randn(8, dtype=torch.float64)}
    a1, a4 = plain.gla_decay(h, w, 2, 4, 1.0), plain.gla_decay(h, w, 2, 4, 4.0)
    torch.testing.assert_close(a4 ** 4, a1)
    assert a1.shape == (5, 2, 4) and float(a1.min()) > 0 and float(a4.max()) < 1


def test_plain_window_with_kept_first_tokens():
    vis = plain.window_visible(10, 3, 2)
    assert vis[9].tolist() == [True, True, False, False, False, False, False, True, True, True]
    assert vis[2].tolist() == [True, True, True] + [False] * 7
    assert plain.window_visible(4, 1, 0).int().tolist() == torch.eye(4).int().tolist()


def test_plain_softmax_with_one_added_is_a_softmax_with_one_more_entry():
    g = torch.Generator().manual_seed(3)
    T, W = 6, 20
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 0.5}
    w = {"q": torch.randn(8, W, generator=g, dtype=torch.float64), "k": torch.randn(4, W, generator=g, dtype=torch.float64),
         "v": torch.randn(3, W, generator=g, dtype=torch.float64), "o": torch.eye(6, dtype=torch.float64),
         "q.norm": torch.ones(4, dtype=torch.float64), "k.norm": torch.ones(4, dtype=torch.float64)}
    got = plain.windowed_attention(h, w, m, 1e-6).reshape(T, 2, 3)
    q = plain.rms((h @ w["q"].T).reshape(T, 2, 4), 1e-6)
    k = plain.rms((h @ w["k"].T).reshape(T, 1, 4), 1e-6)
    v = h @ w["v"].T
    t = 4
    for hh in range(2):
        s = torch.cat([(q[t, hh] @ k[:t + 1, 0].T) * 0.5, torch.zeros(1, dtype=torch.float64)])     # the last entry: score 0, no value
        p = torch.softmax(s, 0)
        torch.testing.assert_close(p[:-1] @ v[:t + 1], got[t, hh])


def test_plain_temperature_steps_and_cap_bound():
    p = torch.arange(0, 40)
    f = plain.query_temperature(p, 0.5, 16)
    assert float(f[0]) == 1.0 and float(f[14]) == 1.0 and math.isclose(float(f[15]), 1 + 0.5 * math.log(2.0))
    assert math.isclose(float(f[31]), 1 + 0.5 * math.log(3.0)) and float(f[30]) == float(f[15])
    g = torch.Generator().manual_seed(5)
    T, W = 9, 12
    h = torch.randn(T, W, generator=g, dtype=torch.float64) * 4
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 3.0, "softcap": 0.01}
    w = {"q": torch.randn(4, W, generator=g, dtype=torch.float64), "k": torch.randn(4, W, generator=g, dtype=torch.float64),
         "v": torch.randn(4, W, generator=g, dtype=torch.float64), "g": torch.zeros(4, W, dtype=torch.float64),
         "o": torch.eye(4, dtype=torch.float64)}
    # a cap that small flattens the scores: every row is (nearly) the mean of the values so far, times sigmoid(0)
    got = plain.capped_attention(h, w, m)
    v = h @ w["v"].T
    want = torch.stack([v[:t + 1].mean(0) for t in range(T)]) * 0.5
    assert float((got - want).abs().max()) < 0.02 * float(v.abs().max())


def test_plain_router_chooses_within_the_best_groups():
    g = torch.Generator().manual_seed(7)
    h = torch.randn(50, 10, generator=g, dtype=torch.float64)
    w = torch.randn(12, 10, generator=g, dtype=torch.float64)
    r = {"experts": 12, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    ids, weights = plain.route(h, w, r)
    s = torch.sigmoid(h @ w.T)
    for t in range(50):
        gs = [sorted(s[t, 3 * c:3 * c + 3].tolist())[-2:] for c in range(4)]
        best = sorted(range(4), key=lambda c: -sum(gs[c]))[:2]
        assert all(int(e) // 3 in best for e in ids[t])
        allowed = sorted((float(s[t, e]) for e in range(12) if e // 3 in best), reverse=True)[:3]
        assert sorted((float(s[t, e]) for e in ids[t]), reverse=True) == allowed
        assert math.isclose(float(weights[t].sum()), 2.0, rel_tol=1e-12)
