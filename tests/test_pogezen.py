"""Pogezen without a GPU: configuration and registry, the spec (tensor names and shapes, one cache entry a layer,
pages for the attention layers with their kept first tokens, state for the input filter and the matrix memory),
refused configurations, the cache's pages under a window that keeps first tokens, and the plain implementation's
own consistency (the matrix memory carried by hand from one half of a sequence to the next and in its closed
form; what a window with kept tokens sees; the filter in two halves; mixed weights as sums of per-head results)."""
import json
import math

import pytest
import torch

import plain_pogezen as plain
import pogezen_models as pm


def test_registry_finds_the_design_by_its_architecture_string(tmp_path):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.registry import lookup
    folder = pm.write_folder(tmp_path, "mixed")
    cfg = ptb.AutoConfig.from_pretrained(folder)
    assert isinstance(cfg, ptb.PogezenConfig) and cfg.vocab == 211 and cfg.width == 96 and len(cfg.layers) == 5
    assert cfg.vocab_size == 211 and cfg.hidden_size == 96 and cfg.num_hidden_layers == 5
    assert lookup({"architecture": "Pogezen"}).model_type == "pogezen"
    back = ptb.PogezenConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert back.layers == cfg.layers and back.canon == cfg.canon and back.embedding == cfg.embedding


@pytest.mark.parametrize("name", sorted(pm.CONFIGS))
def test_spec_names_every_tensor_and_states_every_need(name):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200 import kernels
    from pytorch_transformers_b200.models.pogezen import pogezen_spec
    raw = pm.CONFIGS[name]
    cfg = ptb.PogezenConfig.from_dict(raw)
    spec = pogezen_spec(cfg)
    assert spec.stream_float32 and spec.head_name is None and spec.embedding_scale == raw["embedding"]["scale"]
    model = ptb.CausalLM(spec, cfg, device="cpu", dtype=torch.float32)
    table, want = model.param_table(), pm.tensor_shapes(raw)
    assert set(table) == set(want)
    for tensor, (_, _, decl) in table.items():
        assert tuple(decl.shape) == tuple(want[tensor]), tensor
    needs = model.cache_needs()
    assert [e for e, _, _ in needs] == list(range(len(raw["layers"])))
    filt = (raw["canon"]["taps"] - 1) * raw["width"]
    for (entry, c, s), layer in zip(needs, raw["layers"]):
        m = layer["mixer"]
        if layer["type"] == "mlstm":
            assert c is None and s.numel == filt + kernels.mlstm_state_floats(m["heads"], m["dim"], m["vdim"])
            assert kernels.mlstm_state_floats(m["heads"], m["dim"], m["vdim"]) >= m["heads"] * (m["dim"] * m["vdim"] + m["dim"] + 1)
        else:
            assert (c.kind, c.kv_heads, c.head_dim, c.window, c.v_head_dim, c.keep_first) == \
                ("window", m["kv_heads"], m["dim"], m["mask"]["size"], m["vdim"], m["mask"]["keep_first"])
            assert (s is None and filt == 0) or s.numel == filt
    mixes = [b.children["mixer"].inner.value_mix for b in model.blocks if b.children["mixer"].inner.spec.kind == "sink_attention"]
    said = [bool(l["mixer"].get("v_mix")) for l in raw["layers"] if l["type"] == "attention"]
    assert [x != "none" for x in mixes] == said and mixes.count("source") == (1 if any(said) else 0)
    assert [x for x in mixes if x != "none"][:1] in ([], ["source"])
    assert model.use_graphs


def _with(name, **changes):
    cfg = json.loads(json.dumps(pm.CONFIGS[name]))
    for path, value in changes.items():
        at = cfg
        keys = path.split("__")
        for k in keys[:-1]:
            at = at[int(k)] if k.isdigit() else at[k]
        at[int(keys[-1]) if keys[-1].isdigit() else keys[-1]] = value
    return cfg


@pytest.mark.parametrize("bad", [
    dict(vocab=0), dict(width=-1), dict(layers=[]), dict(norm={"eps": 0}), dict(canon={"taps": 0}), dict(canon={"taps": 9}),
    dict(layers__0__type="conv"), dict(layers__0__mixer__heads=0), dict(layers__0__mixer__kv_heads=4),
    dict(layers__0__mixer__scale=0), dict(layers__0__mixer__rot__dims=7), dict(layers__0__mixer__rot__dims=26),
    dict(layers__0__mixer__rot__scaling={"factor": 2.0}), dict(layers__0__mixer__mask__size=-1),
    dict(layers__1__mixer__gate_cap=0), dict(layers__1__mixer__vdim=0), dict(layers__2__mixer__vdim=24),
    dict(layers__0__mlp={"kind": "moe", "ff": 8}), dict(layers__0__mlp={"kind": "dense"}),
])
def test_configurations_that_cannot_be_built_are_refused(bad):
    import pytorch_transformers_b200 as ptb
    with pytest.raises(ptb.ConfigError):
        ptb.PogezenConfig.from_dict(_with("mixed", **bad))


def test_parts_refuse_what_their_kernels_do_not_take():
    from pytorch_transformers_b200 import kernels
    from pytorch_transformers_b200.parts.base import BuildContext, PartSpec, make_part
    build = BuildContext(torch.device("cpu"), torch.float32, kernels)
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "mlstm", {"hidden": 8, "heads": 1, "dim": 300, "vdim": 8}))
    inner = PartSpec("mixer", "mlstm", {"hidden": 8, "heads": 1, "dim": 8, "vdim": 8})
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "input_conv", {"hidden": 8, "taps": 9}, children={"inner": inner}))
    att = {"hidden": 8, "heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.0, "sink": False, "gate": False}
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "sink_attention", dict(att, keep_first=3)))           # kept tokens without a window
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "sink_attention", dict(att, value_mix="all")))
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "sink_attention", dict(att, talk=True, sink=True)))
    wrapped = make_part(build, PartSpec("mixer", "input_conv", {"hidden": 8, "taps": 3}, children={"inner": inner}))
    assert wrapped.state_need().numel == 2 * 8 + kernels.mlstm_state_floats(1, 8, 8) and wrapped.cache_need() is None


def test_pages_behind_the_window_go_back_but_the_kept_first_ones_stay():
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.parts.base import CacheNeed
    cache = Cache([(0, CacheNeed("window", 1, 8, window=70, v_head_dim=4, keep_first=65), None)], 64 * 8, torch.float32, "cpu")
    s = cache.open()
    for _ in range(6):
        cache.reserve(s, 64)
        cache.commit(s, 64)
    pages = cache.pages(s, 0)
    # 384 tokens: the next query sees positions > 384 - 70, that is from page 4 on, and the first 65 positions (two pages)
    assert [p >= 0 for p in pages] == [True, True, False, False, True, True]
    cache.check()
    cache.close(s)
    assert cache.groups[0].pool.in_use == 0


def test_plain_matrix_memory_in_two_halves_and_in_closed_form():
    g = torch.Generator().manual_seed(3)
    T, H, d, vd = 40, 2, 5, 7
    q, k = torch.randn(T, H, d, generator=g, dtype=torch.float64), torch.randn(T, H, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, H, vd, generator=g, dtype=torch.float64)
    i, f = torch.randn(T, H, generator=g, dtype=torch.float64) * 3, -torch.rand(T, H, generator=g, dtype=torch.float64)
    whole = plain.matrix_memory(q, k, v, i, f)
    # closed form: with F_t the running sum of f, the weight of key j at t is exp(F_t - F_j + i_j - m_t), and
    # m_t = max(F_t, max_j (F_t - F_j + i_j)) because the maximum starts at zero
    F = f.cumsum(0)
    for t in (0, 7, 39):
        logw = F[t][None] - F[:t + 1] + i[:t + 1]                     # [j, H]
        m = torch.maximum(F[t], logw.max(0).values)
        wgt = torch.exp(logw - m)
        num = torch.einsum("jh,jhd,jhv,hd->hv", wgt, k[:t + 1], v[:t + 1], q[t])
        nq = torch.einsum("jh,jhd,hd->h", wgt, k[:t + 1], q[t])
        ref = num / (torch.maximum(nq.abs(), torch.exp(-m)) + 1e-6)[:, None]
        torch.testing.assert_close(whole[t], ref, atol=1e-12, rtol=1e-10)
    assert (whole[:5] - plain.matrix_memory(q[:5], k[:5], v[:5], i[:5], f[:5])).abs().max() == 0     # causal


def test_plain_window_with_kept_tokens_sees_exactly_what_it_should():
    see = plain.visible(12, 4, 2)
    assert see[10].nonzero().flatten().tolist() == [0, 1, 7, 8, 9, 10]
    assert see[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert see[5].nonzero().flatten().tolist() == [0, 1, 2, 3, 4, 5]       # 2 is the window's last, 0 and 1 are kept
    assert plain.visible(5, 0, 0).sum() == 15                                # no window: all earlier positions


def test_plain_filter_is_causal_and_reads_taps_minus_one_inputs_back():
    g = torch.Generator().manual_seed(5)
    h, filt = torch.randn(9, 4, generator=g, dtype=torch.float64), torch.randn(4, 3, generator=g, dtype=torch.float64)
    y = plain.input_conv(h, filt)
    torch.testing.assert_close(y[0], h[0] + filt[:, 2] * h[0])
    torch.testing.assert_close(y[5], h[5] + filt[:, 0] * h[3] + filt[:, 1] * h[4] + filt[:, 2] * h[5])
    assert (plain.input_conv(h[:6], filt) - y[:6]).abs().max() == 0


def test_plain_rotation_keeps_length_up_to_its_factor_and_leaves_the_rest():
    rot = {"base": 100.0, "dims": 6, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, mult = plain.rotary_frequencies(rot)
    plain_f = 100.0 ** (-2.0 * torch.arange(3, dtype=torch.float64) / 6)
    assert mult == pytest.approx(0.1 * math.log(4.0) + 1) and (f <= plain_f).all() and (f >= plain_f / 4).all()
    x = torch.randn(5, 2, 10, dtype=torch.float64)
    y = plain.rotate(x, torch.arange(5), rot)
    assert (y[..., 6:] - x[..., 6:]).abs().max() == 0
    torch.testing.assert_close(y[..., :6].norm(dim=-1), mult * x[..., :6].norm(dim=-1))
    assert (plain.rotate(x, torch.arange(5), None) - x).abs().max() == 0
