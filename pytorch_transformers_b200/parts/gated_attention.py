"""Attention with separate query, key and value projections, and what some designs put around the softmax:

* a norm of queries and keys per head (RMS over the head's ``dim`` entries, one gain [dim] for all heads);
* no position in the scores, or a rotation from a ``position`` child (not built here: the scores of this
  mixer carry no position);
* a sliding window: position i sees j with 0 <= i - j < window (0: all earlier positions);
* a sink: one learned logit per head that takes part in the softmax's normalisation only: ``exp(sink)`` is one
  more term of the denominator, used as stored (``scale`` does not touch it), and nothing is read for it;
* an output gate: head h's result times sigmoid(W_g x)_h, one number per head, read from the mixer's input; with
  ``gate_wide`` W_g has heads * vdim rows and every entry of the concatenated heads has a gate of its own;
* a sink of a fixed value instead of a learned one (``sink_value``; 0 adds one to every softmax's denominator);
* a soft cap on the scores (``softcap``): score <- softcap * tanh(score / softcap) after the scale;
* a query temperature (``q_temp`` = (coef, every)): the query at position p is multiplied by
  1 + coef ln(floor((p + 1) / every) + 1);
* a norm with gains that comes before the rotation (``norm_first``);
* values of a size of their own (``vdim``);
* biases on the four projections (``bias``), added in float32 where queries, keys and values are laid out;
* a rotation of queries and keys from a ``position`` child, applied before the norm of queries and keys, and a
  norm without gains (``qk_gain=False``: plain division by the root mean square);
* first positions that stay visible left of the window (``keep_first``): i sees j if j <= i and
  (i - j < window or j < keep_first); they keep their true positions;
* a mixing of the heads' softmax weights after the softmax (``talk``): w'_h(i, j) = sum_g T[h, g] w_g(i, j) with a
  learned T [heads, heads]; head h applies the mixed weights to the values of its own K/V head. The kernel forms
  every head's weights on every K/V head's values and a second one sums them with T, which is the same;
* a mixing of values across layers (``value_mix``): a ``"source"`` layer leaves its values for the later layers of
  the step; a ``"mix"`` layer caches (1 - lam) v + lam v_source with one learned scalar lam, the same token's values.

score = (q . k) * scale. Query head h reads K/V head h // (heads / kv_heads). Scores, softmax and the
norms' statistics are float32. The four input projections are one matrix [q | k | v | g] and one product;
``forward_projected`` lets a ``pair`` mixer run that product together with another mixer's.
"""
from __future__ import annotations

from typing import Dict

import torch

from .attention import MAX_HEAD_DIM, AttentionTiles
from .base import BuildContext, CacheNeed, ParamDecl, Part, PartSpec, register_part
from .linear import linear, linear_pending


@register_part("mixer", "sink_attention")
class SinkAttention(Part):
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int,
                 scale: float, window: int = 0, eps: float = 1e-6, qk_norm: bool = True, sink: bool = True,
                 gate: bool = True, bias: bool = False, qk_gain: bool = True, keep_first: int = 0, talk: bool = False,
                 value_mix: str = "none", value_mix_key: str = "values", softcap: float = 0.0, q_temp=None,
                 gate_wide: bool = False, sink_value=None, norm_first: bool = False):
        super().__init__(build, spec)
        if heads % kv_heads:
            raise ValueError(f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        if not (0 < dim <= MAX_HEAD_DIM and 0 < vdim <= MAX_HEAD_DIM):
            raise ValueError(f"the attention kernels take head sizes from 1 to {MAX_HEAD_DIM}, got {dim} and {vdim}")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.window, self.eps = float(scale), int(window), float(eps)
        self.qk_norm, self.has_sink, self.has_gate = bool(qk_norm), bool(sink), bool(gate)
        self.has_bias, self.qk_gain, self.keep_first, self.talk = bool(bias), bool(qk_gain), int(keep_first), bool(talk)
        if value_mix not in ("none", "source", "mix"):
            raise ValueError(f"value_mix is 'none', 'source' or 'mix', got {value_mix!r}")
        if self.keep_first < 0 or (self.keep_first > 0 and self.window <= 0):
            raise ValueError("keep_first needs a window and must not be negative")
        if self.talk and (self.has_sink or self.has_gate):
            raise ValueError("mixed softmax weights go with neither a sink nor an output gate")
        self.value_mix, self.value_mix_key = value_mix, str(value_mix_key)
        self.softcap, self.gate_wide, self.norm_first = float(softcap or 0.0), bool(gate_wide), bool(norm_first)
        self.q_temp = None if not q_temp else (float(q_temp[0]), int(q_temp[1]))
        self.sink_value = None if sink_value is None else float(sink_value)
        if self.softcap < 0 or (self.q_temp is not None and self.q_temp[1] <= 0):
            raise ValueError("softcap must not be negative and q_temp's period must be positive")
        if self.sink_value is not None and self.has_sink:
            raise ValueError("a sink is learned (sink=True) or has a fixed value (sink_value), not both")
        if self.gate_wide and not self.has_gate:
            raise ValueError("gate_wide needs gate=True")
        if self.talk and (self.softcap or self.sink_value is not None):
            raise ValueError("mixed softmax weights go with neither a sink nor a soft cap")
        if self.norm_first and not (self.qk_norm and self.qk_gain):
            raise ValueError("norm_first is the norm with gains before the rotation (qk_norm and qk_gain)")
        self.gate_cols = (self.heads * self.vdim if self.gate_wide else self.heads) if self.has_gate else 0
        self.position = self.children.get("position")
        # the second path: rotation, biases, kept first positions, mixed weights or mixed values
        self.extended = bool(self.position is not None or self.has_bias or self.keep_first or self.talk
                             or self.value_mix != "none" or (self.qk_norm and not self.qk_gain) or self.norm_first
                             or self.q_temp is not None)
        self.p_in = self.p_o = self.p_q_norm = self.p_k_norm = self.p_sink = None
        self.p_in_b = self.p_o_b = self.p_talk = self.p_vmix = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, G, d, vd = self.heads, self.kv_heads, self.dim, self.vdim
        decls = {"q": ParamDecl((H * d, self.hidden)), "k": ParamDecl((G * d, self.hidden)),
                 "v": ParamDecl((G * vd, self.hidden)), "o": ParamDecl((self.hidden, H * vd))}
        if self.qk_norm and self.qk_gain:
            decls["q_norm"] = ParamDecl((d,), role="vector", init="one_plus_normal", std=0.1)
            decls["k_norm"] = ParamDecl((d,), role="vector", init="one_plus_normal", std=0.1)
        if self.has_sink:
            decls["sink"] = ParamDecl((H,), role="vector", std=1.0)
        if self.has_gate:
            decls["g"] = ParamDecl((self.gate_cols, self.hidden))
        if self.has_bias:
            decls.update({"q_b": ParamDecl((H * d,), role="vector", std=0.5), "k_b": ParamDecl((G * d,), role="vector", std=0.5),
                          "v_b": ParamDecl((G * vd,), role="vector", std=0.5), "o_b": ParamDecl((self.hidden,), role="vector")})
            if self.has_gate:
                decls["g_b"] = ParamDecl((self.gate_cols,), role="vector")
        if self.talk:
            decls["talk"] = ParamDecl((H, H), role="vector", std=0.5)
        if self.value_mix != "none":
            decls["vmix"] = ParamDecl((), role="vector", std=0.5)     # a source layer stores one too and does not use it
        return decls

    def bind(self, t: Dict[str, torch.Tensor]) -> None:
        rows = [t["q"], t["k"], t["v"]] + ([t["g"]] if self.has_gate else [])
        self.p_in = torch.cat(rows).contiguous()
        self.p_o = t["o"]
        self.p_q_norm, self.p_k_norm, self.p_sink = t.get("q_norm"), t.get("k_norm"), t.get("sink")
        if self.sink_value is not None:
            self.p_sink = torch.full((self.heads,), self.sink_value, dtype=torch.float32, device=t["q"].device)
        if self.has_bias:
            self.p_in_b = torch.cat([t["q_b"], t["k_b"], t["v_b"]] + ([t["g_b"]] if self.has_gate else [])).contiguous()
            self.p_o_b = t["o_b"]
        self.p_talk, self.p_vmix = t.get("talk"), t.get("vmix")

    # ---- the projected protocol (parts/pair.py)
    def in_rows(self) -> int:
        return (self.heads + self.kv_heads) * self.dim + self.kv_heads * self.vdim + self.gate_cols

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def in_weight(self):
        return self.p_in

    def out_weight(self):
        return self.p_o

    def release_projections(self) -> None:
        self.p_in = self.p_o = None

    def cache_need(self):
        return CacheNeed("window" if self.window > 0 else "full", self.kv_heads, self.dim, self.window, v_head_dim=self.vdim,
                         keep_first=self.keep_first)

    def state_need(self):
        return None

    def planner(self):
        return AttentionTiles(self.build.kernels)

    def forward_projected(self, proj, ctx, entry, out, out_scale: float = 1.0) -> None:
        """``proj`` [tokens, in_rows()] -> the gated heads [tokens, heads * vdim] times ``out_scale`` into ``out``."""
        k = self.build.kernels
        k_pool, v_pool, group = ctx.cache.entry_storage(entry.cache_entry)
        batch = ctx.batch_c[group]
        if self.extended:
            return self._forward_extended(proj, ctx, entry, out, out_scale, k_pool, v_pool, batch)
        q = k.qk_norm_store(proj, k_pool, v_pool, batch, self.p_q_norm, self.p_k_norm, self.heads, self.kv_heads, self.dim,
                            self.vdim, self.eps, write_cache=entry.writes_cache)
        gate = proj[:, self.in_rows() - self.gate_cols:] if self.has_gate else None
        tiles = ctx.plan(AttentionTiles.plan_key)
        extras = {"softcap": self.softcap, "gate_wide": self.gate_wide}
        if (q.dtype == torch.bfloat16 and self.dim == self.vdim and k.attention_mma_supports(self.dim)
                and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0 and self._gate_fits_mma(gate)):
            # bfloat16 with a head size of the tensor-core kernel: tiles of tokens x heads of a K/V group; a step of
            # single tokens divides each sequence's visible pages among blocks that a second kernel joins
            tokens = tiles.facts["mma_tokens"]
            q_per_kv = self.heads // self.kv_heads
            if tokens == 1:
                hpk = min(q_per_kv, 128)
                warps, splits = (hpk + 15) // 16, self._decode_splits(ctx, hpk)
            else:
                warps, splits = 8, 1
                hpk = max(1, min(q_per_kv, 128 // tokens))
            k.attention_mma(q, k_pool, v_pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"], tiles.facts["n_mma_tiles"],
                            None, self.kv_heads, self.scale, self.window, tokens, hpk, warps, splits, sinks=self.p_sink,
                            gate=gate, out_scale=out_scale, out=out, wide_weights=True, **extras)
            return
        k.attention_generic(q, k_pool, v_pool, batch, tiles.dev["tile_seq"], tiles.dev["tile_q0"], tiles.facts["n_tiles"],
                            None, self.kv_heads, self.scale, self.window, sinks=self.p_sink, gate=gate, out_scale=out_scale,
                            out=out, **extras)

    def _gate_fits_mma(self, gate) -> bool:
        """A gate per entry is read two entries at a time by the tensor-core kernel: whole 32-bit words."""
        return gate is None or not self.gate_wide or (gate.data_ptr() % 4 == 0 and gate.stride(0) % 2 == 0)

    def _forward_extended(self, proj, ctx, entry, out, out_scale, k_pool, v_pool, batch) -> None:
        k = self.build.kernels
        if self.qk_norm and self.qk_gain and not self.norm_first:
            raise ValueError("sink_attention: a rotation, biases, kept first positions, mixed weights or mixed values go "
                             "with a norm of queries and keys without gains (qk_gain=False), with one before the rotation "
                             "(norm_first=True) or with none")
        if self.has_gate and self.has_bias:
            raise ValueError("sink_attention: an output gate with a bias is not built")
        H, G, d, vd = self.heads, self.kv_heads, self.dim, self.vdim
        first = ctx.shared.get(self.value_mix_key) if self.value_mix == "mix" else None
        if self.value_mix == "mix" and first is None:
            raise ValueError(f"sink_attention: no earlier layer of this step left values under {self.value_mix_key!r}")
        rope = ctx.rope(self.position) if self.position is not None else None
        res = k.rope_norm_store(proj, self.p_in_b, k_pool, v_pool, batch, rope, H, G, d, vd, self.eps,
                                unit_norm=self.qk_norm, v_first=first, lam=self.p_vmix, keep_values=self.value_mix == "source",
                                write_cache=entry.writes_cache, q_gain=self.p_q_norm if self.norm_first else None,
                                k_gain=self.p_k_norm if self.norm_first else None, norm_first=self.norm_first,
                                q_temp=self.q_temp)
        if self.value_mix == "source":
            q, ctx.shared[self.value_mix_key] = res
        else:
            q = res
        tiles = ctx.plan(AttentionTiles.plan_key)
        gate = proj[:, self.in_rows() - self.gate_cols:] if self.has_gate else None
        extras = {"softcap": self.softcap, "gate_wide": self.gate_wide}
        if self.talk and out_scale != 1.0:
            raise ValueError("sink_attention: mixed softmax weights take no output factor")
        if (q.dtype == torch.bfloat16 and d == vd and k.attention_mma_supports(d) and out.stride(0) % 2 == 0
                and out.data_ptr() % 4 == 0 and self._gate_fits_mma(gate)):
            # the tensor-core kernel, tiled as in forward_projected; with mixed weights a block forms one K/V group's
            # weights on one K/V head's values, float32, and talk_mix sums them
            tokens, q_per_kv = tiles.facts["mma_tokens"], H // G
            if tokens == 1:
                hpk = min(q_per_kv, 128)
                warps, splits = (hpk + 15) // 16, self._decode_splits(ctx, hpk, G if self.talk else 1)
            else:
                warps, splits = 8, 1
                hpk = max(1, min(q_per_kv, 128 // tokens))
            margs = (q, k_pool, v_pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"], tiles.facts["n_mma_tiles"], None,
                     G, self.scale, self.window, tokens, hpk, warps, splits)
            if self.talk:
                k.talk_mix(k.attention_mma(*margs, wide_weights=True, keep_first=self.keep_first, wide=True), self.p_talk,
                           q.dtype, out=out)
            else:
                k.attention_mma(*margs, sinks=self.p_sink, gate=gate, out_scale=out_scale, out=out, wide_weights=True,
                                keep_first=self.keep_first, **extras)
            return
        args = (q, k_pool, v_pool, batch, tiles.dev["tile_seq"], tiles.dev["tile_q0"], tiles.facts["n_tiles"], None, G,
                self.scale, self.window)
        if self.talk:
            k.talk_mix(k.attention_generic(*args, keep_first=self.keep_first, wide=True), self.p_talk, q.dtype, out=out)
            return
        k.attention_generic(*args, sinks=self.p_sink, gate=gate, out_scale=out_scale, out=out, keep_first=self.keep_first,
                            **extras)

    def _decode_splits(self, ctx, hpk: int, value_heads: int = 1) -> int:
        """Blocks per (sequence, K/V head) in a step of single tokens: enough to fill the device, each with two
        pages of visible keys at least. ``value_heads``: K/V heads whose values each group's weights meet."""
        k = self.build.kernels
        q_per_kv = self.heads // self.kv_heads
        blocks = ctx.n_seqs * self.kv_heads * ((q_per_kv + hpk - 1) // hpk) * value_heads
        pages = ctx.pages_hint
        if self.window > 0:
            pages = min(pages, self.window // k.PAGE + 2 + (self.keep_first + k.PAGE - 1) // k.PAGE)
        return max(1, min((2 * k.sm_count(self.build.device)) // blocks, pages // 2, 64))

    fuses_add = True

    def forward(self, x, ctx, entry, add=None):
        return linear(self.build.kernels, self._heads(x, ctx, entry), self.p_o, self.p_o_b, add=add)

    def forward_pending(self, x, ctx, entry):
        """The mixer's result as the last product's float32 sums and its bias, for a kernel that adds them to the
        stream later."""
        return linear_pending(self.build.kernels, self._heads(x, ctx, entry), self.p_o, self.p_o_b)

    def _heads(self, x, ctx, entry):
        k = self.build.kernels
        proj = linear(k, x, self.p_in)      # biases, where there are any, are added where q, k, v are laid out
        heads = torch.empty((x.shape[0], self.out_columns()), dtype=x.dtype, device=x.device)
        self.forward_projected(proj, ctx, entry, heads)
        return heads
