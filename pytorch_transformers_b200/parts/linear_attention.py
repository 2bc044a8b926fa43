"""Linear attention with a fixed decay per head (lightning attention).

With ``h`` the mixer's input, per head (``dim`` entries of queries and keys, ``vdim`` of values):

    q = silu(W_q h), k = silu(W_k h), v = silu(W_v h)
    S_t = decay_head * S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t,      S = 0 before the first token
    out = W_o ( rmsnorm(o over all heads side by side) * gain * sigmoid(W_g h) )

Per sequence the mixer keeps S [heads, dim, vdim] in the cache's state area (float32, zero when a sequence
starts) and needs no pages. State, decays and the norm are float32 whatever the model dtype. Prompts of
256 tokens or more run in chunks of 64 (a chunk's own sum, the chunks joined in order, the outputs), shorter
steps token by token; the two differ by float32 rounding. The four input projections are one matrix
[q | k | v | g]; ``forward_projected`` lets a ``pair`` mixer run that product together with another mixer's.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from .base import BuildContext, ParamDecl, Part, PartSpec, StateNeed, register_part
from .linear import linear
from .recurrent import SCAN_CHUNK, RecurrenceChunks


@register_part("mixer", "linear_attention")
class LinearAttention(Part):
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, heads: int, dim: int, vdim: int,
                 decay: Sequence[float], eps: float = 1e-6, activation: str = "silu", gate: bool = True):
        super().__init__(build, spec)
        self.hidden, self.heads, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        if len(decay) != self.heads:
            raise ValueError(f"linear attention wants one decay per head: {len(decay)} for {self.heads} heads")
        if activation not in ("silu", "none"):
            raise ValueError(f"linear attention's activation is 'silu' or 'none', got {activation!r}")
        if SCAN_CHUNK != build.kernels.LINEAR_ATTENTION_CHUNK:
            raise ValueError("the chunk planner and the chunked kernel disagree on the chunk's size")
        self.eps, self.activation, self.has_gate = float(eps), activation, bool(gate)
        self.decay = torch.tensor([float(a) for a in decay], dtype=torch.float32, device=build.device)
        self.p_in = self.p_o = self.p_norm = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, d, vd = self.heads, self.dim, self.vdim
        decls = {"q": ParamDecl((H * d, self.hidden)), "k": ParamDecl((H * d, self.hidden)),
                 "v": ParamDecl((H * vd, self.hidden)), "o": ParamDecl((self.hidden, H * vd)),
                 "norm": ParamDecl((H * vd,), role="vector", init="one_plus_normal", std=0.1)}
        if self.has_gate:
            decls["g"] = ParamDecl((H * vd, self.hidden))
        return decls

    def bind(self, t: Dict[str, torch.Tensor]) -> None:
        self.p_in = torch.cat([t["q"], t["k"], t["v"]] + ([t["g"]] if self.has_gate else [])).contiguous()
        self.p_o, self.p_norm = t["o"], t["norm"]

    # ---- the projected protocol (parts/pair.py)
    def in_rows(self) -> int:
        return 2 * self.heads * self.dim + (2 if self.has_gate else 1) * self.heads * self.vdim

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def in_weight(self):
        return self.p_in

    def out_weight(self):
        return self.p_o

    def release_projections(self) -> None:
        self.p_in = self.p_o = None

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed(self.heads * self.dim * self.vdim)

    def planner(self):
        return RecurrenceChunks()

    def forward_projected(self, proj, ctx, entry, out, out_scale: float = 1.0) -> None:
        k = self.build.kernels
        state = ctx.state_of(entry, self.state_need().numel)
        plan = ctx.plan(RecurrenceChunks.plan_key)
        chunks = None
        if plan.facts["n_chunks"] and k.linear_attention_chunks_supports(self.dim, self.vdim):
            chunks = (plan.dev["chunk_seq"], plan.dev["chunk_q0"], plan.dev["seq_chunk0"], plan.facts["n_chunks"])
        o = k.linear_attention(proj, state, ctx.dev["slots"], ctx.batch_c[0], self.decay, self.heads, self.dim, self.vdim,
                               self.activation, chunks, single_tokens=ctx.is_decode)
        n = self.out_columns()
        gate = proj[:, self.in_rows() - n:] if self.has_gate else None
        k.norm_gate(o, self.p_norm, gate, self.eps, proj.dtype, out_scale, out=out)

    def forward(self, x, ctx, entry):
        k = self.build.kernels
        proj = linear(k, x, self.p_in)
        heads = torch.empty((x.shape[0], self.out_columns()), dtype=x.dtype, device=x.device)
        self.forward_projected(proj, ctx, entry, heads)
        return linear(k, heads, self.p_o)
