"""Gated linear attention: a linear attention whose decay is computed from the mixer's input, per token and per key
channel.

With ``h`` the mixer's input, per head (``dim`` entries of queries and keys, ``vdim`` of values):

    q = W_q h / sqrt(dim),  k = W_k h,  v = W_v h
    a = sigmoid(W_a2 (W_a1 h) + b) ** (1 / tau)                 one decay per key channel, through a low rank
    S_t = diag(a_t) S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t,    S = 0 before the first token
    out = W_o ( rmsnorm per head (o) * gain * silu(W_g h) )      the gain [vdim] is shared by the heads

Per sequence the mixer keeps S [heads, dim, vdim] in the cache's state area (float32, zero when a sequence starts)
and needs no pages. The decay's second product keeps its float32 sums; bias, logsigmoid, the division by tau, the
state, the decays' exponentials and the heads' norm are float32 whatever the model dtype. q, k, v and the output gate
are one product. Prompts of 256 tokens or more run in chunks of 64 (a chunk's own sum, the chunks joined in order,
the outputs), shorter steps token by token; the two differ by float32 rounding. The low rank is the first size of
``W_a1``: given as ``rank``, or read from the checkpoint's tensor when ``rank`` is None.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import BuildContext, ParamDecl, Part, PartSpec, StateNeed, register_part
from .linear import linear, linear_pending
from .recurrent import SCAN_CHUNK, RecurrenceChunks


@register_part("mixer", "gla")
class GatedLinearAttention(Part):
    graph_safe = True
    fuses_add = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, heads: int, dim: int, vdim: int, tau: float,
                 eps: float = 1e-6, rank: Optional[int] = None, gate: bool = True):
        super().__init__(build, spec)
        self.hidden, self.heads, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.tau, self.eps, self.has_gate = float(tau), float(eps), bool(gate)
        self.rank = None if rank is None else int(rank)
        if not self.tau > 0:
            raise ValueError(f"gated linear attention: tau must be positive, got {tau}")
        if not (0 < self.dim <= build.kernels.GLA_MAX_DIM):
            raise ValueError(f"the gated linear attention's kernel takes keys of 1 to {build.kernels.GLA_MAX_DIM} entries, got {dim}")
        if SCAN_CHUNK != build.kernels.GLA_CHUNK:
            raise ValueError("the chunk planner and the chunked kernel disagree on the chunk's size")
        self.p_in = self.p_a1 = self.p_a2 = self.p_a2_b = self.p_norm = self.p_o = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, d, vd = self.heads, self.dim, self.vdim
        r = -1 if self.rank is None else self.rank        # -1: whatever the checkpoint's tensor has
        decls = {"q": ParamDecl((H * d, self.hidden)), "k": ParamDecl((H * d, self.hidden)),
                 "v": ParamDecl((H * vd, self.hidden)), "o": ParamDecl((self.hidden, H * vd)),
                 "norm": ParamDecl((vd,), role="vector", init="one_plus_normal", std=0.1),
                 "a1": ParamDecl((r, self.hidden), std=0.1), "a2": ParamDecl((H * d, r), std=1.0),
                 "a2_b": ParamDecl((H * d,), role="vector", init="one_plus_normal", std=2.0)}
        if self.has_gate:
            decls["g"] = ParamDecl((H * vd, self.hidden), std=0.1)
        return decls

    def bind(self, t: Dict[str, torch.Tensor]) -> None:
        if t["a1"].shape[0] != t["a2"].shape[1]:
            raise ValueError(f"gated linear attention: the decay's two matrices do not fit ({list(t['a1'].shape)}, {list(t['a2'].shape)})")
        self.p_in = torch.cat([t["q"], t["k"], t["v"]] + ([t["g"]] if self.has_gate else [])).contiguous()
        self.p_a1, self.p_a2, self.p_a2_b, self.p_o = t["a1"].contiguous(), t["a2"].contiguous(), t["a2_b"], t["o"]
        self.p_norm = t["norm"].repeat(self.heads).contiguous()      # the one gain vector, once per head

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed(self.heads * self.dim * self.vdim)

    def planner(self):
        return RecurrenceChunks()

    def forward(self, x, ctx, entry, add=None):
        return linear(self.build.kernels, self._heads(x, ctx, entry), self.p_o, add=add)

    def forward_pending(self, x, ctx, entry):
        """The mixer's result as the last product's float32 sums, for a kernel that adds them to the stream later."""
        return linear_pending(self.build.kernels, self._heads(x, ctx, entry), self.p_o)

    def _heads(self, x, ctx, entry):
        k = self.build.kernels
        H, d, vd = self.heads, self.dim, self.vdim
        proj = linear(k, x, self.p_in)
        log_decay = k.gla_decay_(linear(k, linear(k, x, self.p_a1), self.p_a2, wide_out=True), self.p_a2_b, self.tau)
        state = ctx.state_of(entry, self.state_need().numel)
        plan, chunks = ctx.plan(RecurrenceChunks.plan_key), None
        if plan.facts["n_chunks"]:
            chunks = (plan.dev["chunk_seq"], plan.dev["chunk_q0"], plan.dev["seq_chunk0"], plan.facts["n_chunks"])
        o = k.gla(proj, log_decay, state, ctx.dev["slots"], ctx.batch_c[0], H, d, vd, d ** -0.5, chunks)
        gate = proj[:, 2 * H * d + H * vd:] if self.has_gate else None
        return k.head_norm_gate(o, self.p_norm, gate, H, self.eps, proj.dtype, gate_act="silu")
