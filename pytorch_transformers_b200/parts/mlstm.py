"""The matrix memory with exponential gates (mLSTM of xLSTM) as a mixer.

With ``h`` the mixer's input, per head (``dim`` entries of queries and keys, ``vdim`` of values):

    q = W_q h / sqrt(dim),  k = W_k h,  v = W_v h
    i = cap tanh((W_i h + b_i) / cap),   f = logsigmoid(cap tanh((W_f h + b_f) / cap))        the gates' logarithms
    m_t = max(f_t + m_(t-1), i_t)                                         m, S, n are 0 before the first token
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,    n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
    out = W_o ( rmsnorm per head (o) * gain * sigmoid(W_g h) )

Prompts of 256 tokens or more run in chunks of 64 on the tensor cores where the kernel takes the sizes (a chunk's own
sum, the chunks joined in order, the outputs); shorter steps and decoding run token by token. Both carry the same
running maximum m. Per sequence the mixer keeps S, n and m in the cache's state area (float32) and needs no pages. The gates'
projections are a product of their own whose float32 sums stay unrounded; biases, cap, logarithms, decays, state,
the division and the heads' norm are float32 whatever the model dtype. q, k, v and the output gate are one product.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import BuildContext, ParamDecl, Part, PartSpec, StateNeed, register_part
from .linear import linear, linear_pending
from .recurrent import SCAN_CHUNK, RecurrenceChunks


@register_part("mixer", "mlstm")
class MatrixMemory(Part):
    graph_safe = True
    fuses_add = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, heads: int, dim: int, vdim: int, gate_cap: float = 0.0,
                 eps: float = 1e-6, gate: bool = True):
        super().__init__(build, spec)
        self.hidden, self.heads, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.gate_cap, self.eps, self.has_gate = float(gate_cap), float(eps), bool(gate)
        if not (0 < self.dim <= build.kernels.MLSTM_MAX_DIM):
            raise ValueError(f"the matrix memory's kernel takes keys of 1 to {build.kernels.MLSTM_MAX_DIM} entries, got {dim}")
        if SCAN_CHUNK != build.kernels.MLSTM_CHUNK:
            raise ValueError("the chunk planner and the chunked kernel disagree on the chunk's size")
        self.p_in = self.p_gates = self.p_i_b = self.p_f_b = self.p_norm = self.p_o = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, d, vd = self.heads, self.dim, self.vdim
        decls = {"q": ParamDecl((H * d, self.hidden)), "k": ParamDecl((H * d, self.hidden)),
                 "v": ParamDecl((H * vd, self.hidden)), "o": ParamDecl((self.hidden, H * vd)),
                 "norm": ParamDecl((H * vd,), role="vector", init="one_plus_normal", std=0.1),
                 "i": ParamDecl((H, self.hidden), std=0.1), "i_b": ParamDecl((H,), role="vector", std=1.0),
                 "f": ParamDecl((H, self.hidden), std=0.1), "f_b": ParamDecl((H,), role="vector", init="one_plus_normal", std=1.0)}
        if self.has_gate:
            decls["g"] = ParamDecl((H * vd, self.hidden))
        return decls

    def bind(self, t: Dict[str, torch.Tensor]) -> None:
        self.p_in = torch.cat([t["q"], t["k"], t["v"]] + ([t["g"]] if self.has_gate else [])).contiguous()
        self.p_gates = torch.cat([t["i"], t["f"]]).contiguous()
        self.p_i_b, self.p_f_b, self.p_norm, self.p_o = t["i_b"], t["f_b"], t["norm"], t["o"]

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed(self.build.kernels.mlstm_state_floats(self.heads, self.dim, self.vdim))

    def planner(self):
        return RecurrenceChunks()

    def runs_beside(self, ctx) -> bool:
        return False

    def forward(self, x, ctx, entry, add=None):
        return linear(self.build.kernels, self._heads(x, ctx, entry), self.p_o, add=add)

    def forward_pending(self, x, ctx, entry):
        """The mixer's result as the last product's float32 sums, for a kernel that adds them to the stream later."""
        return linear_pending(self.build.kernels, self._heads(x, ctx, entry), self.p_o)

    def _heads(self, x, ctx, entry):
        k = self.build.kernels
        H, d, vd = self.heads, self.dim, self.vdim
        proj = linear(k, x, self.p_in)
        gates = linear(k, x, self.p_gates, wide_out=True)
        state = ctx.state_of(entry, self.state_need().numel)
        plan, chunks = ctx.plan(RecurrenceChunks.plan_key), None
        if plan.facts["n_chunks"] and k.mlstm_chunks_takes(proj, d, vd):
            # a long prompt in bfloat16 with sizes of the tensor-core kernels: chunks of 64 tokens in three passes
            chunks = (plan.dev["chunk_seq"], plan.dev["chunk_q0"], plan.dev["seq_chunk0"], plan.facts["n_chunks"])
        o = k.mlstm(proj, gates, self.p_i_b, self.p_f_b, self.gate_cap, state, ctx.dev["slots"], ctx.batch_c[0], H, d, vd,
                    d ** -0.5, chunks)
        gate = proj[:, 2 * H * d + H * vd:] if self.has_gate else None
        return k.head_norm_gate(o, self.p_norm, gate, H, self.eps, proj.dtype)
