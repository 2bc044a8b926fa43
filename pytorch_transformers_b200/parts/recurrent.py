"""The gated linear recurrence mixer (a recurrent block with a real-gated linear recurrent unit).

With ``h`` the mixer's input and R channels in ``blocks`` equal parts:

    y = gelu_tanh(W_y h + b_y)                              the gate branch
    u = conv(W_x h + b_x)                                   causal, per channel, ``taps`` wide, zeros before the start
    r = sigmoid(A_r[b] u_b + c_r[b]),  i = sigmoid(A_i[b] u_b + c_i[b])      per part b (block-diagonal)
    log a = -decay * r * softplus(lam),  a = exp(log a)
    S_t = a S_(t-1) + sqrt(1 - a^2) * i * u,   S = 0 before the first token
    out = W_o (S * y)

Per sequence the mixer keeps S and the convolution's last ``taps - 1`` inputs in the cache's state
area (float32, zero when a sequence starts): ``StateNeed(R * taps)``; it needs no pages. Gates,
decay and state are float32 whatever the model dtype.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import BuildContext, ParamDecl, Part, PartSpec, StateNeed, register_part
from .linear import linear


SCAN_CHUNK = 64         # tokens of a chunk of the chunked scan
SCAN_CHUNKED_FROM = 256  # a step whose longest sequence brings this many tokens scans in chunks


class RecurrenceChunks:
    """The chunked scan's view of a step, as a planner: every sequence's new tokens cut into chunks of
    ``SCAN_CHUNK`` (sequence and first token of each chunk, and each sequence's first chunk). All recurrent
    layers of a model share the plan."""
    plan_key = "recurrence_chunks"

    def plan(self, ctx):
        from ..engine.batch import StepPlan
        if max(ctx.new) < SCAN_CHUNKED_FROM:
            return StepPlan(arrays={}, facts={"n_chunks": 0})
        seqs, firsts = ctx.tiles(SCAN_CHUNK)
        first_of, at = [], 0
        for n in ctx.new:
            first_of.append(at)
            at += (n + SCAN_CHUNK - 1) // SCAN_CHUNK
        return StepPlan(arrays={"chunk_seq": seqs, "chunk_q0": firsts, "seq_chunk0": first_of}, facts={"n_chunks": len(seqs)})


@register_part("mixer", "rglru")
class GatedLinearRecurrence(Part):
    graph_safe = True
    fuses_add = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, width: int, blocks: int, taps: int,
                 decay: float = 8.0):
        super().__init__(build, spec)
        self.hidden, self.width, self.blocks, self.taps, self.decay = int(hidden), int(width), int(blocks), int(taps), float(decay)
        if self.width <= 0 or self.blocks <= 0 or self.width % self.blocks:
            raise ValueError(f"the recurrence's width ({width}) must be a positive multiple of its blocks ({blocks})")
        if not (1 <= self.taps <= 8):
            raise ValueError(f"the convolution kernel takes 1 to 8 taps, got {taps}")
        self.p_yx = self.p_y_b = self.p_x_b = self.p_conv = self.p_conv_b = self.p_gates = self.p_gates_b = None
        self.p_lam = self.p_o = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        R, B, bw = self.width, self.blocks, self.width // self.blocks
        return {"y": ParamDecl((R, self.hidden)), "y_b": ParamDecl((R,), role="vector"),
                "x": ParamDecl((R, self.hidden)), "x_b": ParamDecl((R,), role="vector"),
                "conv": ParamDecl((R, self.taps), role="vector", std=0.3), "conv_b": ParamDecl((R,), role="vector"),
                "ra": ParamDecl((B, bw, bw)), "ra_b": ParamDecl((B, bw), role="vector"),
                "ri": ParamDecl((B, bw, bw)), "ri_b": ParamDecl((B, bw), role="vector"),
                "lam": ParamDecl((R,), role="vector", std=1.0), "o": ParamDecl((self.hidden, R))}

    def bind(self, t: Dict[str, torch.Tensor]) -> None:
        self.p_yx = torch.cat([t["y"], t["x"]])                  # both branches read the same input: one product
        self.p_y_b, self.p_x_b, self.p_conv, self.p_conv_b = t["y_b"], t["x_b"], t["conv"].contiguous(), t["conv_b"]
        self.p_gates = torch.cat([t["ra"], t["ri"]], dim=1).contiguous()      # [B, 2 bw, bw]: r rows, then i rows
        self.p_gates_b = torch.cat([t["ra_b"], t["ri_b"]], dim=1).contiguous()
        self.p_lam, self.p_o = t["lam"], t["o"]

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed(self.width * self.taps)

    def planner(self):
        return RecurrenceChunks()

    def runs_beside(self, ctx) -> bool:
        return False

    def forward(self, x, ctx, entry, add=None):
        k = self.build.kernels
        t, R, B = x.shape[0], self.width, self.blocks
        proj = linear(k, x, self.p_yx)
        state = ctx.state_of(entry, self.state_need().numel)
        slots, batch = ctx.dev["slots"], ctx.batch_c[0]
        y_act, u = k.rglru_conv(proj, self.p_y_b, self.p_x_b, self.p_conv, self.p_conv_b, state, slots, batch)
        gates = k.block_linear(u.view(t, B, R // B), self.p_gates, self.p_gates_b, act="sigmoid", out_dtype=torch.float32)
        chunks = ctx.plan(RecurrenceChunks.plan_key)
        if chunks.facts["n_chunks"]:       # long prompts: chunks side by side, joined in order
            out = k.rglru_scan_chunks(gates, u, y_act, self.p_lam, proj, self.p_x_b, state, slots, batch, B, self.taps,
                                      self.decay, chunks.dev["chunk_seq"], chunks.dev["chunk_q0"], chunks.dev["seq_chunk0"],
                                      chunks.facts["n_chunks"], SCAN_CHUNK)
        else:
            out = k.rglru_scan(gates, u, y_act, self.p_lam, proj, self.p_x_b, state, slots, batch, B, self.taps, self.decay)
        return linear(k, out, self.p_o, add=add)
