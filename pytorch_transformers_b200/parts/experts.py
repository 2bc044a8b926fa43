"""The routed feed-forward: a mixture of small gated feed-forward experts with a group-limited router.

Router, per token and in float32: ``s = softmax(W_r h)`` over all ``experts + identity`` outputs;
choice scores ``s + correction``; the outputs form ``groups`` equal groups of neighbours, a group's score
is its largest choice score and only the ``keep`` best groups stay eligible; the ``top`` largest eligible
choice scores are chosen; a chosen output weighs ``s * scale`` (no renormalisation). Expert e computes
``W_down (silu(W_gate h) * (W_up h))``; the last ``identity`` outputs are identity experts that pass
``h`` on and have no tensors. The result is the weighted sum over the chosen, added to the residual
stream in float32 in the same kernel.

Variants, all by constructor parameters: ``score="sigmoid"`` scores every output by a sigmoid of its own
instead of the softmax; ``correction=False`` has no correction tensor; ``expert="plain"`` experts have no
gate, ``W_down act(W_up h)`` with ``activation`` by name; ``weight_on="input"`` multiplies the expert's
input by the weight instead of its output: the result is the sum of ``expert(weight * h)``.
``group_score="top2_sum"`` scores a group by the sum of its two largest choice scores instead of its largest.
``normalize=True`` divides the chosen outputs' scores by their sum (+ 1e-20) before ``scale``. A ``shared`` child (a
feed-forward part that returns float32 sums) is an expert that every token uses; its result is added in the kernel
that sums the chosen experts, and with ``shared_gate=True`` it is multiplied by ``sigmoid(w_sg . h)``, one number per
token whose row ``shared_gate`` [1, hidden] is held with the router's matrix and multiplied with it (float32).
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import BuildContext, ParamDecl, Part, PartSpec, register_part


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    graph_safe = True
    fuses_add = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, inner: int, experts: int, top: int,
                 identity: int = 0, groups: int = 1, keep: int = 1, scale: float = 1.0, score: str = "softmax",
                 correction: bool = True, expert: str = "gated_silu", activation: str = "gelu",
                 weight_on: str = "output", group_score: str = "max", normalize: bool = False, shared_gate: bool = False):
        super().__init__(build, spec)
        if group_score not in ("max", "top2_sum"):
            raise ValueError(f"a group's score is 'max' or 'top2_sum', got {group_score!r}")
        self.group_score, self.normalize = group_score, bool(normalize)
        self.shared = self.children.get("shared")
        self.has_shared_gate = bool(shared_gate)
        if self.has_shared_gate and self.shared is None:
            raise ValueError("shared_gate needs a shared expert (a child part 'shared')")
        if score not in build.kernels.ROUTE_SCORES:
            raise ValueError(f"router scores are one of {', '.join(build.kernels.ROUTE_SCORES)}, got {score!r}")
        if expert not in ("gated_silu", "plain") or weight_on not in ("output", "input"):
            raise ValueError(f"experts are 'gated_silu' or 'plain' and weigh their 'output' or 'input', got {expert!r}, {weight_on!r}")
        if (expert == "plain") != (weight_on == "input"):
            # the grouped kernels take the weight in the plain expert's first epilogue, or in the sum of outputs
            raise ValueError("plain experts weigh their input and gated experts their output")
        if expert == "plain" and (activation not in build.kernels.ACTIVATIONS or identity):
            raise ValueError(f"plain experts take an activation of {', '.join(build.kernels.ACTIVATIONS)} and no identity experts")
        self.score, self.has_correction, self.expert, self.activation = score, bool(correction), expert, activation
        self.hidden, self.inner, self.experts, self.top = int(hidden), int(inner), int(experts), int(top)
        self.identity, self.groups, self.keep, self.scale = int(identity), int(groups), int(keep), float(scale)
        n = self.experts + self.identity
        if self.experts <= 0 or self.identity < 0 or self.groups <= 0 or n % self.groups:
            raise ValueError(f"{n} router outputs do not form {self.groups} equal groups")
        if not (0 < self.keep <= self.groups) or not (0 < self.top <= n // self.groups * self.keep):
            raise ValueError(f"cannot choose {self.top} of {n} outputs in {self.keep} of {self.groups} groups")
        if n > 512:
            raise ValueError(f"the router kernel takes up to 512 outputs, got {n}")
        self.p_router = self.p_correction = self.p_gate_up = self.p_down = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        n = self.experts + self.identity
        d = {"router": ParamDecl((n, self.hidden), role="vector")}
        if self.has_correction:
            d["correction"] = ParamDecl((n,), role="vector")
        if self.has_shared_gate:
            d["shared_gate"] = ParamDecl((1, self.hidden), role="vector")
        for e in range(self.experts):
            if self.expert == "gated_silu":
                d[f"e{e}.gate"] = ParamDecl((self.inner, self.hidden))
            d[f"e{e}.up"] = ParamDecl((self.inner, self.hidden))
            d[f"e{e}.down"] = ParamDecl((self.hidden, self.inner))
        return d

    def bind(self, t: Dict[str, torch.Tensor]) -> None:
        self.p_router, self.p_correction = t["router"].contiguous(), t.get("correction")
        if self.has_shared_gate:        # one more row of the router's product: the shared expert's gate
            self.p_router = torch.cat([self.p_router, t["shared_gate"].reshape(1, self.hidden)]).contiguous()
        E, F = self.experts, self.inner
        if self.expert == "plain":      # [E, F, hidden] and [E, hidden, F]
            self.p_gate_up = torch.stack([t.pop(f"e{e}.up") for e in range(E)]).contiguous()
            self.p_down = torch.stack([t.pop(f"e{e}.down") for e in range(E)]).contiguous()
            return
        # all experts in two tensors for the grouped products: [E, 2 F, hidden] (gate rows, then up rows), [E, hidden, F]
        gate_up = torch.empty((E, 2 * F, self.hidden), dtype=t["e0.gate"].dtype, device=t["e0.gate"].device)
        down = torch.empty((E, self.hidden, F), dtype=gate_up.dtype, device=gate_up.device)
        for e in range(E):
            gate_up[e, :F] = t.pop(f"e{e}.gate")
            gate_up[e, F:] = t.pop(f"e{e}.up")
            down[e] = t.pop(f"e{e}.down")
        self.p_gate_up, self.p_down = gate_up, down

    def forward(self, x, ctx, add=None):
        k = self.build.kernels
        if callable(add):
            add = add()
        routed = k.route(x, self.p_router, self.p_correction, self.groups, self.keep, self.top, self.scale, self.score,
                         extra=1 if self.has_shared_gate else 0, group_top=2 if self.group_score == "top2_sum" else 1,
                         normalize=self.normalize)
        ids, weights = routed[0], routed[1]
        shared = shared_gate = None
        if self.shared is not None:
            shared = self.shared.forward(x, ctx)        # float32 sums of the shared expert's last product
            if self.has_shared_gate:
                shared_gate = routed[2][:, self.experts + self.identity:]
        return k.routed_experts(x, ids, weights, self.p_gate_up, self.p_down, base=add,
                                plain_act=self.activation if self.expert == "plain" else None, shared=shared,
                                shared_gate=shared_gate)
