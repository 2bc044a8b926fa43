"""A plain, slow restatement of the Figudra design in float64, one function per mechanism, whole sequences at a
time, written from the design's equations. It shares no code with the package: the tests compare the two.

Notation: ``h`` [T, width] is a sublayer's input (the layer's normed stream), ``p`` a position (from 0), weights are
stored [out, in] and applied as ``W h``. A model is (config dict as in config.json, dict of tensors by name).
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def kv_head_of(h: int, heads: int, kv_heads: int) -> int:
    return h // (heads // kv_heads)


# ---------------------------------------------------------------------------------------------- gated linear attention
def gla_decay(h, w: Dict[str, torch.Tensor], heads: int, dim: int, tau: float):
    """alpha [T, heads, dim] = sigmoid(W_a2 (W_a1 h) + b) ** (1 / tau)."""
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    return torch.sigmoid(z).pow(1.0 / tau).reshape(-1, heads, dim)


def gla_recurrence(q, k, v, alpha, state=None):
    """Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t. q, k, alpha [T, H, d]; v [T, H, dv].
    Returns (o [T, H, dv], the state after the last token [H, d, dv])."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def gla_mixer(h, w, m, eps: float, state=None, return_state=False):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).reshape(T, H, d)
    v = (h @ w["v"].T).reshape(T, H, dv)
    o, S = gla_recurrence(q, k, v, gla_decay(h, w, H, d, float(m["tau"])), state)
    o = rms_norm(o, w["norm"], eps).reshape(T, H * dv)
    y = (o * silu(h @ w["g"].T)) @ w["o"].T
    return (y, S) if return_state else y


# ---------------------------------------------------------------------------------------------- attentions
def query_temperature(p: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef ln(floor((p + 1) / every) + 1) for integer positions p."""
    return 1.0 + coef * torch.log(torch.div(p + 1, every, rounding_mode="floor").to(F64) + 1.0)


def capped_attention(h, w, m, first_pos: int = 0):
    """The mixer 'attention': no rotation, query temperature, soft-capped scores, causal, ordinary softmax, a
    sigmoid gate on the concatenated heads."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(first_pos, first_pos + T)
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    v = (h @ w["v"].T).reshape(T, G, dv)
    temp = m.get("q_temp")
    if temp:
        q = q * query_temperature(pos, float(temp["coef"]), int(temp["every"]))[:, None, None]
    cap = float(m.get("softcap") or 0.0)
    visible = pos[None, :] <= pos[:, None]
    out = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        g = kv_head_of(hh, H, G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~visible, -math.inf)
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def rotate(x, pos, dims: int, base: float, factor: float):
    """Rotary positions on the first ``dims`` entries of each head (x [T, heads, d]); entry i pairs with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=F64) / dims) / factor
    a = pos.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def window_visible(T: int, size: int, keep_first: int, first_pos: int = 0) -> torch.Tensor:
    """visible[i, j]: j <= i and (i - j < size or j < keep_first)."""
    pos = torch.arange(first_pos, first_pos + T)
    i, j = pos[:, None], pos[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def windowed_attention(h, w, m, eps: float):
    """The mixer 'attention_2': per-head RMS norm of q and k with gains, then rotary positions with linear scaling on
    part of a head, a sliding window that keeps the first tokens, a softmax with one added to its denominator."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = rms_norm((h @ w["q"].T).reshape(T, H, d), w["q.norm"], eps)
    k = rms_norm((h @ w["k"].T).reshape(T, G, d), w["k.norm"], eps)
    v = (h @ w["v"].T).reshape(T, G, dv)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if dims:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q, k = rotate(q, pos, dims, float(rot["base"]), factor), rotate(k, pos, dims, float(rot["base"]), factor)
    mask = m.get("mask") or {}
    size = int(mask.get("size", 0))
    visible = window_visible(T, size, int(mask.get("keep_first", 0))) if size > 0 else window_visible(T, T + 1, 0)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        g = kv_head_of(hh, H, G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        e = torch.exp(s).masked_fill(~visible, 0.0)        # small test scores: no maximum is taken off
        out[:, hh] = (e / (1.0 + e.sum(-1, keepdim=True))) @ v[:, g]
    return out.reshape(T, H * dv) @ w["o"].T


# ---------------------------------------------------------------------------------------------- feed-forwards
def gated_ff(h, gate, up, down, act):
    return (act(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, w_router, r: dict):
    """(ids [T, top], weights [T, top]) of the group-limited sigmoid router."""
    n, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    s = torch.sigmoid(h @ w_router.T)                            # [T, n]
    T = s.shape[0]
    per = n // count
    grouped = s.reshape(T, count, per)
    gscore = grouped.topk(min(2, per), -1).values.sum(-1)        # sum of a group's two largest
    best = gscore.topk(keep, -1).indices
    open_ = torch.zeros(T, count, dtype=torch.bool).scatter_(1, best, True)
    masked = grouped.masked_fill(~open_[:, :, None], -math.inf).reshape(T, n)
    ids = masked.topk(top, -1).indices
    chosen = s.gather(1, ids)
    return ids, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))


def moe_ff(h, w, mlp: dict):
    r = mlp["router"]
    ids, weights = route(h, w["router"], r)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), weights[t]):
            out[t] += g * gated_ff(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], silu)[0]
    if mlp.get("shared"):
        shared = gated_ff(h, w["shared.gate"], w["shared.up"], w["shared.down"], silu)
        out = out + shared * torch.sigmoid(h @ w["shared.sg"].T)
    return out


def feed_forward(h, w, mlp: dict):
    if mlp["kind"] == "dense":
        return gated_ff(h, w["gate"], w["up"], w["down"], gelu_tanh)
    return moe_ff(h, w, mlp)


# ---------------------------------------------------------------------------------------------- the model
def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], streams: list = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence fed whole; ``streams`` (a list) receives the stream after every layer."""
    eps = float(config["norm"]["eps"])
    x = rms_norm(weights["embed"].to(F64)[torch.tensor(tokens)], weights["embed.norm"].to(F64), eps)
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        h = rms_norm(x, weights[f"l{src}.norm1"].to(F64), eps)
        mw, m = sub(weights, f"l{src}.mix."), layer["mixer"]
        if layer["type"] == "gla":
            y = gla_mixer(h, mw, m, eps)
        elif layer["type"] == "attention":
            y = capped_attention(h, mw, m)
        elif layer["type"] == "attention_2":
            y = windowed_attention(h, mw, m, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, sub(weights, f"l{src}.mlp."), layer["mlp"])
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, weights["final.norm"].to(F64), eps) @ weights["head"].to(F64).T
