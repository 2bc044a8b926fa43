"""The Pogezen design restated from its equations: whole sequences, float64, one function per mechanism, no
code shared with the package. ``w`` maps tensor names to float64 tensors; ``cfg`` is the config.json dict.

    x0 = embed[token] * embedding.scale
    layer:  x <- x + mixer(h + conv(h)),  h = dyt1(x);    x <- x + W_down relu(W_up dyt2(x))^2   (if the layer has an mlp)
    logits = embed @ dyt_final(x)
"""
import math

import torch


def dyt(x, w, name):
    """tanh(alpha x) * weight + bias with a scalar alpha."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def input_conv(h, filt):
    """h_t + sum_j filt[:, j] h_(t - taps + 1 + j), zeros before the sequence."""
    T, taps = h.shape[0], filt.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += filt[:, j] * h[s]
    return out


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def log_gates(h, w, p, cap):
    """The logarithms of the input and forget gates, [T, heads] each."""
    i = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    return i, f


def matrix_memory(q, k, v, i, f):
    """q, k [T, H, d], v [T, H, vd], i, f [T, H] -> [T, H, vd]; S, n and the running maximum start at zero."""
    T, H, d = q.shape
    vd = v.shape[-1]
    S, n, m = q.new_zeros(H, d, vd), q.new_zeros(H, d), q.new_zeros(H)
    out = []
    for t in range(T):
        m_new = torch.maximum(f[t] + m, i[t])
        a, b = torch.exp(f[t] + m - m_new), torch.exp(i[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out.append(torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None])
    return torch.stack(out)


def mlstm(h, w, p, m, eps):
    H, d, vd, T = m["heads"], m["dim"], m["vdim"], h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, d) / math.sqrt(d)
    k, v = (h @ w[p + "k"].T).view(T, H, d), (h @ w[p + "v"].T).view(T, H, vd)
    i, f = log_gates(h, w, p, float(m["gate_cap"]))
    o = rms(matrix_memory(q, k, v, i, f), eps).reshape(T, H * vd)
    return (o * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def rotary_frequencies(rot):
    """(frequencies [dims / 2], the factor on cos and sin)."""
    dims, base = rot["dims"], float(rot["base"])
    idx = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * idx / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    where = lambda turns: dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
    lo, hi = max(math.floor(where(sc["fast"])), 0), min(math.ceil(where(sc["slow"])), dims - 1)
    ramp = ((idx - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / sc["factor"] * ramp + f * (1 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims entries of each head, entry i paired with i + dims / 2."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    f, mult = rotary_frequencies(rot)
    ang = positions.double()[:, None] * f
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    a, b = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def visible(T, size, keep_first):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    see = j <= i
    if size > 0:
        see = see & ((i - j < size) | (j < keep_first))
    return see


def attention(h, w, p, m, eps, shared):
    """``shared`` carries the first value-mixing layer's values to the later ones."""
    H, G, d, vd, T = m["heads"], m["kv_heads"], m["dim"], m["vdim"], h.shape[0]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, vd)
    q, k = rms(rotate(q, pos, m.get("rot")), eps), rms(rotate(k, pos, m.get("rot")), eps)
    if m.get("v_mix"):
        if "first" in shared:
            lam = w[p + "vmix"]
            v = (1 - lam) * v + lam * shared["first"]
        else:
            shared["first"] = v
    rep = H // G
    scores = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, 1)) * m["scale"]
    mask = m.get("mask") or {}
    scores = scores.masked_fill(~visible(T, int(mask.get("size", 0)), int(mask.get("keep_first", 0))), -math.inf)
    weights = torch.einsum("hg,gij->hij", w[p + "talk"], torch.softmax(scores, -1))
    o = torch.einsum("hij,jhv->ihv", weights, v.repeat_interleave(rep, 1)).reshape(T, H * vd)
    return o @ w[p + "o"].T + w[p + "o.b"]


def feed_forward(h, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def forward(cfg, w, ids, layers_out=None):
    """float64 logits [T, vocab] of one sequence; ``layers_out`` collects the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(ids)] * float(cfg["embedding"]["scale"])
    shared = {}
    for li, layer in enumerate(cfg["layers"]):
        p = f"l{li}."
        h = input_conv(dyt(x, w, p + "norm1"), w[p + "canon1"])
        if layer["type"] == "mlstm":
            x = x + mlstm(h, w, p + "mix.", layer["mixer"], eps)
        else:
            x = x + attention(h, w, p + "mix.", layer["mixer"], eps, shared)
        if layer.get("mlp") is not None:
            x = x + feed_forward(dyt(x, w, p + "norm2"), w, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return dyt(x, w, "final.norm") @ w["embed"].T
