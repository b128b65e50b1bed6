"""A plain, slow implementation of the Gekopel decoder, one function per mechanism, written from the design's
equations in whatever precision the given tensors have (the tests use float64).  It shares no code with the engine:
no cache, no pages, no batching; a sequence is run whole, token by token where the design is a recurrence.

Notation: x is the stream [T, width]; weights are looked up in ``w`` by their checkpoint names (``l3.mix.q`` ...);
``cfg`` is the parsed config.json.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def embed(cfg, w, tokens, first_position: int = 0) -> torch.Tensor:
    ids = torch.as_tensor(tokens, dtype=torch.long)
    places = torch.arange(first_position, first_position + len(ids))
    return w["embed"][ids] * cfg["embedding"]["scale"] + w["pos"][places]


def distance_bucket(n: int, rows: int, reach: int) -> int:
    """Row of the distance-bias table for a key n tokens back: one row per distance below half the table, then rows
    spread evenly over the logarithm of the distance up to ``reach``, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))


def attention(m, w, pre, h: torch.Tensor) -> torch.Tensor:
    """Softmax attention with a learned distance bias, a chunk mask and a sink in the denominator."""
    t = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(t, heads, dim)
    k = (h @ w[pre + "k"].T).view(t, groups, dim)
    v = (h @ w[pre + "v"].T).view(t, groups, vdim)
    rel, sink = w[pre + "rel"], w[pre + "sink"]
    rows = rel.shape[0]
    chunk = m["mask"]["size"] if m.get("mask") else None
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for i in range(t):
        first = 0 if chunk is None else (i // chunk) * chunk
        keys = list(range(first, i + 1))
        rows_of = torch.tensor([distance_bucket(i - j, rows, m["bias_max"]) for j in keys])
        for a in range(heads):
            g = a // (heads // groups)
            s = (k[keys, g] @ q[i, a]) * m["scale"] + rel[rows_of, a]
            top = torch.maximum(s.max(), sink[a])
            e = torch.exp(s - top)
            out[i, a] = (e[:, None] * v[keys, g]).sum(0) / (e.sum() + torch.exp(sink[a] - top))
    return out.reshape(t, heads * vdim) @ w[pre + "o"].T


def short_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Per channel: y_t = sum_k taps[c, k] x_(t - K + 1 + k), zeros before the start."""
    t, k = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, x.shape[1], dtype=x.dtype), x], 0)
    return sum(padded[j:j + t] * taps[:, j] for j in range(k))


def delta_rule(q, k, v, beta, decay):
    """Per head, token by token: S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    q, k [T, heads, dim]; v [T, heads, vdim]; beta, decay [T, heads]."""
    t, heads, dim = q.shape
    state = torch.zeros(heads, dim, v.shape[2], dtype=q.dtype)
    out = torch.zeros_like(v)
    for i in range(t):
        state = state * decay[i, :, None, None]
        u = beta[i, :, None] * (v[i] - torch.einsum("hdv,hd->hv", state, k[i]))
        state = state + torch.einsum("hd,hv->hdv", k[i], u)
        out[i] = torch.einsum("hdv,hd->hv", state, q[i])
    return out


def delta_mixer(m, w, pre, h: torch.Tensor, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(short_convolution(h @ w[pre + "q"].T, w[pre + "q.conv"])).view(t, groups, dim)
    k = silu(short_convolution(h @ w[pre + "k"].T, w[pre + "k.conv"])).view(t, groups, dim)
    v = silu(short_convolution(h @ w[pre + "v"].T, w[pre + "v.conv"])).view(t, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    share = heads // groups
    q, k = q.repeat_interleave(share, 1), k.repeat_interleave(share, 1)
    beta = torch.sigmoid(h @ w[pre + "b"].T)
    decay = torch.exp(-torch.exp(w[pre + "A_log"]) * torch.nn.functional.softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    o = delta_rule(q, k, v, beta, decay)
    o = rms(o, eps) * w[pre + "norm"] * silu(h @ w[pre + "g"].T).view(t, heads, vdim)
    return o.reshape(t, heads * vdim) @ w[pre + "o"].T


def expert(w, pre, h):
    return relu_squared(h @ w[pre + "up"].T) @ w[pre + "down"].T


def route(r, w, pre, h: torch.Tensor):
    """(chosen experts [T, top], their weights [T, top])."""
    s = torch.sigmoid(h @ w[pre + "router"].T)
    choice = s + w[pre + "correction"]
    experts, top = r["experts"], r["top"]
    count, keep = r["groups"]["count"], r["groups"]["keep"]
    per = experts // count
    grouped = choice.view(-1, count, per)
    group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    kept = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, kept, True)
    masked = torch.where(allowed[:, :, None].expand(-1, -1, per).reshape(-1, experts), choice,
                         torch.full_like(choice, -math.inf))
    chosen = masked.topk(top, dim=-1).indices
    weight = s.gather(1, chosen)
    weight = weight / (weight.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return chosen, weight


def feed_forward(mlp, w, pre, h: torch.Tensor) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return expert(w, pre, h)
    chosen, weight = route(mlp["router"], w, pre, h)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e, g in zip(chosen[i].tolist(), weight[i]):
            out[i] += g * expert(w, f"{pre}e{e}.", h[i:i + 1])[0]
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[pre + "shared.sg"].T) * expert(w, pre + "shared.", h)
    return out


def forward(cfg, w, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and, if asked, the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = embed(cfg, w, tokens)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = rms(x, eps) * w[pre + "norm1"]
        if layer["type"] == "attention":
            y = attention(layer["mixer"], w, pre + "mix.", h)
        elif layer["type"] == "delta":
            y = delta_mixer(layer["mixer"], w, pre + "mix.", h, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms(y, eps) * w[pre + "norm1b"]
        if layer.get("mlp") is not None:
            y = feed_forward(layer["mlp"], w, pre + "mlp.", rms(x, eps) * w[pre + "norm2"])
            x = x + rms(y, eps) * w[pre + "norm2b"]
        after.append(x)
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    return (logits, after) if return_layers else logits
