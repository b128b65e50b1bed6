"""A plain, slow restatement of the Nerenex decoder in torch on the host, one function per mechanism.

Nothing here is shared with the engine: the tests compare the engine's kernels, cache and scheduler with these
functions.  Every function works on one whole sequence (no cache, no batching) in the dtype of its inputs (the
tests use float64 or float32).  ``cfg`` is the parsed config.json, ``w`` maps checkpoint tensor names to tensors.

Notation: h is a [T, width] block of sublayer inputs, positions count from 0.
"""

from __future__ import annotations

import math

import torch


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def zero_centred_norm(x, gain, eps):
    """RMS norm whose stored gain is an offset from one."""
    return rms(x, eps) * (1.0 + gain)


def plain_norm(x, gain, eps):
    return rms(x, eps) * gain


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def xielu(z, p, q):
    """Quadratic above zero, exponential below: slopes meet at z/2 on both sides."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    pos = ap * z * z + 0.5 * z
    neg = aq * (torch.expm1(torch.clamp(z, max=0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def embed_tokens(tokens, table, bigram, mul_prev, mul_cur, buckets):
    """Token row plus a hashed row for (previous token, token); the first token uses the table's last row."""
    rows = []
    for t, tok in enumerate(tokens):
        idx = buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets
        rows.append(table[tok] + bigram[idx])
    return torch.stack(rows)


def rotate_interleaved(x, positions, dims, base):
    """x [T, ..., D]: pairs (2i, 2i+1), i < dims/2, turned by positions * base^(-2i/dims); the rest unchanged."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cs, sn = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cs - v * sn
    out[..., 1:dims:2] = v * cs + u * sn
    return out


def latent_attention(h, w, pre, mx, eps):
    """Queries and keys/values through low-rank latents, one shared rotated key part, a sliding window, a gate per head."""
    T = h.shape[0]
    H, dn, dr, dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    pos = torch.arange(T)
    cq = plain_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
    q = (cq @ w[pre + "uq"].T).view(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], q[..., dn:]
    ckv = h @ w[pre + "dkv"].T
    c = plain_norm(ckv[:, :rank], w[pre + "dkv.norm"], eps)
    k_rot = ckv[:, rank:]
    rot = mx["rot"]
    q_rot = rotate_interleaved(q_rot, pos, rot["dims"], rot["base"])
    k_rot = rotate_interleaved(k_rot, pos, rot["dims"], rot["base"])
    k_plain = (c @ w[pre + "uk"].T).view(T, H, dn)
    v = (c @ w[pre + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_rot, k_rot)) * mx["scale"]
    diff = pos[:, None] - pos[None, :]
    seen = diff >= 0
    if mx.get("mask") is not None:
        seen = seen & (diff < mx["mask"]["size"])
    scores = scores.masked_fill(~seen[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shd->thd", probs, v)
    gate = torch.sigmoid(h @ w[pre + "g"].T)  # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, K] with the last column on the current token; zeros before the start."""
    T, C = x.shape
    K = taps_w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x])
    out = torch.zeros_like(x)
    for k in range(K):
        out = out + padded[k:k + T] * taps_w[:, k][None, :]
    return out + bias


def rglru(h, w, pre, mx):
    """Gated linear recurrence on a convolved branch, multiplied by a GELU branch."""
    T = h.shape[0]
    nb = mx["blocks"]
    y = gelu_tanh(h @ w[pre + "y"].T + w[pre + "y.b"])
    u = causal_conv(h @ w[pre + "x"].T + w[pre + "x.b"], w[pre + "conv"], w[pre + "conv.b"])
    ub = u.view(T, nb, -1)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[pre + "ra"]) + w[pre + "ra.b"]).reshape(T, -1)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[pre + "ri"]) + w[pre + "ri.b"]).reshape(T, -1)
    log_a = -8.0 * r * softplus(w[pre + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    s = torch.zeros_like(u[0])
    states = []
    for t in range(T):
        s = a[t] * s + drive[t]
        states.append(s)
    return (torch.stack(states) * y) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    act = w[pre + "act"]
    return xielu(h @ w[pre + "up"].T, act[0], act[1]) @ w[pre + "down"].T


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and, if asked, the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    m = cfg["residual_mult"]
    bg = cfg["embedding"]["bigram"]
    x = embed_tokens(list(tokens), w["embed"], w["bigram"], bg["mul_prev"], bg["mul_cur"], bg["buckets"])
    after = []
    for li, layer in enumerate(cfg["layers"]):
        p = f"l{li}."
        if layer["type"] == "latent_attention":
            y = latent_attention(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "rglru":
            y = rglru(x, w, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        y = y * torch.sigmoid(x @ w[p + "rg1"].T + w[p + "rg1.b"])
        x = x + m * zero_centred_norm(y, w[p + "norm1"], eps)
        if layer["mlp"] is not None:
            y = dense_ff(x, w, p + "mlp.")
            y = y * torch.sigmoid(x @ w[p + "rg2"].T + w[p + "rg2.b"])
            x = x + m * zero_centred_norm(y, w[p + "norm2"], eps)
        after.append(x)
    logits = zero_centred_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
