"""Small Nerenex configurations and random weights of the tests' own making (no code of the package is used to draw
or name a tensor): config.json contents, a tensor dictionary by checkpoint name, and a folder writer."""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import save_file


def attention(heads=3, dim=8, rot_dim=4, vdim=6, q_rank=20, kv_rank=12, scale=0.3, window=7, base=100.0, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, vocab=61, width=24, mult=0.8, eps=2e-5, buckets=53, mul_prev=31, mul_cur=7):
    return {"architecture": "Nerenex", "vocab": vocab, "width": width, "residual_mult": mult, "norm": {"eps": eps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers}


# Sizes that differ wherever a model could happen to make them equal: per-head sizes, ranks, windows per layer, a
# rotation over part of the rotated dimensions, a recurrence wider than the model, one block and several, one tap
# and several, layers with and without a feed-forward, in both orders.
CONFIGS = {
    "attn_only": config([layer("latent_attention", attention(), None)]),
    "rec_only": config([layer("rglru", {"width": 40, "blocks": 5, "conv": 3}, None)]),
    "attn_ff": config([layer("latent_attention", attention(heads=1, window=None), 36)], width=16, vocab=47),
    "mixed": config([
        layer("rglru", {"width": 32, "blocks": 1, "conv": 1}, 28),
        layer("latent_attention", attention(heads=5, dim=6, rot_dim=10, vdim=4, q_rank=9, kv_rank=21, scale=0.21, window=19,
                                            base=5000.0, rot_dims=6), None),
        layer("latent_attention", attention(heads=2, dim=16, rot_dim=2, vdim=24, q_rank=40, kv_rank=33, scale=0.4, window=4), 50),
        layer("rglru", {"width": 48, "blocks": 3, "conv": 5}, None),
        layer("latent_attention", attention(window=33), 31),
    ], vocab=131, width=40, mult=0.45, eps=3e-6, buckets=97, mul_prev=1000003, mul_cur=911),
    # sizes in the multiples the tensor-core products take (rows of 8 and more elements, 16-byte aligned)
    "wide": config([
        layer("latent_attention", attention(heads=4, dim=32, rot_dim=16, vdim=48, q_rank=96, kv_rank=64, scale=0.1, window=40,
                                            base=10000.0), 320),
        layer("rglru", {"width": 192, "blocks": 2, "conv": 4}, 256),
    ], vocab=512, width=128, buckets=509),
}


def tensors(cfg, seed=0, dtype=torch.float32, std=0.35):
    """Checkpoint name -> tensor.  Matrices N(0, std / sqrt(fan-in) * something that keeps activations of order one);
    norm offsets and biases small; the recurrence's decay parameter negative enough for a memory of several tokens."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0):
        return torch.randn(*shape, generator=g) * s

    w = cfg["width"]
    out = {"embed": rnd(cfg["vocab"], w), "bigram": rnd(cfg["embedding"]["bigram"]["buckets"] + 1, w, s=0.5),
           "final.norm": rnd(w, s=0.1)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out[p + "norm1"] = rnd(w, s=0.1)
        out[p + "rg1"] = rnd(w, w, s=std / w ** 0.5 * 2)
        out[p + "rg1.b"] = rnd(w, s=0.3)
        if lay["type"] == "latent_attention":
            h, qk = m["heads"], m["dim"] + m["rot_dim"]
            out[p + "mix.dq"] = rnd(m["q_rank"], w, s=std / w ** 0.5)
            out[p + "mix.dq.norm"] = 1 + rnd(m["q_rank"], s=0.1)
            out[p + "mix.uq"] = rnd(h * qk, m["q_rank"], s=3 * std / m["q_rank"] ** 0.5)
            out[p + "mix.dkv"] = rnd(m["kv_rank"] + m["rot_dim"], w, s=std / w ** 0.5)
            out[p + "mix.dkv.norm"] = 1 + rnd(m["kv_rank"], s=0.1)
            out[p + "mix.uk"] = rnd(h * m["dim"], m["kv_rank"], s=3 * std / m["kv_rank"] ** 0.5)
            out[p + "mix.uv"] = rnd(h * m["vdim"], m["kv_rank"], s=std / m["kv_rank"] ** 0.5)
            out[p + "mix.g"] = rnd(h, w, s=std / w ** 0.5 * 2)
            out[p + "mix.o"] = rnd(w, h * m["vdim"], s=std)
        else:
            cw, nb = m["width"], m["blocks"]
            bw = cw // nb
            out[p + "mix.y"] = rnd(cw, w, s=std / w ** 0.5)
            out[p + "mix.y.b"] = rnd(cw, s=0.2)
            out[p + "mix.x"] = rnd(cw, w, s=std / w ** 0.5)
            out[p + "mix.x.b"] = rnd(cw, s=0.2)
            out[p + "mix.conv"] = rnd(cw, m["conv"], s=0.6)
            out[p + "mix.conv.b"] = rnd(cw, s=0.2)
            out[p + "mix.ra"] = rnd(nb, bw, bw, s=1.0 / bw ** 0.5)
            out[p + "mix.ra.b"] = rnd(nb, bw, s=0.5)
            out[p + "mix.ri"] = rnd(nb, bw, bw, s=1.0 / bw ** 0.5)
            out[p + "mix.ri.b"] = rnd(nb, bw, s=0.5)
            out[p + "mix.lam"] = rnd(cw, s=1.0) - 3.0
            out[p + "mix.o"] = rnd(w, cw, s=std)
        if lay["mlp"] is not None:
            ff = lay["mlp"]["ff"]
            out[p + "norm2"] = rnd(w, s=0.1)
            out[p + "rg2"] = rnd(w, w, s=std / w ** 0.5 * 2)
            out[p + "rg2.b"] = rnd(w, s=0.3)
            out[p + "mlp.up"] = rnd(ff, w, s=2 * std / w ** 0.5)
            out[p + "mlp.down"] = rnd(w, ff, s=std)
            out[p + "mlp.act"] = rnd(2, s=0.5)
    return {k: v.to(dtype).contiguous() for k, v in out.items()}


def write_folder(folder, cfg, weights) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder


def as_double(weights):
    return {k: v.double() for k, v in weights.items()}
