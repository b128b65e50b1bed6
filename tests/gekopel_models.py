"""Small Gekopel configurations and random weights of the tests' own making (no code of the package is used to draw or
name a tensor): config.json contents, a tensor dictionary by checkpoint name, and a folder writer."""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import save_file


def attention(heads=3, kv_heads=1, dim=8, vdim=6, scale=0.3, bias_max=24, chunk=13, rows=10):
    """``rows``: rows of the layer's distance-bias table; config.json does not carry it (the tensor's shape does)."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max, "_rows": rows}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def delta(heads=2, kv_heads=1, dim=8, vdim=12, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=10, groups=3, keep=2, scale=1.3, shared=7):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, vocab=61, width=24, eps=2e-5, scale=3.0, max_positions=400):
    return {"architecture": "Gekopel", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": eps},
            "embedding": {"scale": scale}, "layers": layers}


def for_file(cfg):
    """The configuration as config.json holds it (without the tests' own notes)."""
    out = json.loads(json.dumps(cfg))
    for lay in out["layers"]:
        lay["mixer"].pop("_rows", None)
    return out


# Sizes that differ wherever a model could happen to make them equal or 1: key and value sizes, query heads per
# key/value head, chunk sizes that are no multiple of a page, bias tables with an odd number of rows and a reach
# below and above the chunk, groups of one and of several experts, every group kept and not, with and without a
# shared expert, one tap and several, layers without a feed-forward, both mixers first and last.
CONFIGS = {
    "attn_only": config([layer("attention", attention(), None)]),
    "delta_only": config([layer("delta", delta(), None)]),
    "moe_only": config([layer("delta", delta(heads=1, kv_heads=1, dim=4, vdim=4, conv=1), moe())], width=16, vocab=47),
    "mixed": config([
        layer("delta", delta(heads=4, kv_heads=2, dim=6, vdim=10, conv=4), dense(28)),
        layer("attention", attention(heads=4, kv_heads=2, dim=6, vdim=10, scale=0.21, bias_max=50, chunk=37, rows=11),
              moe(experts=8, top=3, ff=12, groups=4, keep=3, scale=0.7, shared=None)),
        layer("delta", delta(heads=3, kv_heads=3, dim=16, vdim=5, conv=2), moe(experts=4, top=4, ff=9, groups=1, keep=1, shared=20)),
        layer("attention", attention(heads=2, kv_heads=2, dim=16, vdim=24, scale=0.4, bias_max=9, chunk=None, rows=6), dense(50)),
        layer("attention", attention(heads=5, kv_heads=1, dim=4, vdim=3, scale=0.5, bias_max=300, chunk=64, rows=32), None),
        layer("delta", delta(heads=2, kv_heads=1, dim=33, vdim=7, conv=5), moe(experts=5, top=1, ff=6, groups=5, keep=2, shared=3)),
    ], vocab=131, width=40, eps=3e-6, scale=5.5),
    # nothing routed: every bfloat16 row can be held to the oracle (no token that rounding could send to another expert)
    "dense": config([
        layer("attention", attention(heads=6, kv_heads=3, dim=5, vdim=9, scale=0.35, bias_max=40, chunk=29, rows=9), dense(40)),
        layer("delta", delta(heads=4, kv_heads=1, dim=12, vdim=6, conv=3), None),
        layer("attention", attention(heads=2, kv_heads=1, dim=24, vdim=8, scale=0.2, bias_max=16, chunk=None, rows=7), dense(33)),
        layer("delta", delta(heads=2, kv_heads=2, dim=10, vdim=20, conv=4), dense(64)),
    ], vocab=97, width=48, eps=1e-5, scale=2.0),
    # sizes in the multiples the tensor-core products take (rows of 8 and more elements, 16-byte aligned)
    "wide": config([
        layer("delta", delta(heads=4, kv_heads=2, dim=32, vdim=48, conv=4), moe(experts=8, top=2, ff=64, groups=2, keep=1, shared=96)),
        layer("attention", attention(heads=4, kv_heads=2, dim=32, vdim=64, scale=0.15, bias_max=128, chunk=48, rows=16), dense(320)),
    ], vocab=512, width=128),
}


def tensors(cfg, seed=0, dtype=torch.float32, std=0.5):
    """Checkpoint name -> tensor.  Matrices scaled so that activations stay of order one; norm gains around one; decay
    parameters that give a memory of several tokens; router corrections large enough to change choices."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0):
        return torch.randn(*shape, generator=g) * s

    w = cfg["width"]
    out = {"embed": rnd(cfg["vocab"], w, s=0.3), "pos": rnd(cfg["max_positions"], w, s=0.5), "final.norm": 1 + rnd(w, s=0.1),
           "head": rnd(cfg["vocab"], w, s=1.0 / w ** 0.5)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        for n in ("norm1", "norm1b"):
            out[p + n] = 1 + rnd(w, s=0.1)
        if lay["type"] == "attention":
            h, kv = m["heads"], m["kv_heads"]
            out[p + "mix.q"] = rnd(h * m["dim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.k"] = rnd(kv * m["dim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.v"] = rnd(kv * m["vdim"], w, s=std / w ** 0.5)
            out[p + "mix.rel"] = rnd(m["_rows"], h, s=1.0)
            out[p + "mix.sink"] = rnd(h, s=1.0)
            out[p + "mix.o"] = rnd(w, h * m["vdim"], s=std)
        else:
            h, kv = m["heads"], m["kv_heads"]
            out[p + "mix.q"] = rnd(kv * m["dim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.q.conv"] = rnd(kv * m["dim"], m["conv"], s=0.6)
            out[p + "mix.k"] = rnd(kv * m["dim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.k.conv"] = rnd(kv * m["dim"], m["conv"], s=0.6)
            out[p + "mix.v"] = rnd(h * m["vdim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.v.conv"] = rnd(h * m["vdim"], m["conv"], s=0.6)
            out[p + "mix.b"] = rnd(h, w, s=2 * std / w ** 0.5)
            out[p + "mix.A_log"] = rnd(h, s=0.5) - 1.0
            out[p + "mix.norm"] = 1 + rnd(m["vdim"], s=0.1)
            out[p + "mix.a"] = rnd(h, w, s=2 * std / w ** 0.5)
            out[p + "mix.dt_bias"] = rnd(h, s=0.5) - 1.0
            out[p + "mix.g"] = rnd(h * m["vdim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.o"] = rnd(w, h * m["vdim"], s=std)
        mlp = lay["mlp"]
        if mlp is None:
            continue
        for n in ("norm2", "norm2b"):
            out[p + n] = 1 + rnd(w, s=0.1)
        if mlp["kind"] == "dense":
            out[p + "mlp.up"] = rnd(mlp["ff"], w, s=2 * std / w ** 0.5)
            out[p + "mlp.down"] = rnd(w, mlp["ff"], s=std)
        else:
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out[p + f"mlp.e{e}.up"] = rnd(ff, w, s=2 * std / w ** 0.5)
                out[p + f"mlp.e{e}.down"] = rnd(w, ff, s=std)
            out[p + "mlp.router"] = rnd(mlp["router"]["experts"], w, s=3 * std / w ** 0.5)
            out[p + "mlp.correction"] = rnd(mlp["router"]["experts"], s=0.3) - 0.5   # choice scores of both signs
            if mlp.get("shared") is not None:
                out[p + "mlp.shared.up"] = rnd(mlp["shared"]["ff"], w, s=2 * std / w ** 0.5)
                out[p + "mlp.shared.down"] = rnd(w, mlp["shared"]["ff"], s=std)
                out[p + "mlp.shared.sg"] = rnd(1, w, s=2 * std / w ** 0.5)
    return {k: v.to(dtype).contiguous() for k, v in out.items()}


def write_folder(folder, cfg, weights) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(for_file(cfg)))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder
