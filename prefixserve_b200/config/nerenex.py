"""Typed Nerenex configuration, read from the keys of a model folder's config.json.

Nerenex is a decoder whose layers are listed one by one: each entry of
``layers`` names its mixer (``latent_attention``: attention through low-rank
latents with a sliding window; ``rglru``: a gated linear recurrence behind a
short convolution), the mixer's sizes, and its feed-forward (or none).  Keys:

    architecture: "Nerenex"
    vocab, width, residual_mult, norm.eps
    embedding.bigram.{buckets, mul_prev, mul_cur}
    layers[i].type, layers[i].mixer.{...}, layers[i].mlp = {kind: "dense", ff} | null
      latent_attention: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask.size, rot.{base, dims}
      rglru: width, blocks, conv

Every size and constant the engine uses for such a model comes from here;
what the design fixes (the recurrence's decay factor, the activations) is in
the parts.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .llama import UnsupportedModelError

ARCHITECTURE = "Nerenex"


def _need(d: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise UnsupportedModelError(f"config.json: {where} lacks {key!r}")
    return d[key]


def _positive(value: Any, what: str) -> int:
    n = int(value)
    if n < 1 or n != value:
        raise UnsupportedModelError(f"config.json: {what} must be a positive integer, is {value!r}")
    return n


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int        # unrotated query/key dimensions per head
    rot_dim: int    # rotated query/key dimensions per head (the key's are shared by all heads)
    vdim: int       # value dimensions per head
    q_rank: int
    kv_rank: int
    scale: float
    window: int | None   # a query sees itself and the window - 1 tokens before it; None: all
    rot_base: float
    rot_dims: int   # how many of the rotated part's dimensions actually turn

    kind = "latent_attention"

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        rot = _need(m, "rot", where)
        mask = m.get("mask")
        cfg = LatentAttentionConfig(
            heads=_positive(_need(m, "heads", where), f"{where}.heads"),
            dim=_positive(_need(m, "dim", where), f"{where}.dim"),
            rot_dim=_positive(_need(m, "rot_dim", where), f"{where}.rot_dim"),
            vdim=_positive(_need(m, "vdim", where), f"{where}.vdim"),
            q_rank=_positive(_need(m, "q_rank", where), f"{where}.q_rank"),
            kv_rank=_positive(_need(m, "kv_rank", where), f"{where}.kv_rank"),
            scale=float(_need(m, "scale", where)),
            window=None if mask is None else _positive(_need(mask, "size", f"{where}.mask"), f"{where}.mask.size"),
            rot_base=float(_need(rot, "base", f"{where}.rot")),
            rot_dims=_positive(_need(rot, "dims", f"{where}.rot"), f"{where}.rot.dims"),
        )
        if cfg.rot_dims % 2 or cfg.rot_dims > cfg.rot_dim:
            raise UnsupportedModelError(f"config.json: {where}.rot.dims {cfg.rot_dims} must be even and at most rot_dim {cfg.rot_dim}")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                               "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale,
                               "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class RecurrentConfig:
    width: int    # channels of the recurrence
    blocks: int   # the gates' matrices are block-diagonal with this many blocks
    conv: int     # taps of the causal convolution

    kind = "rglru"

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "RecurrentConfig":
        cfg = RecurrentConfig(width=_positive(_need(m, "width", where), f"{where}.width"),
                              blocks=_positive(_need(m, "blocks", where), f"{where}.blocks"),
                              conv=_positive(_need(m, "conv", where), f"{where}.conv"))
        if cfg.width % cfg.blocks:
            raise UnsupportedModelError(f"config.json: {where}: {cfg.width} channels cannot be cut into {cfg.blocks} equal blocks")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


_MIXERS = {"latent_attention": LatentAttentionConfig, "rglru": RecurrentConfig}


@dataclass(frozen=True)
class NerenexLayer:
    mixer: LatentAttentionConfig | RecurrentConfig
    ff: int | None   # inner size of the dense feed-forward; None: the layer has no feed-forward


@dataclass(frozen=True)
class NerenexConfig:
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    bigram_buckets: int | None   # None: a config.json without embedding.bigram, the plain token embedding
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: tuple[NerenexLayer, ...]
    stop_token_ids: frozenset[int] = frozenset()

    architecture = ARCHITECTURE

    @staticmethod
    def from_dicts(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "NerenexConfig":
        if raw.get("architecture") != ARCHITECTURE and ARCHITECTURE not in (raw.get("architectures") or []):
            raise UnsupportedModelError(f"config.json does not describe a {ARCHITECTURE} model")
        bigram = (raw.get("embedding") or {}).get("bigram")
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the top level")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in _MIXERS:
                raise UnsupportedModelError(f"config.json: {where}.type {kind!r} is not one of {sorted(_MIXERS)}")
            mixer = _MIXERS[kind].from_dict(_need(entry, "mixer", where), f"{where}.mixer")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise UnsupportedModelError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r} is not built (dense)")
                ff = _positive(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff")
            layers.append(NerenexLayer(mixer, ff))
        if not layers:
            raise UnsupportedModelError("config.json: a model needs at least one layer")
        stops: set[int] = set()
        eos = (generation or {}).get("eos_token_id")
        if eos is not None:
            stops.update(int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return NerenexConfig(
            vocab=_positive(_need(raw, "vocab", "the top level"), "vocab"),
            width=_positive(_need(raw, "width", "the top level"), "width"),
            residual_mult=float(_need(raw, "residual_mult", "the top level")),
            norm_eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            bigram_buckets=None if bigram is None else _positive(_need(bigram, "buckets", "embedding.bigram"), "embedding.bigram.buckets"),
            bigram_mul_prev=0 if bigram is None else int(_need(bigram, "mul_prev", "embedding.bigram")),
            bigram_mul_cur=0 if bigram is None else int(_need(bigram, "mul_cur", "embedding.bigram")),
            layers=tuple(layers),
            stop_token_ids=frozenset(stops),
        )

    def to_config_json(self) -> dict[str, Any]:
        embedding = {} if self.bigram_buckets is None else {
            "bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev, "mul_cur": self.bigram_mul_cur}}
        return {
            "architecture": ARCHITECTURE,
            "vocab": self.vocab,
            "width": self.width,
            "residual_mult": self.residual_mult,
            "norm": {"eps": self.norm_eps},
            "embedding": embedding,
            "layers": [{"type": layer.mixer.kind, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}} for layer in self.layers],
        }
