"""Typed Gekopel configuration, read from the keys of a model folder's config.json.

Gekopel is a decoder whose layers are listed one by one: each entry of ``layers`` names its mixer (``attention``:
softmax attention with a learned distance bias, a chunk mask and a sink; ``delta``: the gated delta rule behind short
convolutions), the mixer's sizes, and its feed-forward (dense, a mixture of experts, or none).  Keys:

    architecture: "Gekopel"
    vocab, width, max_positions, norm.eps, embedding.scale
    layers[i].type, layers[i].mixer.{...}, layers[i].mlp
      attention: heads, kv_heads, dim, vdim, scale, bias_max, mask.size (mask absent: no chunk mask)
      delta: heads, kv_heads, dim, vdim, conv
      mlp: null | {kind: "dense", ff}
           | {kind: "moe", expert.ff, router.{experts, top, scale, groups.{count, keep}}, shared.ff (shared absent: none)}

Every size and constant the engine uses for such a model comes from here or from a tensor's shape (the rows of a
layer's distance-bias table); what the design fixes (activations, the small constants of the norms) is in the parts.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .llama import UnsupportedModelError
from .nerenex import _need, _positive

ARCHITECTURE = "Gekopel"
DEFAULT_BIAS_ROWS = 64  # rows of a layer's distance-bias table when a configuration is made here (random-weights mode)


@dataclass(frozen=True)
class BiasedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int            # query/key size per head
    vdim: int           # value size per head
    scale: float
    bias_max: int       # the distance from which every key shares the table's last row
    chunk: int | None   # a query sees keys of its own run of this many positions; None: all earlier keys
    bias_rows: int = DEFAULT_BIAS_ROWS   # rows of the distance-bias table (taken from the tensor's shape when loading)

    kind = "attention"

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "BiasedAttentionConfig":
        mask = m.get("mask")
        cfg = BiasedAttentionConfig(
            heads=_positive(_need(m, "heads", where), f"{where}.heads"),
            kv_heads=_positive(_need(m, "kv_heads", where), f"{where}.kv_heads"),
            dim=_positive(_need(m, "dim", where), f"{where}.dim"),
            vdim=_positive(_need(m, "vdim", where), f"{where}.vdim"),
            scale=float(_need(m, "scale", where)),
            bias_max=_positive(_need(m, "bias_max", where), f"{where}.bias_max"),
            chunk=None if mask is None else _positive(_need(mask, "size", f"{where}.mask"), f"{where}.mask.size"),
        )
        if cfg.heads % cfg.kv_heads:
            raise UnsupportedModelError(f"config.json: {where}: {cfg.heads} heads cannot share {cfg.kv_heads} key/value heads")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "bias_max": self.bias_max}
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        return out


@dataclass(frozen=True)
class DeltaConfig:
    heads: int      # value heads (and states)
    kv_heads: int   # query/key groups
    dim: int
    vdim: int
    conv: int       # taps of the short convolutions

    kind = "delta"

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "DeltaConfig":
        cfg = DeltaConfig(heads=_positive(_need(m, "heads", where), f"{where}.heads"),
                          kv_heads=_positive(_need(m, "kv_heads", where), f"{where}.kv_heads"),
                          dim=_positive(_need(m, "dim", where), f"{where}.dim"),
                          vdim=_positive(_need(m, "vdim", where), f"{where}.vdim"),
                          conv=_positive(_need(m, "conv", where), f"{where}.conv"))
        if cfg.heads % cfg.kv_heads:
            raise UnsupportedModelError(f"config.json: {where}: {cfg.heads} heads cannot share {cfg.kv_heads} query/key groups")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class DenseFF:
    ff: int

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    top: int
    ff: int                 # inner size of every expert
    scale: float            # multiplies the normalised weights
    groups: int             # equal groups of neighbouring experts
    keep: int               # groups whose experts can be chosen
    shared_ff: int | None   # inner size of the expert every token uses; None: none

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "RoutedFF":
        router = _need(m, "router", where)
        groups = router.get("groups") or {}
        count = _positive(groups.get("count", 1), f"{where}.router.groups.count")
        shared = m.get("shared")
        cfg = RoutedFF(experts=_positive(_need(router, "experts", f"{where}.router"), f"{where}.router.experts"),
                       top=_positive(_need(router, "top", f"{where}.router"), f"{where}.router.top"),
                       ff=_positive(_need(_need(m, "expert", where), "ff", f"{where}.expert"), f"{where}.expert.ff"),
                       scale=float(router.get("scale", 1.0)),
                       groups=count,
                       keep=_positive(groups.get("keep", count), f"{where}.router.groups.keep"),
                       shared_ff=None if shared is None else _positive(_need(shared, "ff", f"{where}.shared"), f"{where}.shared.ff"))
        if cfg.experts % cfg.groups or cfg.keep > cfg.groups:
            raise UnsupportedModelError(f"config.json: {where}.router: {cfg.experts} experts cannot form {cfg.groups} equal groups of which {cfg.keep} are kept")
        if cfg.top > cfg.keep * (cfg.experts // cfg.groups):
            raise UnsupportedModelError(f"config.json: {where}.router: {cfg.keep} groups of {cfg.experts // cfg.groups} experts cannot give {cfg.top} choices")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                               "router": {"experts": self.experts, "top": self.top, "scale": self.scale,
                                          "groups": {"count": self.groups, "keep": self.keep}}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


_MIXERS = {"attention": BiasedAttentionConfig, "delta": DeltaConfig}


@dataclass(frozen=True)
class GekopelLayer:
    mixer: BiasedAttentionConfig | DeltaConfig
    mlp: DenseFF | RoutedFF | None


@dataclass(frozen=True)
class GekopelConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[GekopelLayer, ...]
    stop_token_ids: frozenset[int] = frozenset()

    architecture = ARCHITECTURE

    @staticmethod
    def from_dicts(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "GekopelConfig":
        if raw.get("architecture") != ARCHITECTURE and ARCHITECTURE not in (raw.get("architectures") or []):
            raise UnsupportedModelError(f"config.json does not describe a {ARCHITECTURE} model")
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the top level")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in _MIXERS:
                raise UnsupportedModelError(f"config.json: {where}.type {kind!r} is not one of {sorted(_MIXERS)}")
            mixer = _MIXERS[kind].from_dict(_need(entry, "mixer", where), f"{where}.mixer")
            mlp = entry.get("mlp")
            ff: DenseFF | RoutedFF | None = None
            if mlp is not None:
                kind = mlp.get("kind")
                if kind == "dense":
                    ff = DenseFF(_positive(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff"))
                elif kind == "moe":
                    ff = RoutedFF.from_dict(mlp, f"{where}.mlp")
                else:
                    raise UnsupportedModelError(f"config.json: {where}.mlp.kind {kind!r} is not built (dense, moe)")
            layers.append(GekopelLayer(mixer, ff))
        if not layers:
            raise UnsupportedModelError("config.json: a model needs at least one layer")
        stops: set[int] = set()
        eos = (generation or {}).get("eos_token_id")
        if eos is not None:
            stops.update(int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return GekopelConfig(
            vocab=_positive(_need(raw, "vocab", "the top level"), "vocab"),
            width=_positive(_need(raw, "width", "the top level"), "width"),
            max_positions=_positive(_need(raw, "max_positions", "the top level"), "max_positions"),
            norm_eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            layers=tuple(layers),
            stop_token_ids=frozenset(stops),
        )

    def to_config_json(self) -> dict[str, Any]:
        return {
            "architecture": ARCHITECTURE,
            "vocab": self.vocab,
            "width": self.width,
            "max_positions": self.max_positions,
            "norm": {"eps": self.norm_eps},
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": layer.mixer.kind, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.mlp is None else layer.mlp.to_dict()} for layer in self.layers],
        }
