"""Gekopel as a list of parts.

Embedding: token row times a constant plus a learned row per position.  Layers in the order config.json lists them,
each a mixer (``attention``: the ``biased_attention`` part with its chunk mask, distance bias and sink; ``delta``: the
``gated_delta_rule`` part) and, where the entry has one, a feed-forward (dense with the squared-ReLU activation, or
routed experts of that form with a shared expert); every sublayer has an RMS norm in front of it and one on its result
(the ``sandwich_norm`` arrangement).  Final norm, untied head.

The rows of a layer's distance-bias table are not in config.json: ``read_folder_config`` takes them from the shape
of the layer's ``mix.rel`` tensor in the checkpoint's header.
"""

from __future__ import annotations

import dataclasses
import json
import re
import struct
from pathlib import Path

from ..config.gekopel import ARCHITECTURE, BiasedAttentionConfig, DeltaConfig, DenseFF, GekopelConfig, RoutedFF
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, part, sequential_schedule


def _mixer_spec(cfg: GekopelConfig, m):
    if isinstance(m, BiasedAttentionConfig):
        return part("biased_attention", hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                    scale=m.scale, chunk=m.chunk, window=None, bias_rows=m.bias_rows, bias_reach=m.bias_max, sink=True)
    if isinstance(m, DeltaConfig):
        return part("gated_delta_rule", hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                    taps=m.conv, eps=cfg.norm_eps)
    raise TypeError(f"no mixer for {type(m).__name__}")


def _ffn_spec(cfg: GekopelConfig, f):
    if f is None:
        return None
    if isinstance(f, DenseFF):
        return part("mlp", hidden_size=cfg.width, intermediate_size=f.ff, activation="relu2")
    if isinstance(f, RoutedFF):
        return part("routed_experts", hidden_size=cfg.width, experts=f.experts, expert_size=f.ff, top=f.top, groups=f.groups,
                    keep=f.keep, scale=f.scale, correction=True, shared_size=f.shared_ff, shared_gate=True, activation="relu2")
    raise TypeError(f"no feed-forward for {type(f).__name__}")


def gekopel_spec(cfg: GekopelConfig) -> ModelSpec:
    norm = part("rms", size=cfg.width, eps=cfg.norm_eps)
    layers = []
    for layer in cfg.layers:
        ffn = _ffn_spec(cfg, layer.mlp)
        layers.append(LayerSpec(mixer=_mixer_spec(cfg, layer.mixer), ffn=ffn, mixer_norm=norm,
                                ffn_norm=None if ffn is None else norm, arrangement="sandwich_norm", mixer_post_norm=norm,
                                ffn_post_norm=None if ffn is None else norm))
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding=part("token_position_embedding", vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=cfg.max_positions,
                       scale=cfg.embedding_scale),
        layers=tuple(layers),
        schedule=sequential_schedule(len(layers)),
        final_norm=norm,
        head=part("lm_head", vocab_size=cfg.vocab, hidden_size=cfg.width, tied=False),
        stop_token_ids=cfg.stop_token_ids,
    )


_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")
_EXPERT = re.compile(r"^ffn\.experts\.(\d+)\.(up|down)_proj$")
_IN_LAYER = {
    "mixer_norm.weight": "norm1",
    "mixer_post_norm.weight": "norm1b",
    "ffn_norm.weight": "norm2",
    "ffn_post_norm.weight": "norm2b",
    # both mixers
    "mixer.q_proj": "mix.q",
    "mixer.k_proj": "mix.k",
    "mixer.v_proj": "mix.v",
    "mixer.o_proj": "mix.o",
    # attention
    "mixer.rel_bias": "mix.rel",
    "mixer.sink": "mix.sink",
    # delta rule
    "mixer.q_conv": "mix.q.conv",
    "mixer.k_conv": "mix.k.conv",
    "mixer.v_conv": "mix.v.conv",
    "mixer.beta_proj": "mix.b",
    "mixer.decay_rate": "mix.A_log",
    "mixer.out_norm": "mix.norm",
    "mixer.decay_proj": "mix.a",
    "mixer.decay_bias": "mix.dt_bias",
    "mixer.gate_proj": "mix.g",
    # feed-forward
    "ffn.up_proj": "mlp.up",
    "ffn.down_proj": "mlp.down",
    "ffn.router": "mlp.router",
    "ffn.correction": "mlp.correction",
    "ffn.shared.up_proj": "mlp.shared.up",
    "ffn.shared.down_proj": "mlp.shared.down",
    "ffn.shared.gate": "mlp.shared.sg",
}
_TOP = {"embedding.weight": "embed", "embedding.position_weight": "pos", "final_norm.weight": "final.norm", "head.weight": "head"}


def gekopel_tensor_name(path: str) -> str:
    if path in _TOP:
        return _TOP[path]
    m = _LAYER.match(path)
    if m:
        if m.group(2) in _IN_LAYER:
            return f"l{m.group(1)}.{_IN_LAYER[m.group(2)]}"
        e = _EXPERT.match(m.group(2))
        if e:
            return f"l{m.group(1)}.mlp.e{e.group(1)}.{e.group(2)}"
    raise KeyError(f"{ARCHITECTURE} has no tensor for part path {path!r}")


def tensor_shapes(folder: Path) -> dict[str, tuple[int, ...]]:
    """Tensor name -> shape from the header of a folder's model.safetensors (8 bytes of length, then JSON); {} if there
    is no such file."""
    file = Path(folder) / "model.safetensors"
    if not file.exists():
        return {}
    with open(file, "rb") as f:
        (length,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(length))
    return {name: tuple(entry["shape"]) for name, entry in header.items() if name != "__metadata__"}


def with_folder_shapes(cfg: GekopelConfig, folder) -> GekopelConfig:
    """The sizes config.json leaves to the tensors: the rows of every attention layer's distance-bias table."""
    shapes = tensor_shapes(Path(folder))
    layers = list(cfg.layers)
    for i, layer in enumerate(layers):
        shape = shapes.get(f"l{i}.mix.rel")
        if isinstance(layer.mixer, BiasedAttentionConfig) and shape:
            layers[i] = dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, bias_rows=int(shape[0])))
    return dataclasses.replace(cfg, layers=tuple(layers))


GEKOPEL = Architecture(
    name=ARCHITECTURE,
    model_types=("gekopel",),
    read_config=GekopelConfig.from_dicts,
    to_spec=gekopel_spec,
    tensor_name=gekopel_tensor_name,
    refine_config=with_folder_shapes,
)

register_architecture(GEKOPEL, replace=True)
