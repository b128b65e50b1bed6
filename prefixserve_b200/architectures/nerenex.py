"""Nerenex as a list of parts.

Embedding: token row plus a hashed (previous token, token) row.  Layers in the
order config.json lists them, each a mixer (``latent_attention`` or ``rglru``)
and, where the entry has one, a dense feed-forward with the xIELU activation;
both sublayers read the stream itself, their result is gated by a sigmoid of a
linear function of that input, normed (RMS, gain stored around zero) and added
times ``residual_mult`` (the ``gated_post_norm`` arrangement).  Final norm of
the same kind, logits through the embedding table.

The design has no position limit of its own (rotation by absolute position,
a window, a recurrence): ``max_positions`` is only the bound up to which the
engine may be asked to build angle tables.
"""

from __future__ import annotations

import re

from ..config.nerenex import ARCHITECTURE, LatentAttentionConfig, NerenexConfig, RecurrentConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, part, sequential_schedule

MAX_POSITIONS = 1 << 20
RECURRENCE_DECAY = 8.0  # log a = -8 * r * softplus(lam): fixed by the design


def _mixer_spec(cfg: NerenexConfig, m):
    if isinstance(m, LatentAttentionConfig):
        position = part("rope", head_dim=m.rot_dim, rotary_dim=m.rot_dims, theta=m.rot_base, scaling=None, layout="interleaved")
        return part("latent_attention", hidden_size=cfg.width, num_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim,
                    q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale, window=m.window, eps=cfg.norm_eps, head_gate=True,
                    position=position)
    if isinstance(m, RecurrentConfig):
        return part("gated_linear_recurrence", hidden_size=cfg.width, width=m.width, blocks=m.blocks, taps=m.conv,
                    decay=RECURRENCE_DECAY)
    raise TypeError(f"no mixer for {type(m).__name__}")


def nerenex_spec(cfg: NerenexConfig) -> ModelSpec:
    norm = part("rms", size=cfg.width, eps=cfg.norm_eps, zero_centred=True)
    gate = part("sigmoid_linear", size=cfg.width, bias=True)
    layers = []
    for layer in cfg.layers:
        ffn = None if layer.ff is None else part("mlp", hidden_size=cfg.width, intermediate_size=layer.ff, activation="xielu")
        layers.append(LayerSpec(mixer=_mixer_spec(cfg, layer.mixer), ffn=ffn, mixer_norm=norm,
                                ffn_norm=None if ffn is None else norm, arrangement="gated_post_norm", mixer_gate=gate,
                                ffn_gate=None if ffn is None else gate, residual_scale=cfg.residual_mult))
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=MAX_POSITIONS,
        embedding=part("hashed_pair_embedding", vocab_size=cfg.vocab, hidden_size=cfg.width, buckets=cfg.bigram_buckets,
                       mul_prev=cfg.bigram_mul_prev, mul_cur=cfg.bigram_mul_cur) if cfg.bigram_buckets is not None
        else part("token_embedding", vocab_size=cfg.vocab, hidden_size=cfg.width),
        layers=tuple(layers),
        schedule=sequential_schedule(len(layers)),
        final_norm=norm,
        head=part("lm_head", vocab_size=cfg.vocab, hidden_size=cfg.width, tied=True),
        stop_token_ids=cfg.stop_token_ids,
    )


_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")
_IN_LAYER = {
    "mixer_norm.weight": "norm1",
    "ffn_norm.weight": "norm2",
    "mixer_gate.weight": "rg1",
    "mixer_gate.bias": "rg1.b",
    "ffn_gate.weight": "rg2",
    "ffn_gate.bias": "rg2.b",
    # latent attention
    "mixer.q_down": "mix.dq",
    "mixer.q_down_norm": "mix.dq.norm",
    "mixer.q_up": "mix.uq",
    "mixer.kv_down": "mix.dkv",
    "mixer.kv_down_norm": "mix.dkv.norm",
    "mixer.k_up": "mix.uk",
    "mixer.v_up": "mix.uv",
    "mixer.head_gate": "mix.g",
    "mixer.o_proj": "mix.o",
    # recurrence
    "mixer.gate_proj": "mix.y",
    "mixer.gate_bias": "mix.y.b",
    "mixer.in_proj": "mix.x",
    "mixer.in_bias": "mix.x.b",
    "mixer.conv_weight": "mix.conv",
    "mixer.conv_bias": "mix.conv.b",
    "mixer.recurrence_gate": "mix.ra",
    "mixer.recurrence_gate_bias": "mix.ra.b",
    "mixer.input_gate": "mix.ri",
    "mixer.input_gate_bias": "mix.ri.b",
    "mixer.decay_param": "mix.lam",
    # feed-forward
    "ffn.up_proj": "mlp.up",
    "ffn.down_proj": "mlp.down",
    "ffn.act": "mlp.act",
}
_TOP = {"embedding.weight": "embed", "embedding.pair_weight": "bigram", "final_norm.weight": "final.norm"}


def nerenex_tensor_name(path: str) -> str:
    if path in _TOP:
        return _TOP[path]
    m = _LAYER.match(path)
    if m and m.group(2) in _IN_LAYER:
        return f"l{m.group(1)}.{_IN_LAYER[m.group(2)]}"
    raise KeyError(f"{ARCHITECTURE} has no tensor for part path {path!r}")


NERENEX = Architecture(
    name=ARCHITECTURE,
    model_types=("nerenex",),
    read_config=NerenexConfig.from_dicts,
    to_spec=nerenex_spec,
    tensor_name=nerenex_tensor_name,
)

register_architecture(NERENEX, replace=True)
