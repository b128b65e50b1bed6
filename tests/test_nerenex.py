"""Nerenex on the host: the configuration reader and its refusals, the model description, the checkpoint's tensor
names, and the plain implementation's own consistency (the oracle the GPU tests compare the engine with)."""

import copy

import pytest
import torch

import nerenex_models as nm
import plain_nerenex as plain
from prefixserve_b200 import architectures  # noqa: F401
from prefixserve_b200.config import NerenexConfig, UnsupportedModelError, architecture_of
from prefixserve_b200.parts.model import build_model


def test_config_reads_every_size_and_round_trips():
    raw = nm.CONFIGS["mixed"]
    arch = architecture_of(raw)
    assert arch.name == "Nerenex"
    cfg = arch.read_config(raw, None)
    assert cfg.vocab == 131 and cfg.width == 40 and cfg.residual_mult == 0.45 and cfg.norm_eps == 3e-6
    assert (cfg.bigram_buckets, cfg.bigram_mul_prev, cfg.bigram_mul_cur) == (97, 1000003, 911)
    assert [type(l.mixer).__name__ for l in cfg.layers] == ["RecurrentConfig", "LatentAttentionConfig", "LatentAttentionConfig",
                                                            "RecurrentConfig", "LatentAttentionConfig"]
    assert [l.ff for l in cfg.layers] == [28, None, 50, None, 31]
    a = cfg.layers[1].mixer
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.q_rank, a.kv_rank, a.window, a.rot_dims, a.rot_base) == (5, 6, 10, 4, 9, 21, 19, 6, 5000.0)
    assert NerenexConfig.from_dicts(cfg.to_config_json()) == cfg
    assert cfg.to_config_json()["layers"] == raw["layers"]


def test_a_missing_mask_means_every_earlier_token_is_seen():
    cfg = NerenexConfig.from_dicts(nm.CONFIGS["attn_ff"])
    assert cfg.layers[0].mixer.window is None
    spec = architecture_of(nm.CONFIGS["attn_ff"]).to_spec(cfg)
    assert build_model(spec).cache_needs()[0].paged.window is None


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv_only"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 3), "rot.dims"),
    (lambda c: c["layers"][0].__setitem__("mlp", {"kind": "routed", "ff": 8}), "kind"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c.__setitem__("layers", []), "layer"),
])
def test_config_refusals_name_the_key(damage, word):
    raw = copy.deepcopy(nm.CONFIGS["attn_only"])
    damage(raw)
    with pytest.raises(UnsupportedModelError, match=word):
        NerenexConfig.from_dicts(raw)


def test_without_a_pair_table_the_embedding_is_the_plain_one():
    raw = copy.deepcopy(nm.CONFIGS["rec_only"])
    raw["embedding"] = {}
    arch = architecture_of(raw)
    model = build_model(arch.to_spec(arch.read_config(raw, None)))
    names = {arch.tensor_name(path) for path in model.param_table()}
    assert "bigram" not in names and "embed" in names and len(model.cache_needs()) == 1


def test_recurrence_blocks_must_divide_the_channels():
    raw = copy.deepcopy(nm.CONFIGS["rec_only"])
    raw["layers"][0]["mixer"]["blocks"] = 7
    with pytest.raises(UnsupportedModelError, match="blocks"):
        NerenexConfig.from_dicts(raw)


@pytest.mark.parametrize("which", sorted(nm.CONFIGS))
def test_parameter_table_is_the_checkpoint(which):
    """Every tensor the tests' writer makes is wanted by the model under that name and shape, and nothing else is."""
    raw = nm.CONFIGS[which]
    arch = architecture_of(raw)
    model = build_model(arch.to_spec(arch.read_config(raw, None)))
    wanted = {arch.tensor_name(path): tuple(ps.shape) for path, ps in model.param_table().items()}
    made = {name: tuple(t.shape) for name, t in nm.tensors(raw).items()}
    assert wanted == made


def test_cache_needs_one_latent_row_per_token_and_states_for_the_rest():
    raw = nm.CONFIGS["mixed"]
    arch = architecture_of(raw)
    needs = build_model(arch.to_spec(arch.read_config(raw, None))).cache_needs()
    assert len(needs) == 6  # five layers and the embedding's previous token
    assert needs[0].paged is None and needs[0].state.shape == (1, 32)
    assert (needs[1].paged.planes, needs[1].paged.num_kv_heads, needs[1].paged.head_dim, needs[1].paged.window) == (1, 1, 31, 19)
    assert needs[2].paged.window == 4 and needs[4].paged.window == 33
    assert needs[3].state.shape == (5, 48) and needs[3].state.dtype == torch.float32
    assert needs[5].paged is None and needs[5].state.dtype == torch.int32


# ---- the plain implementation against itself -----------------------------------------------------------------

def test_plain_rotation_keeps_lengths_and_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 8, generator=g, dtype=torch.float64), torch.randn(1, 8, generator=g, dtype=torch.float64)
    def dot(pq, pk):
        return float((plain.rotate_interleaved(q, torch.tensor([pq]), 6, 50.0) * plain.rotate_interleaved(k, torch.tensor([pk]), 6, 50.0)).sum())
    assert abs(dot(9, 4) - dot(105, 100)) < 1e-9 and abs(dot(9, 4) - dot(9, 5)) > 1e-6
    r = plain.rotate_interleaved(q, torch.tensor([7]), 6, 50.0)
    assert torch.allclose(r[:, 6:], q[:, 6:]) and abs(float(r.norm() - q.norm())) < 1e-12


def test_plain_xielu_is_continuous_with_slope_one_half_at_zero():
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.2, dtype=torch.float64)
    z = torch.tensor([-1e-6, 0.0, 1e-6], dtype=torch.float64)
    v = plain.xielu(z, p, q)
    assert abs(float(v[1])) < 1e-15 and abs(float((v[2] - v[0]) / 2e-6) - 0.5) < 1e-5
    assert float(plain.xielu(torch.tensor(2.0, dtype=torch.float64), p, q)) == pytest.approx(float(plain.softplus(p)) * 4 + 1)


def test_plain_window_hides_exactly_the_tokens_beyond_it():
    """Changing a token that lies just outside every later window does not change the last logits; just inside does."""
    raw = nm.CONFIGS["attn_only"]  # window 7, one layer
    w = nm.as_double(nm.tensors(raw, seed=3))
    toks = [5, 9, 33, 2, 17, 40, 8, 21, 3, 11, 50, 6]
    base = plain.forward(raw, w, toks)[-1]
    outside, inside = list(toks), list(toks)
    outside[len(toks) - 1 - 7 - 1] = 59   # two tokens before the window: neither its key nor its hashed pair is in reach
    inside[len(toks) - 1 - 6] = 59
    assert torch.allclose(plain.forward(raw, w, outside)[-1], base, atol=1e-12)
    assert not torch.allclose(plain.forward(raw, w, inside)[-1], base, atol=1e-6)


def test_plain_recurrence_carries_state_and_convolution_inputs():
    """Running a sequence in two halves with the state handed over equals the whole: checked by a step-by-step
    restatement of the recurrence written here."""
    raw = nm.CONFIGS["rec_only"]
    w = nm.as_double(nm.tensors(raw, seed=5))
    m = raw["layers"][0]["mixer"]
    x = torch.randn(11, raw["width"], generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    whole = plain.rglru(x, w, "l0.mix.", m)
    # token by token: a window of the last inputs and a state
    K, W, nb = m["conv"], m["width"], m["blocks"]
    hist = torch.zeros(K - 1, W, dtype=torch.float64)
    s = torch.zeros(W, dtype=torch.float64)
    rows = []
    for t in range(x.shape[0]):
        xin = x[t] @ w["l0.mix.x"].T + w["l0.mix.x.b"]
        win = torch.cat([hist, xin[None]])
        u = (win * w["l0.mix.conv"].T).sum(0) + w["l0.mix.conv.b"]
        hist = win[1:]
        ub = u.view(nb, -1)
        r = torch.sigmoid(torch.einsum("bi,boi->bo", ub, w["l0.mix.ra"]) + w["l0.mix.ra.b"]).reshape(-1)
        i = torch.sigmoid(torch.einsum("bi,boi->bo", ub, w["l0.mix.ri"]) + w["l0.mix.ri.b"]).reshape(-1)
        a = torch.exp(-8.0 * r * torch.nn.functional.softplus(w["l0.mix.lam"]))
        s = a * s + torch.sqrt(1 - a * a) * i * u
        rows.append((s * plain.gelu_tanh(x[t] @ w["l0.mix.y"].T + w["l0.mix.y.b"])) @ w["l0.mix.o"].T)
    assert torch.allclose(torch.stack(rows), whole, atol=1e-12)


def test_plain_first_token_takes_the_last_pair_row():
    raw = nm.CONFIGS["attn_only"]
    w = nm.as_double(nm.tensors(raw))
    b = raw["embedding"]["bigram"]
    x = plain.embed_tokens([4, 9], w["embed"], w["bigram"], b["mul_prev"], b["mul_cur"], b["buckets"])
    assert torch.equal(x[0], w["embed"][4] + w["bigram"][b["buckets"]])
    assert torch.equal(x[1], w["embed"][9] + w["bigram"][(4 * b["mul_prev"] + 9 * b["mul_cur"]) % b["buckets"]])
