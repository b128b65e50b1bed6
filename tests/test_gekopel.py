"""Gekopel without a GPU: the configuration reader, the parts list and tensor names, the cache manager's chunk groups,
the distance buckets, and the plain implementation's own consistency (a prompt run whole against the same prompt run
as a recurrence from carried state is what the engine is tested for on a GPU; here the oracle's pieces are checked
against each other where the design says two forms are the same)."""

import json
import math

import pytest
import torch

import gekopel_models as gm
import plain_gekopel as plain


def test_config_reader_takes_every_key_and_refuses_what_is_missing():
    from prefixserve_b200.config import GekopelConfig, RoutedFF, UnsupportedModelError
    raw = gm.for_file(gm.CONFIGS["mixed"])
    cfg = GekopelConfig.from_dicts(raw)
    assert (cfg.vocab, cfg.width, cfg.max_positions, cfg.norm_eps, cfg.embedding_scale) == (131, 40, 400, 3e-6, 5.5)
    assert [l.mixer.kind for l in cfg.layers] == ["delta", "attention", "delta", "attention", "attention", "delta"]
    assert cfg.layers[1].mixer.chunk == 37 and cfg.layers[3].mixer.chunk is None and cfg.layers[4].mlp is None
    moe = cfg.layers[1].mlp
    assert isinstance(moe, RoutedFF) and (moe.experts, moe.top, moe.groups, moe.keep, moe.shared_ff) == (8, 3, 4, 3, None)
    assert cfg.to_config_json() == raw  # what is written is what was read
    for drop in (("vocab",), ("norm", "eps"), ("layers", 0, "mixer", "conv"), ("layers", 1, "mixer", "bias_max"),
                 ("layers", 1, "mlp", "router", "top"), ("max_positions",)):
        broken = json.loads(json.dumps(raw))
        at = broken
        for k in drop[:-1]:
            at = at[k]
        del at[drop[-1]]
        with pytest.raises(UnsupportedModelError):
            GekopelConfig.from_dicts(broken)
    broken = json.loads(json.dumps(raw))
    broken["layers"][1]["mlp"]["router"]["groups"] = {"count": 3, "keep": 2}  # 8 experts in 3 groups
    with pytest.raises(UnsupportedModelError):
        GekopelConfig.from_dicts(broken)


def test_every_tensor_of_a_checkpoint_has_a_part_and_the_table_rows_come_from_the_file(tmp_path):
    from prefixserve_b200.config.registry import read_model_folder
    from prefixserve_b200 import architectures  # noqa: F401
    from prefixserve_b200.parts.model import build_model
    for which, cfg in gm.CONFIGS.items():
        weights = gm.tensors(cfg, seed=1)
        folder = gm.write_folder(tmp_path / which, cfg, weights)
        arch, typed = read_model_folder(folder)
        model = build_model(arch.to_spec(typed))
        wanted = {arch.tensor_name(path): tuple(spec.shape) for path, spec in model.param_table().items()}
        assert wanted == {k: tuple(v.shape) for k, v in weights.items()}, which
        rows = [l["mixer"]["_rows"] for l in cfg["layers"] if l["type"] == "attention"]
        assert [l.mixer.bias_rows for l in typed.layers if l.mixer.kind == "attention"] == rows


def test_cache_needs_chunk_groups_and_states(tmp_path):
    from prefixserve_b200.config.registry import read_model_folder
    from prefixserve_b200 import architectures  # noqa: F401
    from prefixserve_b200.parts.model import build_model
    from prefixserve_b200.cache.manager import CacheManager
    arch, typed = read_model_folder(gm.write_folder(tmp_path, gm.CONFIGS["mixed"], gm.tensors(gm.CONFIGS["mixed"])))
    model = build_model(arch.to_spec(typed))
    needs = model.cache_needs()
    assert [n.paged.chunk if n.paged else "-" for n in needs] == ["-", 37, "-", None, 64, "-", "-"]
    assert needs[1].paged.head_dim == 16 and needs[1].paged.planes == 1 and needs[3].paged.head_dim == 40
    assert needs[0].state.shape == (3 * (2 * 2 * 6 + 4 * 10) + 4 * 6 * 10,)
    cache = CacheManager(needs, num_pages=40, num_slots=2, max_seq_len=320, page_size=8, device=None)
    assert [(g.window, g.chunk) for g in cache.groups] == [(None, 37), (None, None), (None, 64)]
    assert not cache.prefix_cache_possible
    slot = cache.open()
    assert cache.reserve(slot, 100)
    cache.advance(slot, 100)
    # position 100 reads from 74 on in runs of 37 and from 64 on in runs of 64: earlier pages are back in the pool
    assert [cache.free_pages(g) for g in range(3)] == [40 - (13 - 74 // 8), 40 - 13, 40 - (13 - 64 // 8)]
    cache.advance(slot, 111)   # 111 = 3 * 37: the next token starts a run, nothing before it is read again
    assert cache.free_pages(0) == 40 - (13 - 111 // 8)
    cache.check()
    cache.close(slot)
    assert [cache.free_pages(g) for g in range(3)] == [40, 40, 40]


@pytest.mark.parametrize("rows, reach", [(32, 100), (10, 24), (11, 50), (6, 9), (32, 300), (16, 128), (2, 5)])
def test_distance_buckets(rows, reach):
    from prefixserve_b200.parts.biased_attention import distance_bucket
    half = rows // 2
    got = [distance_bucket(n, rows, reach) for n in range(2 * reach + 5)]
    assert got[:half] == list(range(half))
    assert all(b - a in (0, 1) or a < half for a, b in zip(got, got[1:])) or rows - half > reach - half
    assert all(a <= b for a, b in zip(got, got[1:])) and got[-1] == rows - 1 and max(got) == rows - 1
    assert all(got[n] == rows - 1 for n in range(reach, len(got)))
    assert got == [plain.distance_bucket(n, rows, reach) for n in range(len(got))]
    for n in range(half, reach):  # the defining inequality, in exact terms: (n / half)^(rows - half) against (reach / half)^k
        k = got[n] - half
        if got[n] < rows - 1:
            assert (reach / half) ** k <= (n / half) ** (rows - half) * (1 + 1e-9)
            assert (n / half) ** (rows - half) < (reach / half) ** (k + 1) * (1 + 1e-9)


def test_plain_delta_rule_reads_the_current_write_and_forgets():
    """With beta = 1, no decay and orthogonal unit keys the state stores v under k exactly; the read-out with q = k
    returns the value written at the same token; a decay of 1/2 halves what an earlier token left."""
    k = torch.eye(4, dtype=torch.float64)[:3].reshape(3, 1, 4)
    v = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=torch.float64).reshape(3, 1, 2)
    one = torch.ones(3, 1, dtype=torch.float64)
    assert torch.equal(plain.delta_rule(k, k, v, one, one), v)
    q = k[[0, 0, 0]]
    out = plain.delta_rule(q, k, v, one, 0.5 * one)
    assert torch.allclose(out[:, 0], torch.stack([v[0, 0], v[0, 0] / 2, v[0, 0] / 4]))
    # writing under the same key again replaces the value (that is the "delta")
    same = k[[0, 0, 0]]
    assert torch.allclose(plain.delta_rule(same, same, v, one, one), v)


def test_plain_router_groups_and_weights():
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    w = {"m.router": torch.eye(6, dtype=torch.float64), "m.correction": torch.tensor([0, 0, 0, 0, 0.9, 0], dtype=torch.float64)}
    # logits: expert 0 is the single best, but the pair (2, 3) is the best group without the correction, and the
    # correction lifts the group (4, 5) above it
    h = torch.tensor([[3.0, -9, 1.5, 1.5, 1.0, 1.0]], dtype=torch.float64)
    chosen, weight = plain.route(r, w, "m.", h)
    assert sorted(chosen[0].tolist()) == [4, 5]
    s = torch.sigmoid(h[0, [4, 5]])
    assert torch.allclose(weight[0].sort().values, (s / s.sum() * 2.0).sort().values)   # weights without the correction
    w["m.correction"] = torch.zeros(6, dtype=torch.float64)
    chosen, _ = plain.route(r, w, "m.", h)
    assert sorted(chosen[0].tolist()) == [2, 3]
    # dropped experts count as minus infinity even when every choice score is negative
    w["m.correction"] = torch.full((6,), -5.0, dtype=torch.float64)
    chosen, _ = plain.route(r, w, "m.", h)
    assert sorted(chosen[0].tolist()) == [2, 3]


def test_plain_attention_chunks_sink_and_bias():
    m = gm.attention(heads=2, kv_heads=1, dim=4, vdim=3, scale=0.5, bias_max=9, chunk=5, rows=6)
    g = torch.Generator().manual_seed(3)
    w = {"a.q": torch.randn(8, 7, generator=g).double(), "a.k": torch.randn(4, 7, generator=g).double(),
         "a.v": torch.randn(3, 7, generator=g).double(), "a.o": torch.eye(6, dtype=torch.float64),
         "a.rel": torch.randn(6, 2, generator=g).double(), "a.sink": torch.tensor([0.3, -20.0], dtype=torch.float64)}
    h = torch.randn(12, 7, generator=g).double()
    out = plain.attention(m, w, "a.", h)
    # a chunk's first token sees itself only: with a sink far below (head 1) its output is its own value
    v = h @ w["a.v"].T
    for i in (0, 5, 10):
        assert torch.allclose(out[i, 3:], v[i], atol=1e-8)
        assert out[i, :3].norm() < v[i].norm()          # head 0's sink takes its share of the weight
    # tokens of one chunk do not depend on anything before the chunk
    h2 = h.clone()
    h2[:5] = torch.randn(5, 7, generator=g).double()
    assert torch.equal(plain.attention(m, w, "a.", h2)[5:], out[5:])
    # without a chunk mask they do
    m2 = dict(m)
    m2.pop("mask")
    assert not torch.allclose(plain.attention(m2, w, "a.", h2)[5:], plain.attention(m2, w, "a.", h)[5:])
