"""Nerenex through the engine against the plain implementation (tests/plain_nerenex.py): every mechanism alone, every
cutting of the work, reused pages and slots, keys at the edges of windows and pages, long decoding, generation through
the scheduler.  Models and weights are made here (tests/nerenex_models.py)."""

import copy

import numpy as np
import pytest
import torch

import helpers
import nerenex_models as nm
import plain_nerenex as plain

pytestmark = pytest.mark.gpu

LIMIT = {"float32": 2e-5, "bfloat16": 4e-2}
TRACES = {"whole": helpers.trace_whole, "tail_decode": helpers.trace_tail_decode, "portions": helpers.trace_portions,
          "mixed": helpers.trace_mixed}
LENGTHS = [1, 2, 19, 53, 97, 140]


def row_error(got, want):
    """Root mean square of the difference (its mean taken off) over that of the wanted row."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean()
    w = want - want.mean()
    return float(np.sqrt((d * d).mean()) / max(np.sqrt((w * w).mean()), 1e-30))


def sequences(vocab, lengths=LENGTHS, seed=100):
    return {f"r{i}": helpers.random_tokens(vocab, n, seed=seed + i) for i, n in enumerate(lengths)}


def stored(weights, dtype):
    """The weights as a checkpoint of ``dtype`` holds them, and their exact values in float64 for the oracle."""
    held = {k: v.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in weights.items()}
    return held, {k: v.double() for k, v in held.items()}


def replay(folder, dtype, steps, *, max_tokens=None, max_live=64, page_size=16, poison=True, graphs=True):
    from prefixserve_b200.engine.replay import Replayer
    rp = Replayer(folder, dtype, max_tokens or helpers.peak_tokens(steps), max_live=max_live, page_size=page_size,
                  use_graphs=graphs)
    rp.cache.poison_freed = poison
    if poison:  # pages nobody has written yet are as void as pages given back
        for kv in rp.cache.kv:
            if kv is not None:
                kv.fill_(float("nan"))
    outputs = {}
    for st in steps:
        out = rp.run_step(st)
        if out is not None:
            outputs[st["step"]] = out
    rp.cache.check()
    return helpers.collect(steps, outputs)


def worst_error(rows, truth):
    worst = 0.0
    for (rid, pos), got in rows.items():
        assert np.isfinite(got).all(), f"{rid} position {pos}: not finite"
        worst = max(worst, row_error(got, truth[rid][pos].numpy()))
    return worst


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    """(configuration name, dtype) -> (folder, float64 logits of every test sequence)."""
    out = {}
    for which, cfg in nm.CONFIGS.items():
        weights = nm.tensors(cfg, seed=sorted(nm.CONFIGS).index(which))
        for dtype in ("float32", "bfloat16"):
            held, exact = stored(weights, dtype)
            folder = nm.write_folder(tmp_path_factory.mktemp(f"{which}-{dtype}"), cfg, held)
            truth = {rid: plain.forward(cfg, exact, toks) for rid, toks in sequences(cfg["vocab"]).items()}
            out[which, dtype] = (folder, truth)
    return out


@pytest.mark.parametrize("trace", sorted(TRACES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(nm.CONFIGS))
def test_every_cutting_matches_the_plain_model(made, which, dtype, trace):
    """Whole prompts, a decoded tail, portions down to two tokens, and up to four requests at once over a pool that
    only holds what is live (pages and slots are used again; freed pages are filled with NaN)."""
    folder, truth = made[which, dtype]
    seqs = sequences(nm.CONFIGS[which]["vocab"])
    steps = TRACES[trace](seqs)
    rows = replay(folder, dtype, steps, max_live=4 if trace == "mixed" else 64)
    assert len(rows) == sum(len(t) for t in seqs.values())
    assert worst_error(rows, truth) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [1, 4, 64])
def test_token_by_token_through_small_and_large_pages(made, dtype, page_size):
    """Every token decoded alone, far beyond every window (4, 19 and 33 tokens) and over many page borders."""
    folder, truth = made["mixed", dtype]
    seqs = {rid: toks for rid, toks in sequences(131).items() if len(toks) in (2, 140)}
    steps = helpers.trace_tail_decode(seqs, tail=10 ** 6)
    rows = replay(folder, dtype, steps, page_size=page_size, max_tokens=helpers.peak_tokens(steps, page=max(page_size, 64)))
    assert worst_error(rows, truth) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_slots_and_an_exact_pool_serve_six_requests(made, dtype):
    folder, truth = made["mixed", dtype]
    seqs = sequences(131)
    steps = helpers.trace_mixed(seqs, max_live=2, seed=7)
    rows = replay(folder, dtype, steps, max_live=2, page_size=4, max_tokens=helpers.peak_tokens(steps, page=4))
    assert worst_error(rows, truth) < LIMIT[dtype]


def test_a_batch_gives_each_request_what_it_gets_alone(made):
    """float32: the same kernels run either way, so the rows agree to the last bits, not only within the limit."""
    folder, _ = made["mixed", "float32"]
    seqs = sequences(131)
    together = replay(folder, "float32", helpers.trace_mixed(seqs, max_live=4, seed=3), max_live=4)
    alone = replay(folder, "float32", helpers.trace_whole(seqs))
    for key, row in alone.items():
        assert row_error(together[key], row) < 2e-6


# ---- keys that must not be lost --------------------------------------------------------------------------------

def loud_key_model(dtype, window):
    """One attention layer in which a marked token's rotated key part is huge, so that whoever sees it attends to it
    almost alone (for the heads whose query points its way) and whoever does not, does not."""
    cfg = nm.config([nm.layer("latent_attention", nm.attention(heads=4, dim=8, rot_dim=8, vdim=8, q_rank=16, kv_rank=16,
                                                                scale=0.5, window=window, base=1e6), 32)], vocab=64, width=32)
    weights = nm.tensors(cfg, seed=11)
    weights["embed"][63] *= 8.0   # the key/value latent is normed, the rotated key part is not: it grows with the row
    return cfg, *stored(weights, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("place", ["first", "page_last", "page_first", "window_edge"])
def test_a_loud_key_is_seen_exactly_where_the_window_says(tmp_path, dtype, place):
    window, n = 40, 110
    marked = {"first": 0, "page_last": 63, "page_first": 64, "window_edge": 44}[place]
    cfg, held, exact = loud_key_model(dtype, window)
    folder = nm.write_folder(tmp_path / "m", cfg, held)
    toks = helpers.random_tokens(63, n, seed=5)
    toks[marked] = 63
    truth = {"a": plain.forward(cfg, exact, toks)}
    quiet = list(toks)
    quiet[marked] = 1
    hidden = plain.forward(cfg, exact, quiet)
    # the oracle itself says the marked key matters inside the window and not beyond it
    inside, outside = marked + window - 1, marked + window + 1
    seen = [row_error(truth["a"][i].numpy(), hidden[i].numpy()) for i in range(marked + 1, min(n, marked + window))]
    assert max(seen) > 0.15 and seen[-1] > 1e-4
    if outside < n:
        assert row_error(truth["a"][outside].numpy(), hidden[outside].numpy()) < 1e-9
    seqs = {"a": toks}
    for steps in (helpers.trace_whole(seqs), helpers.trace_tail_decode(seqs, tail=60), helpers.trace_portions(seqs, sizes=(3, 2, 40, 7, 2, 31))):
        rows = replay(folder, dtype, steps)
        assert worst_error(rows, truth) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_loud_key_far_back_without_a_window(tmp_path, dtype):
    cfg, held, exact = loud_key_model(dtype, None)
    folder = nm.write_folder(tmp_path / "m", cfg, held)
    toks = helpers.random_tokens(63, 330, seed=6)
    toks[3] = 63
    truth = {"a": plain.forward(cfg, exact, toks)}
    seqs = {"a": toks}
    for steps in (helpers.trace_tail_decode(seqs, tail=40), helpers.trace_portions(seqs, sizes=(100, 2, 64, 33))):
        rows = replay(folder, dtype, steps)
        assert worst_error(rows, truth) < LIMIT[dtype]


@pytest.mark.parametrize("window, heads", [(300, 2), (None, 3)])
def test_single_tokens_whose_keys_several_blocks_share(tmp_path, window, heads):
    """bfloat16 rows in multiples of eight with hundreds of visible keys: the blocks of a (token, head) split the keys
    among them and a second kernel joins their shares; two heads share a block where the head count is even."""
    cfg = nm.config([nm.layer("latent_attention", nm.attention(heads=heads, dim=16, rot_dim=8, vdim=16, q_rank=32, kv_rank=24,
                                                                scale=0.3, window=window, base=1e4), 48)], vocab=96, width=64)
    held, exact = stored(nm.tensors(cfg, seed=31), "bfloat16")
    folder = nm.write_folder(tmp_path / "m", cfg, held)
    seqs = {"a": helpers.random_tokens(96, 420, seed=8), "b": helpers.random_tokens(96, 150, seed=9)}
    truth = {rid: plain.forward(cfg, exact, toks) for rid, toks in seqs.items()}
    from prefixserve_b200.ops import library
    before = library.launch_counts.copy()
    rows = replay(folder, "bfloat16", helpers.trace_tail_decode(seqs, tail=100))
    assert worst_error(rows, truth) < LIMIT["bfloat16"]
    rows = replay(folder, "bfloat16", helpers.trace_mixed(seqs, max_live=2, seed=2))
    assert worst_error(rows, truth) < LIMIT["bfloat16"]
    assert (library.launch_counts - before)["latent_attention"] > 0


def test_a_long_memory_survives_portions_and_decoding(tmp_path):
    """A recurrence that forgets slowly: a lost state or a lost convolution input at a portion's start shows for long."""
    cfg = nm.CONFIGS["rec_only"]
    weights = nm.tensors(cfg, seed=21)
    weights["l0.mix.lam"] -= 4.0   # a close to one
    held, exact = stored(weights, "float32")
    folder = nm.write_folder(tmp_path / "m", cfg, held)
    seqs = sequences(cfg["vocab"], lengths=[3, 64, 200], seed=40)
    truth = {rid: plain.forward(cfg, exact, toks) for rid, toks in seqs.items()}
    for steps in (helpers.trace_portions(seqs, sizes=(2, 2, 3, 1, 2, 50, 2)), helpers.trace_tail_decode(seqs, tail=150),
                  helpers.trace_mixed(seqs, max_live=3, seed=1)):
        assert worst_error(replay(folder, "float32", steps), truth) < LIMIT["float32"]


# ---- mechanisms alone -------------------------------------------------------------------------------------------

def test_hashed_pair_embedding_alone():
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(0)
    table, pair = torch.randn(50, 24, generator=g), torch.randn(38, 24, generator=g)   # 37 buckets and the first-token row
    # three portions: a sequence's start, a continuation whose previous token is in the slot, a single token
    ids = [4, 9, 9, 30, 2, 49, 7]
    item_of = [0, 0, 0, 1, 1, 1, 2]
    starts, positions = [0, 3, 6, 7], [0, 1, 2, 10, 11, 12, 5]
    slots, last = [2, 0, 3], torch.tensor([17, -1, -1, 41], dtype=torch.int32).cuda()
    dev = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    h, copy = ops.hashed_embedding(dev(ids), dev(positions), dev(item_of), dev(starts), dev(slots), last, table.cuda(), pair.cuda(),
                                   mul_prev=1000003, mul_cur=911, copy_dtype=torch.bfloat16)
    prev = [None, 4, 9, 17, 30, 2, 41]
    for t, (tok, p) in enumerate(zip(ids, prev)):
        row = 37 if p is None else (p * 1000003 + tok * 911) % 37
        assert torch.equal(h[t].cpu(), table[tok] + pair[row])
    assert torch.equal(copy.cpu(), h.cpu().to(torch.bfloat16))
    assert last.tolist() == [49, -1, 9, 7]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_norm_add_and_activation_alone(dtype):
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(1)
    h, y, gate = torch.randn(5, 40, generator=g), torch.randn(5, 40, generator=g).to(dtype), torch.randn(5, 40, generator=g).to(dtype)
    bias, gain = torch.randn(40, generator=g), 1 + 0.1 * torch.randn(40, generator=g)
    want = h.double() + 0.45 * plain.plain_norm(y.double() * torch.sigmoid(gate.double() + bias.double()), gain.double(), 3e-6)
    hd = h.cuda()
    copy = ops.gated_norm_add(hd, y.cuda(), gate.cuda(), bias.cuda(), gain.cuda(), 3e-6, 0.45, dtype)
    assert torch.allclose(hd.cpu().double(), want, atol=1e-5)
    assert (copy is None) == (dtype == torch.float32)
    if copy is not None:
        assert torch.equal(copy.cpu(), hd.cpu().to(dtype))
    z = (3 * torch.randn(1000, generator=g)).to(dtype)
    pq = torch.tensor([0.3, -0.7])
    got = ops.activation(z.cuda(), "xielu", pq.cuda()).cpu().double()
    want = plain.xielu(z.double(), pq[0].double(), pq[1].double())
    assert torch.allclose(got, want, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-2 if dtype == torch.bfloat16 else 1e-6)


def test_per_head_product_on_slices_of_wider_tensors():
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(2)
    a = torch.randn(70, 3, 11, generator=g).cuda()      # heads of 11, of which the first 7 are multiplied
    w = torch.randn(3, 5, 7, generator=g).cuda()
    out = torch.zeros(70, 3, 9, device="cuda")
    ops.linear_per_head(a[:, :, :7], w, out=out[:, :, :5])
    want = torch.einsum("thk,hnk->thn", a[:, :, :7].double(), w.double())
    assert torch.allclose(out[:, :, :5].double(), want, atol=1e-5) and float(out[:, :, 5:].abs().max()) == 0.0


@pytest.mark.parametrize("m", [1, 8, 9, 33, 64, 65, 127, 128, 300, 1100])
def test_products_with_the_output_widths_this_design_brings(m):
    """The fused input projections have output widths such as q_rank + kv_rank + rot_dim + heads, which are multiples
    of nothing; every route of ``ops.linear`` (few rows, a few dozen, the tensor-core tiles, the library) takes them."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(m)
    for k, n in [(64, 6), (96, 294), (512, 1900), (512, 2047), (72, 100), (100, 37), (256, 4098)]:
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16).cuda()
        got = ops.linear(x, w).float().cpu()
        want = (x.double() @ w.double().T).cpu()
        assert got.shape == (m, n)
        assert float((got.double() - want).abs().max()) < 0.03 * max(1.0, float(want.abs().max())), (m, k, n)
    from prefixserve_b200.ops import library
    assert library.tcgen05_status() == 0


# ---- generation through the scheduler --------------------------------------------------------------------------

def greedy(cfg, exact, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain.forward(cfg, exact, toks)[-1].argmax()))
    return toks[len(prompt):]


def test_greedy_generation_through_the_entry_point_and_scheduler(made):
    """Prompts longer than a portion, more requests than run at once, captured decode steps: the same tokens as the
    plain model's greedy continuation (float32: a tie would have to be exact to differ)."""
    from prefixserve_b200.engine.llm import LLM
    from prefixserve_b200.sampling import SamplingParams
    folder, _ = made["mixed", "float32"]
    cfg = nm.CONFIGS["mixed"]
    _, exact = stored(nm.tensors(cfg, seed=sorted(nm.CONFIGS).index("mixed")), "float32")
    prompts = [helpers.random_tokens(131, n, seed=70 + n) for n in (1, 5, 23, 40)]
    llm = LLM(folder, dtype="float32", max_seq_len=128, num_blocks=64, max_running_requests=3, chunked_prefill_size=16)
    got = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert got == [greedy(cfg, exact, p, 12) for p in prompts]
    assert llm.engine.runner.graph_replays > 0
    llm.engine.cache.check()
    # a second call on the same engine starts from clean slots
    assert llm.generate(prompts[:2], SamplingParams(max_tokens=5, ignore_eos=True)) == [greedy(cfg, exact, p, 5) for p in prompts[:2]]


def test_command_line_generates_from_a_nerenex_folder(made):
    import json
    import subprocess
    import sys
    folder, _ = made["attn_ff", "bfloat16"]
    out = subprocess.run([sys.executable, "-m", "prefixserve_b200", "--model", str(folder), "--prompt-ids", "5,17,3", "--max-tokens", "6",
                          "--num-blocks", "32", "--max-seq-len", "64", "--max-running-requests", "2"],
                         capture_output=True, text=True, timeout=600, cwd=str(helpers.__file__).rsplit("/tests/", 1)[0])
    assert out.returncode == 0, out.stderr[-2000:]
    first = json.loads(out.stdout.splitlines()[0])
    assert first["prompt_ids"] == [5, 17, 3] and len(first["output_ids"]) == 6
