"""Tazadra on the GPU against the plain implementation: every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, unequal batches
against each request alone, slots and pages used again, keys far away, at page borders and
on both sides of a chunk's edge with attention made sharp, the first tokens, long
decoding, other sizes, greedy generation through the Python entry point, and the replay
program."""
import json
import os
import random
import subprocess

import numpy as np
import pytest
import torch

import plain_tazadra as P
from helpers import TraceBuilder, check_logits, random_tokens, read_step, three_cuts
from tazadra_models import CONFIGS, load_weights, make_model, read_config

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: make_model(str(tmp_path_factory.mktemp(f"tazadra_{name}")), cfg, seed=500 + i)
            for i, (name, cfg) in enumerate(CONFIGS.items())}


_engines, _plain = {}, {}


def engine_for(models, name, dtype):
    from nnis_b200.engine import Engine
    if (name, dtype) not in _engines:
        _engines[(name, dtype)] = Engine.from_dir(models[name], dtype=dtype, max_tokens=64 * 64)
    return _engines[(name, dtype)]


# A router's close call may go either way under bfloat16 rounding, and the token then runs
# another expert: in bfloat16 a position is compared only where every router of the plain
# implementation chose with at least this gap between the last score in and the first out.
# An earlier position's other expert still reaches later ones through the recurrent layers
# and the keys, so in bfloat16 a model with routers is held to the bound by three rows in four
# of those compared (a fault of a kernel moves nearly every row) (float32 holds it everywhere; so does bfloat16 on models without routers).
CLOSE_CALL = 0.005


def _plain_run(models, name, dtype, tokens):
    key = (name, dtype, tuple(tokens))
    if key not in _plain:
        bf = dtype == "bfloat16"
        margins = []
        logits = P.forward(read_config(models[name]), load_weights(models[name], bf), tokens, emulate_bf16=bf,
                           margins=margins)
        gap = torch.stack(margins).min(dim=0).values if margins else torch.full((len(tokens),), float("inf"))
        _plain[key] = (logits, gap, bool(margins))
    return _plain[key]


def plain_logits(models, name, dtype, tokens):
    return _plain_run(models, name, dtype, tokens)[0]


def clear_calls(models, name, dtype, tokens):
    gap = _plain_run(models, name, dtype, tokens)[1]
    return torch.ones_like(gap, dtype=torch.bool) if dtype == "float32" else gap >= CLOSE_CALL


def replay_and_check(models, name, dtype, trace, sequences, tmp_path, what, most_skipped=0.5):
    from nnis_b200.engine.replay import replay
    engine = engine_for(models, name, dtype)
    out = str(tmp_path / f"out_{name}_{dtype}")
    replay(engine, trace.lines, out)
    usage = engine.cache.usage()
    assert usage["slots_held"] == 0 and not any(usage["pages_held"]), usage
    engine.cache.check()
    vocab = read_config(models[name])["vocab"]
    compared = skipped = missed = 0
    for step, rows in trace.rows.items():
        got = read_step(out, step, vocab)
        assert got.shape[0] == len(rows) and np.isfinite(got).all()
        keep = [j for j, (rid, pos) in enumerate(rows) if bool(clear_calls(models, name, dtype, sequences[rid])[pos])]
        compared, skipped = compared + len(keep), skipped + len(rows) - len(keep)
        if not keep:
            continue
        want = torch.stack([plain_logits(models, name, dtype, sequences[rows[j][0]])[rows[j][1]] for j in keep])
        routed = _plain_run(models, name, dtype, sequences[rows[0][0]])[2]
        if dtype == "float32" or not routed:
            check_logits(got[keep], want, dtype, f"{what} {name} {dtype} step {step}")
        else:
            missed += rows_beyond_the_bound(got[keep], want)
    assert skipped <= most_skipped * (compared + skipped), (compared, skipped)
    assert missed <= 0.25 * compared, (what, name, dtype, missed, compared)


def rows_beyond_the_bound(got, want, rel=0.03):
    want = want.float().numpy()
    scale = max(1.0, float(np.abs(want).max()))
    return int((np.abs(got - want).max(axis=1) > rel * scale).sum())


def run_whole(engine, tokens, want=None):
    from nnis_b200.engine import SequenceStep
    slot = engine.acquire_slot()
    try:
        return engine.step([SequenceStep(slot, tokens, list(range(len(tokens))) if want is None else want)]).cpu().numpy()
    finally:
        engine.release_slot(slot)


# ---- row-wise kernels against plain float32 torch ------------------------------------------
def test_norm_on_a_branch_activations_and_the_soft_cap():
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    for n, width in ((37, 90), (1, 7), (5, 1000)):
        branch, hidden, w = (torch.randn(n, width, generator=g) * 3, torch.randn(n, width, generator=g),
                             torch.randn(width, generator=g))
        want = hidden.double() + 0.7 * P.rms_norm(branch.double(), w.double(), 1e-5)
        for dtype in (torch.float32, torch.bfloat16):
            h = hidden.to(dev).clone()
            out = torch.empty(n, width, dtype=dtype, device=dev)
            b = branch.to(dev)
            ops.norm_scale_add(b, w.to(dev), 1e-5, 0.7, h, out)
            assert torch.allclose(h.cpu().double(), want, atol=2e-5, rtol=1e-5)
            assert torch.equal(out.cpu(), h.cpu().to(dtype)) and torch.equal(b.cpu(), branch)
            h2 = hidden.to(dev).clone()
            ops.norm_scale_add(b, w.to(dev), 1e-5, 0.7, h2, None, clear=True)  # the buffer is left zero
            assert torch.equal(h2, h) and float(b.abs().max()) == 0.0
        x = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
        ops.cast_rows(hidden.to(dev), x)
        assert torch.equal(x.cpu(), hidden.to(torch.bfloat16))
    gu = torch.randn(19, 2 * 33, generator=g) * 3
    out = torch.empty(19, 33, dtype=torch.float32, device=dev)
    ops.glu_clamp(gu.to(dev), out, 2.0, 1.702)
    gate, up = gu[:, :33].double().clamp(max=2.0), gu[:, 33:].double().clamp(-2.0, 2.0)
    assert torch.allclose(out.cpu().double(), gate * torch.sigmoid(1.702 * gate) * (up + 1), atol=1e-5)
    assert float((gu[:, :33] > 2.0).float().mean()) > 0.1 and float((gu[:, 33:] < -2.0).float().mean()) > 0.1
    logits = (torch.randn(4, 50, generator=g) * 40).to(dev)
    want = 30.0 * torch.tanh(logits.cpu().double() / 30.0)
    ops.softcap_rows(logits, 30.0)
    assert torch.allclose(logits.cpu().double(), want, atol=1e-4)
    t = torch.empty(4, 50, dtype=torch.float32, device=dev)
    ops.tanh_rows(torch.linspace(-5, 5, 200).reshape(4, 50).to(dev), t)
    assert torch.allclose(t.cpu().flatten(), torch.tanh(torch.linspace(-5, 5, 200)), atol=1e-6)


def test_scaled_frequencies_follow_the_three_ranges():
    from nnis_b200.parts import POSITIONS
    for rot in ({"dims": 32, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
                {"dims": 6, "base": 3.0}, {"dims": 0, "base": 10.0},
                {"dims": 64, "base": 500000.0, "scaling": {"factor": 2.5, "low": 0.5, "high": 3.0, "original": 2048}}):
        part = POSITIONS.build("rope_frequencies", {**rot, "pairing": "neighbours"}, "", torch.float32, "cuda:0")
        got = part.frequencies().cpu()[:rot["dims"] // 2].double()
        want = P.frequencies(rot)
        assert torch.allclose(got, want, rtol=1e-6, atol=0)
    f = P.frequencies({"dims": 32, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}})
    plain = P.frequencies({"dims": 32, "base": 10000.0})
    ratio = (plain / f)
    assert float(ratio[0]) == 1.0 and abs(float(ratio[-1]) - 8.0) < 1e-9 and bool(((ratio > 1.001) & (ratio < 7.999)).any())


# ---- whole models ------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention", "heads64", "wkv", "wide_wkv", "mamba", "wide_mamba", "dense", "moe"])
def test_each_mechanism_alone(models, name, dtype, tmp_path):
    rng = random.Random(11)
    vocab = read_config(models[name])["vocab"]
    sequences, trace = {}, TraceBuilder()
    # the first tokens, a page's border, a chunk's edge, more tokens than a tile of the scans
    for i, n in enumerate((1, 2, 3, 50, 51, 64, 65, 131, 300)):
        sequences[f"w{i}"] = random_tokens(rng, n, vocab)
        trace.step([(f"w{i}", sequences[f"w{i}"], range(n))], end=[f"w{i}"])
    toks = sequences["d"] = random_tokens(rng, 75, vocab)  # decoding from the second token on
    trace.step([("d", toks[:1], [0])])
    for t in range(1, 75):
        trace.step([("d", toks[t:t + 1], [0])], end=["d"] if t == 74 else [])
    replay_and_check(models, name, dtype, trace, sequences, tmp_path, "alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd", "heads64"])
def test_whole_last_tokens_and_unequal_batches(models, name, dtype, tmp_path):
    vocab = read_config(models[name])["vocab"]
    trace, sequences = three_cuts(random.Random(3), vocab)
    replay_and_check(models, name, dtype, trace, sequences, tmp_path, "three cuts")


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_portions_batches_and_reuse_agree_with_each_request_alone(models, name):
    """float32: the same position's logits whatever the cut, the batch, the slot or the pages."""
    from nnis_b200.engine import SequenceStep
    engine = engine_for(models, name, "float32")
    vocab = read_config(models[name])["vocab"]
    rng = random.Random(9)
    prompts = [random_tokens(rng, n, vocab) for n in (200, 3, 67, 130)]
    alone = [run_whole(engine, p) for p in prompts]
    scale = max(float(np.abs(a).max()) for a in alone)
    for p, a in zip(prompts, alone):
        check_logits(a, plain_logits(models, name, "float32", p), "float32", "alone")
    # portions of several sizes, down to two tokens and one
    for cuts in ([2, 2, 60, 1, 64, 71], [64, 64, 64, 8], [199, 1], [1, 199], [39, 2, 7, 152], [3, 17, 16, 164]):
        slot = engine.acquire_slot()
        rows, at = [], 0
        for c in cuts:
            rows.append(engine.step([SequenceStep(slot, prompts[0][at:at + c], list(range(c)))]).cpu().numpy())
            at += c
        engine.release_slot(slot)
        assert at == 200 and np.abs(np.concatenate(rows) - alone[0]).max() < 3e-5 * scale, cuts
    # one batch of all four, then the same again in slots and pages that were used before
    for _ in range(2):
        slots = [engine.acquire_slot() for _ in prompts]
        heads = [max(1, len(p) - 20) for p in prompts]
        got = engine.step([SequenceStep(s, p[:h], list(range(h))) for s, p, h in zip(slots, prompts, heads)]).cpu().numpy()
        at = 0
        for i, h in enumerate(heads):
            assert np.abs(got[at:at + h] - alone[i][:h]).max() < 3e-5 * scale
            at += h
        live = list(range(len(prompts)))
        step = 0
        while live:  # decoded together; the shorter ones end earlier
            batch = [SequenceStep(slots[i], prompts[i][heads[i] + step:heads[i] + step + 1], [0]) for i in live]
            got = engine.step(batch).cpu().numpy()
            for r, i in enumerate(live):
                assert np.abs(got[r] - alone[i][heads[i] + step]).max() < 3e-5 * scale, (i, step)
            step += 1
            for i in list(live):
                if heads[i] + step == len(prompts[i]):
                    engine.release_slot(slots[i])
                    live.remove(i)
    assert engine.cache.usage()["slots_held"] == 0
    engine.cache.check()


def test_a_slot_used_again_starts_from_nothing(models):
    """The recurrent layers' state and the convolution's last inputs are zero when a slot is
    taken again, whatever its last owner left; a snapshot brings a sequence back."""
    from nnis_b200.engine import SequenceStep
    engine = engine_for(models, "mixed", "float32")
    vocab = read_config(models["mixed"])["vocab"]
    rng = random.Random(2)
    a, b = random_tokens(rng, 90, vocab), random_tokens(rng, 33, vocab)
    want = run_whole(engine, b)
    slot = engine.acquire_slot()
    engine.step([SequenceStep(slot, a, [])])
    engine.release_slot(slot)
    again = engine.acquire_slot()
    assert again == slot
    got = engine.step([SequenceStep(again, b[:20], list(range(20)))]).cpu().numpy()
    kept = engine.snapshot(again)
    rest = engine.step([SequenceStep(again, b[20:], list(range(13)))]).cpu().numpy()
    assert np.abs(np.concatenate([got, rest]) - want).max() < 3e-5 * np.abs(want).max()
    engine.step([SequenceStep(again, a[:5], [])])
    engine.restore(kept)
    rest = engine.step([SequenceStep(again, b[20:], list(range(13)))]).cpu().numpy()
    assert np.abs(rest - want[20:]).max() < 3e-5 * np.abs(want).max()
    engine.release_slot(again)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_shape_that_recurs_is_captured_and_replayed(models, dtype):
    """A large prompt step whose shape comes a second time is recorded as a CUDA graph and replayed from
    the third time on: the recurrent layers' states, the runs' tables and the branch buffers must all
    live where the graph expects them.  Other tokens every time, the same shape."""
    from nnis_b200.engine import Engine, SequenceStep
    engine = Engine.from_dir(models["mixed"], dtype=dtype, max_tokens=64 * 64)
    vocab = read_config(models["mixed"])["vocab"]
    rng = random.Random(77)
    graphs = []
    for round_ in range(4):
        a, b = random_tokens(rng, 300, vocab), random_tokens(rng, 40, vocab)
        slots = [engine.acquire_slot(), engine.acquire_slot()]
        got = engine.step([SequenceStep(slots[0], a[:290], [0, 150, 289]), SequenceStep(slots[1], b[:30], [29])]).cpu().numpy()
        more = engine.step([SequenceStep(slots[0], a[290:291], [0]), SequenceStep(slots[1], b[30:31], [0])]).cpu().numpy()
        for s_ in slots:
            engine.release_slot(s_)
        graphs.append(len(engine._step_graphs))
        keep_a, keep_b = clear_calls(models, "mixed", dtype, a), clear_calls(models, "mixed", dtype, b)
        rows = [(a, 0, got[0], keep_a), (a, 150, got[1], keep_a), (a, 289, got[2], keep_a), (b, 29, got[3], keep_b),
                (a, 290, more[0], keep_a), (b, 30, more[1], keep_b)]
        missed = 0
        for toks, pos, row, keep in rows:
            if not bool(keep[pos]):
                continue
            want = plain_logits(models, "mixed", dtype, toks)[pos][None, :]
            if dtype == "float32":
                check_logits(row[None, :], want, dtype, f"captured step, round {round_}, position {pos}")
            else:
                missed += rows_beyond_the_bound(row[None, :], want)
        assert missed <= 2, (round_, missed)
    assert graphs == [0, 1, 1, 1], graphs


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_page_and_chunk_borders(models, dtype, tmp_path):
    vocab = read_config(models["mixed"])["vocab"]
    toks = random_tokens(random.Random(21), 5 + 200, vocab)
    trace = TraceBuilder()
    trace.step([("a", toks[:5], [4])])
    for t in range(5, len(toks)):
        trace.step([("a", toks[t:t + 1], [0])], end=["a"] if t == len(toks) - 1 else [])
    replay_and_check(models, "mixed", dtype, trace, {"a": toks}, tmp_path, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["wkv", "wide_wkv", "mamba", "wide_mamba", "mixed"])
def test_long_prompts_of_the_recurrent_mixers_in_runs_and_portions(models, name, dtype, tmp_path):
    """Prompts longer than two runs of the scans (runs are worked side by side and put together
    afterwards), alone, in a batch with short ones, continued after a first portion, and decoded on: a
    state lost or joined wrongly at a run's edge shows, since the slowest channels forget next to
    nothing over hundreds of tokens."""
    vocab = read_config(models[name])["vocab"]
    rng = random.Random(31)
    a, b, c = (random_tokens(rng, n, vocab) for n in (700, 257, 40))
    trace = TraceBuilder()
    trace.step([("a", a[:690], [0, 63, 64, 65, 127, 128, 129, 511, 512, 689])])
    for t in range(690, 700):
        trace.step([("a", a[t:t + 1], [0])], end=["a"] if t == 699 else [])
    trace.step([("b", b[:100], [99]), ("c", c[:39], [38])])          # a first portion, then runs after it
    trace.step([("b", b[100:], list(range(150, 157))), ("c", c[39:], [0])], end=["b", "c"])
    trace.step([("a2", a, [256, 600, 699]), ("c2", c, [39]), ("b2", b, [255, 256])], end=["a2", "c2", "b2"])
    replay_and_check(models, name, dtype, trace, {"a": a, "b": b, "c": c, "a2": a, "c2": c, "b2": b}, tmp_path,
                     "runs")


def test_far_keys_page_borders_chunk_edges_and_the_sink_with_sharp_attention(models, tmp_path):
    """Scores times a large scale and no cap: most of a query's weight lies on one key, and
    the plain implementation says which.  Among those keys are far ones, ones on both sides
    of page borders and the first ones of a chunk; queries just past a chunk's edge must not
    see the key they would prefer, and queries whose sink outweighs every key show a sink
    that is left out.  Both layers read the same keys under chunks of different sizes."""
    cfg = read_config(models["sharp"])
    toks = random_tokens(random.Random(8), 420, cfg["vocab"])
    probes = {}
    P.forward(cfg, load_weights(models["sharp"], False), toks, probes=probes)
    for layer, chunk in ((0, 192), (1, 70)):
        weights = torch.stack(probes[layer]["weights"])  # [heads, T, T]
        sink = torch.stack(probes[layer]["sink"])  # [heads, T]
        top, arg = weights.max(dim=-1)
        queries = torch.arange(420)[None, :].expand_as(arg)
        strong = top > 0.5
        assert int(strong.sum()) > 150, int(strong.sum())
        distance = (queries - arg)[strong]
        assert int((distance > 0.6 * chunk).sum()) >= 5
        assert int(((arg % chunk) == 0)[strong & (queries > arg)].sum()) >= 1  # a chunk's first key, from later on
        assert bool((weights[:, chunk, :chunk] == 0).all()) and bool((weights[:, chunk - 1, 0] > 0).all())
        assert int((sink > 0.3).sum()) >= 10
        if chunk > 64:
            in_page = (arg % 64)[strong & (queries // 64 != arg // 64)]
            assert int((in_page == 63).sum()) >= 1 and int((in_page == 0).sum()) >= 1
    trace = TraceBuilder()
    trace.step([("w", toks, range(420))], end=["w"])
    trace.step([("d", toks[:150], range(150))])
    for t in range(150, 300):  # decoding over the edges at 192 and 210, 280
        trace.step([("d", toks[t:t + 1], [0])])
    trace.step([("d", toks[300:], range(120))], end=["d"])  # and a later portion that starts inside a chunk
    for dtype in DTYPES:
        replay_and_check(models, "sharp", dtype, trace, {"w": toks, "d": toks}, tmp_path, "sharp")


def _random_config(rng):
    """Sizes, layer order, heads, experts and constants drawn at random (small ones)."""
    from tazadra_models import attention, config, dense, layer, mamba, moe, wkv
    width = rng.choice([8, 24, 36, 40, 64, 72, 100, 128])
    layers, sources = [], []
    for i in range(rng.randint(1, 6)):
        r = rng.random()
        if r < 0.4:
            if sources and rng.random() < 0.4:
                j = rng.choice(sources)
                src = layers[j]["mixer"]
                heads = src["kv_heads"] * rng.randint(1, 3)
                mixer = attention(heads, src["kv_heads"], src["dim"], src["vdim"], src["rot"]["dims"],
                                  rng.choice([0.1, 0.25, 1.0]), base=src["rot"]["base"],
                                  scaling=tuple(src["rot"]["scaling"].values()) if "scaling" in src["rot"] else None,
                                  softcap=rng.choice([None, 8.0, 50.0]), chunk=rng.choice([None, 1, 5, 33, 64, 100]),
                                  kv_from=j)
            else:
                kv = rng.randint(1, 3)
                dim = 2 * rng.randint(1, 40)
                mixer = attention(kv * rng.randint(1, 4), kv, dim, rng.randint(1, 70),
                                  2 * rng.randint(0, dim // 2), rng.choice([0.1, 0.25, 1.0]),
                                  base=rng.choice([10.0, 10000.0, 1e6]),
                                  scaling=rng.choice([None, (8.0, 1.0, 4.0, 64), (3.0, 0.25, 2.0, 16)]),
                                  softcap=rng.choice([None, 8.0, 50.0]), chunk=rng.choice([None, 2, 5, 33, 64, 100]))
                sources.append(i)
        elif r < 0.7:
            mixer = wkv(rng.randint(1, 4), rng.choice([1, 3, 8, 16, 24, 32, 48, 64, 100, 128]), rng.randint(1, 20))
        else:
            mixer = mamba(rng.choice([8, 20, 64, 130, 200]), rng.choice([1, 4, 8, 16, 24, 33, 64]), rng.randint(1, 12),
                          rng.randint(1, 5))
        r = rng.random()
        if r < 0.2:
            ff = None
        elif r < 0.5:
            ff = dense(rng.choice([8, 16, 40, 64, 96, 136]), rng.choice([0.5, 2.0, 7.0]))
        else:
            experts = rng.randint(1, 12)
            ff = moe(experts, rng.randint(1, experts), rng.choice([8, 12, 16, 24, 40, 64]))
        layers.append(layer(mixer, ff))
    return config(rng.choice([50, 131, 256, 577]), width, rng.choice([1e-5, 1e-6]), rng.choice([0.25, 0.5, 1.0, 1.5]),
                  rng.choice([None, 10.0, 30.0]), layers)


@pytest.mark.parametrize("trial", range(10))
def test_configurations_drawn_at_random(trial, tmp_path):
    """A prompt in one step, a second portion and six tokens one by one, both dtypes, on a model
    whose sizes, layer order and constants are drawn at random: whatever kernels the sizes select."""
    from nnis_b200.engine import Engine, SequenceStep
    rng = random.Random(7000 + trial)
    cfg = _random_config(rng)
    d = make_model(str(tmp_path / "m"), cfg, seed=trial)
    toks = random_tokens(rng, 150, cfg["vocab"])
    for dtype in DTYPES:
        bf = dtype == "bfloat16"
        margins = []
        want = P.forward(cfg, load_weights(d, bf), toks, emulate_bf16=bf, margins=margins)
        gap = torch.stack(margins).min(dim=0).values if margins else torch.full((len(toks),), float("inf"))
        engine = Engine.from_dir(d, dtype=dtype, max_tokens=1024)
        slot = engine.acquire_slot()
        got = [engine.step([SequenceStep(slot, toks[:101], list(range(101)))]).cpu().numpy(),
               engine.step([SequenceStep(slot, toks[101:144], list(range(43)))]).cpu().numpy()]
        for t in range(144, 150):
            got.append(engine.step([SequenceStep(slot, toks[t:t + 1], [0])]).cpu().numpy())
        engine.release_slot(slot)
        engine.check_status()
        got = np.concatenate(got)
        what = f"random configuration {trial} {dtype}: {json.dumps(cfg)}"
        keep = (gap >= (CLOSE_CALL if bf else 1e-6)).numpy()
        assert np.isfinite(got).all(), what
        if not keep.any():
            continue
        if bf and margins:
            assert rows_beyond_the_bound(got[keep], want[torch.from_numpy(keep)]) <= 0.25 * keep.sum(), what
        else:
            check_logits(got[keep], want[torch.from_numpy(keep)], dtype, what)


def _middle_config(rng):
    """Sizes of a small real model (widths of a few hundred, heads of 32 to 128, a few thousand
    vocabulary entries): the shapes at which the tensor-core products, the decode projections
    over tiles of rows and the tensor-core attention take over from the any-size kernels."""
    from tazadra_models import attention, config, dense, layer, mamba, moe, wkv
    width = rng.choice([192, 256, 320, 384, 512])
    dim = rng.choice([32, 64, 128])
    kv = rng.choice([1, 2, 4])
    heads = kv * rng.choice([1, 2, 3, 4])
    vdim = rng.choice([dim, dim, 32, 96])
    rot = rng.choice([dim, dim // 2])
    scaling = rng.choice([None, (8.0, 1.0, 4.0, 256), (4.0, 1.0, 2.0, 64)])
    att = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, rot_dims=rot, base=rng.choice([10000.0, 500000.0]),
               scaling=scaling)
    first = attention(scale=dim ** -0.5 * 4, softcap=rng.choice([None, 20.0, 50.0]), chunk=rng.choice([64, 100, 128]), **att)
    second = attention(scale=dim ** -0.5 * 4, softcap=rng.choice([None, 20.0]), chunk=rng.choice([None, 48, 128]),
                       kv_from=0, **{**att, "heads": kv * rng.choice([1, 2, 4])})
    recurrent = [wkv(rng.choice([2, 4, 8]), rng.choice([32, 64]), rng.choice([16, 32, 40])),
                 mamba(rng.choice([1, 2]) * width, rng.choice([8, 16, 24, 32]), rng.choice([8, 16, 24]), rng.choice([3, 4]))]
    ffs = [dense(rng.choice([384, 512, 768]), rng.choice([2.0, 7.0])),
           moe(rng.choice([4, 8, 16]), rng.choice([1, 2]), rng.choice([64, 96, 128]))]
    layers = [layer(first, rng.choice(ffs))]
    for _ in range(rng.randint(2, 4)):
        layers.append(layer(rng.choice(recurrent), rng.choice(ffs + [None])))
    layers.insert(rng.randint(2, len(layers)), layer(second, rng.choice(ffs)))
    return config(rng.choice([640, 1000, 2048, 4099]), width, 1e-6, rng.choice([0.5, 1.0]), rng.choice([None, 30.0]), layers)


@pytest.mark.parametrize("trial", range(6))
def test_middle_sizes_drawn_at_random(trial, tmp_path):
    """A batch of two prompts (one of them in two portions) and eight tokens decoded together, both
    dtypes, at sizes of a small real model."""
    from nnis_b200.engine import Engine, SequenceStep
    rng = random.Random(9100 + trial)
    cfg = _middle_config(rng)
    d = make_model(str(tmp_path / "m"), cfg, seed=40 + trial)
    a, b = random_tokens(rng, 208, cfg["vocab"]), random_tokens(rng, 77, cfg["vocab"])
    for dtype in DTYPES:
        bf = dtype == "bfloat16"
        want, keep = {}, {}
        for name, toks in (("a", a), ("b", b)):
            margins = []
            want[name] = P.forward(cfg, load_weights(d, bf), toks, emulate_bf16=bf, margins=margins)
            gap = torch.stack(margins).min(dim=0).values if margins else torch.full((len(toks),), float("inf"))
            keep[name] = (gap >= (CLOSE_CALL if bf else 1e-6)).numpy()
        engine = Engine.from_dir(d, dtype=dtype, max_tokens=2048)
        sa, sb = engine.acquire_slot(), engine.acquire_slot()
        rows = []  # (request, position, logits row)
        got = engine.step([SequenceStep(sa, a[:130], [0, 63, 64, 129]), SequenceStep(sb, b[:69], [0, 68])]).cpu().numpy()
        rows += [("a", p, got[i]) for i, p in enumerate([0, 63, 64, 129])] + [("b", 0, got[4]), ("b", 68, got[5])]
        got = engine.step([SequenceStep(sa, a[130:200], [0, 69])]).cpu().numpy()
        rows += [("a", 130, got[0]), ("a", 199, got[1])]
        for t in range(8):
            got = engine.step([SequenceStep(sa, a[200 + t:201 + t], [0]), SequenceStep(sb, b[69 + t:70 + t], [0])]).cpu().numpy()
            rows += [("a", 200 + t, got[0]), ("b", 69 + t, got[1])]
        engine.release_slot(sa)
        engine.release_slot(sb)
        engine.check_status()
        what = f"middle size {trial} {dtype}: {json.dumps(cfg)}"
        kept = [(r, p, row) for r, p, row in rows if keep[r][p]]
        assert len(kept) >= len(rows) // 4, what
        gotten = np.stack([row for _, _, row in kept])
        wanted = torch.stack([want[r][p] for r, p, _ in kept])
        assert np.isfinite(gotten).all(), what
        if bf and any(l["mlp"] and l["mlp"]["kind"] == "moe" for l in cfg["layers"]):
            assert rows_beyond_the_bound(gotten, wanted) <= 0.25 * len(kept), what
        else:
            check_logits(gotten, wanted, dtype, what)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(models, dtype):
    from nnis_b200 import LLM
    d = models["mixed"]
    cfg = read_config(d)
    bf = dtype == "bfloat16"
    w = load_weights(d, bf)
    llm = LLM(d, dtype=dtype, max_tokens=64 * 32, max_batch=3)
    prompts = [[5, 9, 1, 200, 33], [7], [100, 101, 102, 103, 104, 105, 106, 107, 108], [250, 3], [9] * 70]
    results = llm.generate(prompts, max_new_tokens=10, stop_token_ids=())
    for p, r in zip(prompts, results):
        assert r.ok and r.finish_reason == "length"
        if not bf:
            assert r.token_ids == P.greedy_generate(cfg, w, p, 10), (dtype, p)
        else:  # a bfloat16 near-tie may go either way: every pick must be (nearly) the plain best
            seq = list(p)
            for t in r.token_ids:
                logits = P.forward(cfg, w, seq, emulate_bf16=True)[-1]
                assert float(logits.max() - logits[t]) <= 0.05 * max(1.0, float(logits.abs().max())), (p, t)
                seq.append(t)
    # a session goes on from where generation left it, state and all
    session = llm.new_session()
    from nnis_b200 import GenerationConfig
    ids = session.generate(prompts[0], GenerationConfig(6))
    more = session.decode_one(17)
    if not bf:
        want = P.forward(cfg, w, prompts[0] + ids + [17])[-1]
        check_logits(np.asarray(more).reshape(1, -1), want[None, :], dtype, "session")
    assert llm.engine.cache.usage()["slots_held"] <= 1


def test_replay_program_runs_a_model_folder(models, tmp_path):
    cfg = read_config(models["odd"])
    toks = random_tokens(random.Random(4), 40, cfg["vocab"])
    trace = TraceBuilder()
    trace.step([("a", toks[:30], [0, 29]), ("b", toks[:7], [6])])
    trace.step([("a", toks[30:31], [0]), ("b", toks[7:8], [0])], end=["b"])
    trace.step([("a", toks[31:32], [])], end=["a"])
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", models["odd"], "--dtype", "float32",
                        "--out", out, "--max-tokens", "256"], input="\n".join(trace.lines) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "2.f32"))
    want = plain_logits(models, "odd", "float32", toks)
    check_logits(read_step(out, 0, cfg["vocab"]), torch.stack([want[0], want[29], want[6]]), "float32", "program")
    check_logits(read_step(out, 1, cfg["vocab"]), torch.stack([want[30], want[7]]), "float32", "program")
