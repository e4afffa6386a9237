"""The Vopedra design through the library's loader, cache, step function, scheduler and kernels,
against the plain implementation (tests/plain_vopedra.py) on small models whose weights the tests
make themselves."""
import numpy as np
import pytest
import torch

import plain_vopedra as pv
import vopedra_models as vm

pytestmark = pytest.mark.gpu

# the largest |difference| of a position's logits is bounded by TOL * max(1, max|reference|); in bfloat16
# (small widths, unit-gain random weights, up to seven layer runs) also the mean over positions by MEAN_TOL
TOL = {"float32": 3e-4, "bfloat16": 1e-1}
MEAN_TOL = {"float32": 1e-4, "bfloat16": 3e-2}
_REF = {}


def plain_logits(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _REF:
        cfg, t = pv.read_folder(folder)
        _REF[key] = pv.forward(cfg, t, list(tokens)).numpy()
    return _REF[key]


def load(folder, dtype, max_tokens=4096, **kw):
    import gopherllm_b200 as gl
    return gl.load(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def feed(model, slot, tokens, cuts):
    """Feed ``tokens`` in pieces of the given sizes (the rest one by one); logits of every position."""
    out, at = [], 0
    cuts = list(cuts)
    while at < len(tokens):
        n = min(cuts.pop(0) if cuts else 1, len(tokens) - at)
        out.append(model.step([(slot, tokens[at:at + n])], [list(range(n))]).cpu().numpy())
        at += n
    return np.concatenate(out, 0)


def check(got, ref, dtype, what=""):
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = np.abs(got - ref).max(-1)
    bound = TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    worst = int(err.argmax())
    assert err.max() <= bound, f"{what} {dtype}: position {worst} differs by {err.max():.3e} (bound {bound:.3e})"
    mean_bound = MEAN_TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    assert err.mean() <= mean_bound, f"{what} {dtype}: positions differ by {err.mean():.3e} on average (bound {mean_bound:.3e})"


def tokens_for(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], size=n)]


FOLDERS = {}


def folder_for(name, cfg, seed, **kw):
    key = (name, seed, tuple(sorted(kw.items())))
    if key not in FOLDERS:
        FOLDERS[key] = vm.write_folder(cfg, vm.draw(cfg, seed, **kw))
    return FOLDERS[key]


ALONE = [("mlstm", vm.only(vm.ALPHA, 0)), ("mlstm_bare_wide", vm.only(vm.BETA, 2, mlp=False)),
         ("mamba1", vm.only(vm.ALPHA, 1)), ("mamba1_short_filter", vm.only(vm.BETA, 1)), ("mamba1_one_tap", vm.only(vm.GAMMA, 0)),
         ("pair", vm.only(vm.ALPHA, 2)), ("pair_full_rotation", vm.only(vm.BETA, 0, mlp=False)),
         ("pair_no_rotation", vm.only(vm.GAMMA, 1)),
         ("pair_looped", vm.only(vm.ALPHA, 2, loop={"start": 0, "stop": 1, "times": 2}))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", ALONE, ids=[a[0] for a in ALONE])
def test_each_mechanism_alone(name, cfg, dtype):
    """One layer of one kind: a whole prompt across a page's edge, then single tokens."""
    folder = folder_for(name, cfg, 11)
    toks = tokens_for(cfg, 78, 1)
    m = load(folder, dtype)
    s = m.open_sequence()
    got = feed(m, s, toks, [70])
    m.engine.check_device()
    check(got, plain_logits(folder, toks), dtype, name)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg_name", ["ALPHA", "BETA", "GAMMA", "DELTA"])
def test_whole_pieces_and_single_tokens(cfg_name, dtype):
    """The same tokens whole, in pieces of many sizes down to two, and mostly one by one."""
    cfg = getattr(vm, cfg_name)
    folder = folder_for(cfg_name, cfg, 5)
    toks = tokens_for(cfg, 150, 2)
    ref = plain_logits(folder, toks)
    m = load(folder, dtype)
    for cuts in ([150], [2, 2, 3, 57, 1, 64, 2, 19], [40]):
        s = m.open_sequence()
        got = feed(m, s, toks, cuts)
        m.close_sequence(s)
        check(got, ref, dtype, f"{cfg_name} cuts {cuts}")
    m.engine.check_device()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(dtype):
    folder = folder_for("ALPHA", vm.ALPHA, 5)
    m = load(folder, dtype)
    for n in (1, 2, 3):
        toks = tokens_for(vm.ALPHA, n, 20 + n)
        s = m.open_sequence()
        check(feed(m, s, toks, [n]), plain_logits(folder, toks), dtype, f"{n} tokens")
        m.close_sequence(s)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(dtype):
    """Three prompts of different lengths as one batch, then decoded together while the shorter ones
    leave; every sequence must get what it gets alone."""
    cfg = vm.ALPHA
    folder = folder_for("ALPHA", cfg, 5)
    lens, prompt = [9, 140, 71], [5, 131, 66]
    seqs = [tokens_for(cfg, n, 30 + i) for i, n in enumerate(lens)]
    m = load(folder, dtype)
    slots = [m.open_sequence() for _ in seqs]
    got = [[] for _ in seqs]
    out = m.step([(slots[i], seqs[i][:prompt[i]]) for i in range(3)], [list(range(p)) for p in prompt]).cpu().numpy()
    at = 0
    for i, p in enumerate(prompt):
        got[i].append(out[at:at + p])
        at += p
    pos = list(prompt)
    while any(pos[i] < lens[i] for i in range(3)):
        live = [i for i in range(3) if pos[i] < lens[i]]
        out = m.step([(slots[i], [seqs[i][pos[i]]]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
            pos[i] += 1
            if pos[i] == lens[i]:
                m.close_sequence(slots[i])
    m.engine.check_device()
    for i in range(3):
        check(np.concatenate(got[i], 0), plain_logits(folder, seqs[i]), dtype, f"sequence {i} in the batch")
    if dtype == "float32":
        alone = load(folder, dtype)
        s = alone.open_sequence()
        one = feed(alone, s, seqs[2], [prompt[2]])
        assert np.abs(one - np.concatenate(got[2], 0)).max() <= 2e-5 * max(1.0, np.abs(one).max())
        alone.close()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype):
    """A sequence that takes the slot, the state rows and the pages another one left must not see them."""
    cfg = vm.ALPHA
    folder = folder_for("ALPHA", cfg, 5, long_memory=True)
    a, b, c = tokens_for(cfg, 130, 40), tokens_for(cfg, 90, 41), tokens_for(cfg, 70, 42)
    m = load(folder, dtype, max_tokens=512)
    sa = m.open_sequence()
    feed(m, sa, a, [100])
    sb = m.open_sequence()
    gb = [feed(m, sb, b[:50], [50])]
    m.close_sequence(sa)
    sc = m.open_sequence()                      # takes a's slot and pages while b is still live
    assert sc == sa
    gc = feed(m, sc, c, [33, 2])
    gb.append(feed(m, sb, b[50:], [7]))
    m.engine.check_device()
    check(gc, plain_logits(folder, c), dtype, "the sequence in the used slot")
    check(np.concatenate(gb, 0), plain_logits(folder, b), dtype, "the sequence that stayed")
    m.engine.cache.check()
    m.close()


def test_far_tokens_and_page_edges():
    """Weights with long memories and a sharp softmax: the logits late in a sequence hang on single
    tokens hundreds of positions back and on keys right at the pages' edges."""
    cfg = vm.ALPHA
    folder = folder_for("ALPHA_far", cfg, 7, long_memory=True, sharp=4.0)
    toks = tokens_for(cfg, 200, 50)
    ref = plain_logits(folder, toks)
    other = list(toks)
    other[3] = (other[3] + 1) % cfg["vocab"]
    moved = np.abs(plain_logits(folder, other)[190:] - ref[190:]).max()
    assert moved > 20 * TOL["float32"] * max(1.0, np.abs(ref).max()), "the test's model forgets its early tokens"
    m = load(folder, "float32")
    for cuts in ([200], [63, 1, 1, 63, 2], [129], [64, 64, 64]):
        s = m.open_sequence()
        check(feed(m, s, toks, cuts), ref, "float32", f"cuts {cuts}")
        m.close_sequence(s)
    m.close()
    m = load(folder, "bfloat16")
    s = m.open_sequence()
    got = feed(m, s, toks, [127])
    m.engine.check_device()
    check(got, ref, "bfloat16", "far tokens")
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """A few tokens of prompt, then single tokens across two pages' edges (captured steps in bfloat16)."""
    cfg = vm.BETA
    folder = folder_for("BETA", cfg, 9, long_memory=True)
    toks = tokens_for(cfg, 140, 60)
    m = load(folder, dtype)
    s = m.open_sequence()
    got = feed(m, s, toks, [3])
    m.engine.check_device()
    check(got, plain_logits(folder, toks), dtype, "long decoding")
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_runs_walked_as_chunks(dtype, monkeypatch):
    """Long runs of the scans are cut into chunks that are walked side by side, with a carry between two
    walks.  With chunks of 16 tokens from 32 tokens on: a whole prompt (a ragged last chunk), pieces above
    and below the threshold, and a batch whose shorter sequence has fewer chunks than the longer one."""
    from gopherllm_b200 import ops
    monkeypatch.setattr(ops, "SCAN_CHUNK_TOKENS", 16)
    monkeypatch.setattr(ops, "SCAN_CHUNKED_FROM", 32)
    for cfg_name in ("ALPHA", "BETA"):
        cfg = getattr(vm, cfg_name)
        folder = folder_for(cfg_name, cfg, 5, long_memory=True)
        toks = tokens_for(cfg, 150, 2)
        ref = plain_logits(folder, toks)
        m = load(folder, dtype)
        for cuts in ([150], [33, 31, 64, 17]):
            s = m.open_sequence()
            check(feed(m, s, toks, cuts), ref, dtype, f"{cfg_name} cuts {cuts}")
            m.close_sequence(s)
        short = tokens_for(cfg, 37, 3)
        sa, sb = m.open_sequence(), m.open_sequence()
        out = m.step([(sa, short), (sb, toks[:100])], [list(range(37)), list(range(100))]).cpu().numpy()
        check(out[:37], plain_logits(folder, short), dtype, "the shorter of two")
        check(out[37:], ref[:100], dtype, "the longer of two")
        m.engine.check_device()
        m.close()


def test_greedy_generation_through_the_scheduler():
    """Model.generate, greedy, for prompts of different lengths in one call: the tokens the plain
    implementation chooses."""
    cfg = vm.GAMMA
    folder = folder_for("GAMMA", cfg, 3)
    prompts = [tokens_for(cfg, n, 70 + n) for n in (4, 37, 66)]
    m = load(folder, "float32")
    outs = m.generate(prompts, max_tokens=8, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())
    pcfg, t = pv.read_folder(folder)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(8):
            logits = pv.forward(pcfg, t, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 1e-3:        # a tie within rounding proves nothing either way
                break
            seq.append(int(logits.argmax()))
        want = seq[len(p):]
        assert o.tokens[:len(want)] == want, (o.tokens, want)
    m.close()
    mb = load(folder, "bfloat16")
    outs_b = mb.generate(prompts, max_tokens=8, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())
    assert all(len(o.tokens) == 8 for o in outs_b)
    mb.engine.check_device()
    mb.close()


def test_replay_of_a_trace(tmp_path):
    """The trace runner's loop on a Vopedra model: a batch of two requests, one ends, the other goes on."""
    import json
    from gopherllm_b200.engine.replay import run
    cfg = vm.ALPHA
    folder = folder_for("ALPHA", cfg, 5)
    a, b = tokens_for(cfg, 70, 80), tokens_for(cfg, 12, 81)
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 63, 65]},
                                                 {"id": "b", "tokens": b[:11], "want": []}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]},
                                                 {"id": "b", "tokens": b[11:], "want": [0]}], "end": ["b"]})]
    lines += [json.dumps({"step": 2 + i, "entries": [{"id": "a", "tokens": [a[67 + i]], "want": [0]}],
                          "end": ["a"] if i == 2 else []}) for i in range(3)]
    m = load(folder, "float32")
    said = []
    run(m, lines, str(tmp_path), said.append)
    assert said == [f"done {i}" for i in range(5)]
    ra, rb = plain_logits(folder, a), plain_logits(folder, b)
    got0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(3, -1)
    check(got0, ra[[0, 63, 65]], "float32", "step 0")
    got1 = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(2, -1)
    check(got1, np.stack([ra[66], rb[11]]), "float32", "step 1")
    got4 = np.fromfile(tmp_path / "4.f32", dtype="<f4").reshape(1, -1)
    check(got4, ra[69:70], "float32", "step 4")
    assert not m.engine.cache.live_slots()
    m.close()
