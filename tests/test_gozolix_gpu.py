"""The Gozolix design through the library's loader, cache, step function, scheduler and kernels, against
the plain implementation (tests/plain_gozolix.py) on small models whose weights the tests make themselves."""
import json

import numpy as np
import pytest
import torch

import gozolix_models as gm
import plain_gozolix as pg

pytestmark = pytest.mark.gpu

# the largest |difference| of a position's logits is bounded by TOL * max(1, max|reference|); in bfloat16 also
# the mean over positions by MEAN_TOL
TOL = {"float32": 3e-4, "bfloat16": 1e-1}
MEAN_TOL = {"float32": 1e-4, "bfloat16": 3e-2}
_REF = {}


def plain_logits(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _REF:
        cfg, t = gm.read_folder(folder)
        _REF[key] = pg.forward(list(tokens), t, cfg).numpy()
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


def has_router(cfg):
    return any((L.get("mlp") or {}).get("kind") == "moe" for L in cfg["layers"])


def check(got, ref, dtype, what="", routed=False):
    """In bfloat16 a router may choose another expert than the 64-bit reference where two scores lie within
    the rounding of its input; such a position (and, faintly, those that read it) proves nothing, so with a
    router a few positions may lie outside the bound there.  The 32-bit path is held to the bound everywhere."""
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = np.abs(got - ref).max(-1)
    bound = TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    worst = int(err.argmax())
    if routed and dtype == "bfloat16":
        over = int((err > bound).sum())
        assert over <= max(1, len(err) // 8), f"{what} {dtype}: {over} of {len(err)} positions differ by more than {bound:.3e}"
        assert float(np.median(err)) <= MEAN_TOL[dtype] * max(1.0, float(np.abs(ref).max())), what
        return
    assert err.max() <= bound, f"{what} {dtype}: position {worst} differs by {err.max():.3e} (bound {bound:.3e})"
    mean_bound = MEAN_TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    assert err.mean() <= mean_bound, f"{what} {dtype}: positions differ by {err.mean():.3e} on average (bound {mean_bound:.3e})"


def tokens_for(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], size=n)]


FOLDERS = {}


def folder_for(name, cfg, seed, **kw):
    key = (name, seed, tuple(sorted(kw.items())))
    if key not in FOLDERS:
        FOLDERS[key] = gm.write_folder(cfg, gm.draw(cfg, seed, **kw))
    return FOLDERS[key]


# layer sizes nearer a real model's: rows of a memory that fill a thread's registers, heads of 128, many experts
WIDE = dict(
    architecture="Gozolix", vocab=500, width=256, norm={"eps": 1e-6},
    embedding={"scale": 2.0, "bigram": {"buckets": 4093, "mul_prev": 40503, "mul_cur": 17}},
    layers=[
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 4},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "shared": {"ff": 128},
                 "router": {"experts": 32, "top": 4, "scale": 1.0, "groups": {"count": 8, "keep": 3}}}},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09, "softcap": 20.0,
                                        "q_temp": {"coef": 0.3, "every": 32}}, "mlp": {"kind": "dense", "ff": 512}},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09, "softcap": 20.0,
                                        "kv_from": 1}, "mlp": None},
    ])

ALONE = [("delta", gm.only(gm.ALPHA, 0)), ("attention_routed_groups", gm.only(gm.ALPHA, 1)),
         ("delta_routed_plain", gm.only(gm.ALPHA, 3)), ("delta_bare_wide_one_tap", gm.only(gm.BETA, 1, mlp=False)),
         ("attention_bare", gm.only(gm.BETA, 0, mlp=False)), ("attention_six_on_one_groups_of_one", gm.only(gm.BETA, 2)),
         ("delta_odd", gm.only(gm.GAMMA, 0)), ("attention_nine_on_one", gm.only(gm.GAMMA, 1)),
         ("attention_ten_key_heads", gm.only(gm.GAMMA, 2))]


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
    check(got, plain_logits(folder, toks), dtype, name, routed=has_router(cfg))
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg_name", ["ALPHA", "BETA", "GAMMA"])
def test_whole_pieces_and_single_tokens(cfg_name, dtype):
    """The same tokens whole, in pieces of many sizes down to two, and mostly one by one."""
    cfg = getattr(gm, cfg_name)
    folder = folder_for(cfg_name, cfg, 5)
    toks = tokens_for(cfg, 150, 2)
    ref = plain_logits(folder, toks)
    m = load(folder, dtype)
    for cuts in ([150], [2, 2, 3, 57, 1, 64, 2, 19], [40]):
        s = m.open_sequence()
        got = feed(m, s, toks, cuts)
        m.close_sequence(s)
        check(got, ref, dtype, f"{cfg_name} cuts {cuts}", routed=True)
    m.engine.check_device()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_nearer_a_real_layer(dtype):
    folder = folder_for("WIDE", WIDE, 21)
    toks = tokens_for(WIDE, 200, 4)
    ref = plain_logits(folder, toks)
    m = load(folder, dtype)
    for cuts in ([200], [130, 66]):
        s = m.open_sequence()
        check(feed(m, s, toks, cuts), ref, dtype, f"cuts {cuts}", routed=True)
        m.close_sequence(s)
    m.engine.check_device()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(dtype):
    folder = folder_for("ALPHA", gm.ALPHA, 5)
    m = load(folder, dtype)
    for n in (1, 2, 3):
        toks = tokens_for(gm.ALPHA, n, 20 + n)
        s = m.open_sequence()
        check(feed(m, s, toks, [n]), plain_logits(folder, toks), dtype, f"{n} tokens", routed=True)
        m.close_sequence(s)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(dtype):
    """Three prompts of different lengths as one batch, then decoded together while the shorter ones leave;
    every sequence must get what it gets alone."""
    cfg = gm.ALPHA
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
        check(np.concatenate(got[i], 0), plain_logits(folder, seqs[i]), dtype, f"sequence {i} in the batch", routed=True)
    if dtype == "float32":
        alone = load(folder, dtype)
        s = alone.open_sequence()
        one = feed(alone, s, seqs[2], [prompt[2]])
        assert np.abs(one - np.concatenate(got[2], 0)).max() <= 2e-5 * max(1.0, np.abs(one).max())
        alone.close()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype):
    """A sequence that takes the slot, the state rows (memory, filter inputs, the token before) and the pages
    another one left must not see them."""
    cfg = gm.ALPHA
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
    check(gc, plain_logits(folder, c), dtype, "the sequence in the used slot", routed=True)
    check(np.concatenate(gb, 0), plain_logits(folder, b), dtype, "the sequence that stayed", routed=True)
    m.engine.cache.check()
    m.close()


def test_far_tokens_and_page_edges():
    """Memories that decay slowly and a sharp softmax: the logits late in a sequence hang on single tokens
    hundreds of positions back and on keys right at the pages' edges; pieces end on, before and after them."""
    cfg = gm.ALPHA
    folder = folder_for("ALPHA_far", cfg, 7, long_memory=True, sharp=4.0)
    toks = tokens_for(cfg, 200, 50)
    ref = plain_logits(folder, toks)
    other = list(toks)
    other[3] = (other[3] + 1) % cfg["vocab"]
    moved = np.abs(plain_logits(folder, other)[190:] - ref[190:]).max()
    assert moved > 20 * TOL["float32"] * max(1.0, np.abs(ref).max()), "the test's model forgets its early tokens"
    m = load(folder, "float32")
    for cuts in ([200], [63, 1, 1, 63, 2], [129], [64, 64, 64], [65, 63]):
        s = m.open_sequence()
        check(feed(m, s, toks, cuts), ref, "float32", f"cuts {cuts}")
        m.close_sequence(s)
    m.close()
    m = load(folder, "bfloat16")
    s = m.open_sequence()
    got = feed(m, s, toks, [127])
    m.engine.check_device()
    check(got, ref, "bfloat16", "far tokens", routed=True)
    m.close()


def test_one_far_key_decides():
    """An attention layer alone whose last head (the gentlest slope) is given, by hand, a query that matches
    the key of one position far back, many times stronger than any other: the late logits then hang on that
    position's value.  The score is capped smoothly, so the match must survive the cap and the distance."""
    cfg = gm.only(gm.BETA, 0, mlp=False)
    cfg["layers"][0]["mixer"].update({"softcap": 40.0, "scale": 1.0})
    t = gm.draw(cfg, 13)
    H, D = 3, 16
    wq, wk = t["l0.mix.q"].float(), t["l0.mix.k"].float()
    wq[(H - 1) * D:] *= 6.0
    wk[(H - 1) * D:] *= 6.0
    t["l0.mix.q"], t["l0.mix.k"] = wq.to(torch.bfloat16), wk.to(torch.bfloat16)
    folder = gm.write_folder(cfg, t)
    toks = tokens_for(cfg, 300, 8)
    ref = plain_logits(folder, toks)
    for dtype in ("float32", "bfloat16"):
        m = load(folder, dtype)
        for cuts in ([300], [256, 1, 1, 40], [10]):
            s = m.open_sequence()
            check(feed(m, s, toks, cuts), ref, dtype, f"cuts {cuts}")
            m.close_sequence(s)
        m.engine.check_device()
        m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """A few tokens of prompt, then single tokens across two pages' edges and several periods of the query
    temperature (captured steps in bfloat16)."""
    cfg = gm.BETA
    folder = folder_for("BETA", cfg, 9, long_memory=True)
    toks = tokens_for(cfg, 140, 60)
    m = load(folder, dtype)
    s = m.open_sequence()
    got = feed(m, s, toks, [3])
    m.engine.check_device()
    check(got, plain_logits(folder, toks), dtype, "long decoding", routed=True)
    m.close()


def test_greedy_generation_through_the_scheduler():
    """Model.generate, greedy, for prompts of different lengths in one call: the tokens the plain
    implementation chooses."""
    cfg = gm.GAMMA
    folder = folder_for("GAMMA", cfg, 3)
    prompts = [tokens_for(cfg, n, 70 + n) for n in (4, 37, 66)]
    m = load(folder, "float32")
    outs = m.generate(prompts, max_tokens=8, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())
    pcfg, t = gm.read_folder(folder)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(8):
            logits = pg.forward(seq, t, pcfg)[-1]
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


def test_generation_on_the_device_keeps_the_token_before():
    """The on-device loop feeds tokens back without the host: the hashed pair embedding must see each of them
    as the next step's token before.  Greedy, against Model.generate."""
    from gopherllm_b200.sampling.sampler import DeviceSampler, SamplerConfig
    cfg = gm.ALPHA
    folder = folder_for("ALPHA", cfg, 5)
    prompt = tokens_for(cfg, 21, 90)
    m = load(folder, "bfloat16")
    want = m.generate([prompt], max_tokens=12, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())[0].tokens
    s = m.open_sequence()
    logits = m.step([(s, prompt)])
    first = int(logits[0].argmax())
    assert first == want[0]
    sampler = DeviceSampler(SamplerConfig.greedy(), [1], [prompt], cfg["vocab"], m.engine.device)
    chosen = m.engine.decode_loop([s], [first], 11, sampler).cpu().numpy()[:, 0].tolist()
    assert [first] + chosen == want
    m.engine.check_device()
    m.close()


def test_command_line_generates_and_samples():
    """python -m gopherllm_b200 on a Gozolix folder: greedy tokens equal the plain implementation's, a sampled
    run with the sampler's options ends by length, and the isolated kernel bench knows the parts' products."""
    import os
    import subprocess
    import sys
    cfg = gm.GAMMA
    folder = folder_for("GAMMA", cfg, 3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = lambda *a: subprocess.run([sys.executable, "-m", "gopherllm_b200", folder, *a], cwd=root,
                                    capture_output=True, text=True, timeout=600)
    prompt = tokens_for(cfg, 9, 77)
    pcfg, t = gm.read_folder(folder)
    seq = list(prompt)
    for _ in range(5):
        logits = pg.forward(seq, t, pcfg)[-1]
        top2 = torch.topk(logits, 2).values
        if float(top2[0] - top2[1]) < 1e-3:
            break
        seq.append(int(logits.argmax()))
    want = seq[len(prompt):]
    p = run("--prompt", " ".join(map(str, prompt)), "--max-tokens", "5", "--temp", "0", "--repeat-penalty", "1",
            "--dtype", "float32", "--stop", "100000")
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.split()][:len(want)] == want
    p = run("--prompt", " ".join(map(str, prompt)), "--max-tokens", "12", "--temp", "0.9", "--top-k", "20", "--top-p", "0.95",
            "--seed", "4", "--stop", "100000")
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(x) for x in p.stdout.split()]
    assert len(out) == 12 and all(0 <= x < cfg["vocab"] for x in out) and "finish=length" in p.stderr
    p = run("--kernel-bench-json", "--kernel-bench-runs", "2")
    assert p.returncode == 0, p.stderr[-2000:]
    assert json.loads(p.stdout)["kernels"]


def test_replay_of_a_trace(tmp_path):
    """The trace runner's loop on a Gozolix model: a batch of two requests, one ends, the other goes on."""
    from gopherllm_b200.engine.replay import run
    cfg = gm.ALPHA
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


# ---------------------------------------------------------------------------
# the new kernels alone, against the plain functions
def test_router_kernel_against_the_plain_router():
    from gopherllm_b200 import ops
    g = torch.Generator().manual_seed(3)
    for E, top, groups, keep, scale in ((64, 6, 8, 4, 1.7), (5, 5, 1, 1, 1.0), (12, 1, 12, 5, 0.3), (33, 4, 3, 2, 2.0),
                                        (256, 8, 8, 4, 2.5)):
        z = torch.randn(97, E, generator=g) * 2.0
        ids, w = ops.moe_route(z.cuda(), top, groups, keep, scale)
        r = {"experts": E, "top": top, "scale": scale}
        if groups > 1:
            r["groups"] = {"count": groups, "keep": keep}
        chosen, weights = pg.route(z.double(), {"router": torch.eye(E, dtype=torch.float64)}, "", r)
        order = torch.argsort(ids.cpu().long(), dim=1)
        want_order = torch.argsort(chosen, dim=1)
        assert torch.equal(torch.gather(ids.cpu().long(), 1, order), torch.gather(chosen, 1, want_order)), (E, top, groups)
        assert torch.allclose(torch.gather(w.cpu().double(), 1, order), torch.gather(weights, 1, want_order), atol=1e-6)
    # with the router's product in front, from 32-bit and from bfloat16 inputs
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(50, 40, generator=g).to(dtype)
        wr = torch.randn(12, 40, generator=g)
        ids, w = ops.moe_route_from(x.cuda(), wr.cuda(), 3, 4, 2, 1.5)
        chosen, weights = pg.route(x.double(), {"router": wr.double()}, "", {"experts": 12, "top": 3, "scale": 1.5,
                                                                             "groups": {"count": 4, "keep": 2}})
        order, want_order = torch.argsort(ids.cpu().long(), dim=1), torch.argsort(chosen, dim=1)
        assert torch.equal(torch.gather(ids.cpu().long(), 1, order), torch.gather(chosen, 1, want_order))
        assert torch.allclose(torch.gather(w.cpu().double(), 1, order), torch.gather(weights, 1, want_order), atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_expert_products_with_given_choices(dtype):
    """The experts' kernels with the choices given (no router in the way): many tokens on few experts, experts
    nobody chose, tiles that end ragged, inner sizes that are multiples of nothing; both kernels in bfloat16."""
    from gopherllm_b200 import ops
    g = torch.Generator().manual_seed(5)
    for T, K, F, N, E, top in ((150, 64, 40, 64, 7, 3), (3, 96, 24, 96, 16, 2), (70, 40, 11, 36, 4, 4), (1, 128, 64, 128, 32, 4),
                               (20, 72, 24, 40, 16, 2), (2, 2304, 16, 32, 4, 2), (700, 256, 320, 192, 8, 2)):
        x = torch.randn(T, K, generator=g).to(dtype)
        wgu = (torch.randn(E, 2 * F, K, generator=g) / K ** 0.5).to(dtype)
        wd = (torch.randn(E, N, F, generator=g) / F ** 0.5).to(dtype)
        ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
        if T in (150, 20):
            ids[:, 0] = 2                                  # one expert takes every token: several tiles, several chunks of rows
        wts = torch.rand(T, top, generator=g)
        add = torch.randn(T, N, generator=g)
        ref = add.double().clone()
        xd = x.double()
        for t in range(T):
            for k in range(top):
                e = int(ids[t, k])
                gate, up = wgu[e, :F].double() @ xd[t], wgu[e, F:].double() @ xd[t]
                h = gate * torch.sigmoid(gate) * up
                if dtype == torch.bfloat16:
                    h = h.to(torch.bfloat16).double()
                ref[t] += float(wts[t, k]) * (wd[e].double() @ h)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        # bfloat16: the kernel the sizes choose (few rows an expert, or one grouped product on tcgen05), tiles of
        # rows on mma.sync, and the CUDA-core kernels
        for grouped, tc in (((True, True), (False, True), (False, False)) if dtype == torch.bfloat16 else ((True, True),)):
            ops.USE_MOE_GROUPED, ops.USE_MOE_TC = grouped, tc
            try:
                out = ops.moe_experts(x.cuda(), ids.cuda(), wts.cuda(), wgu.cuda(), wd.cuda(), add=add.cuda())
            finally:
                ops.USE_MOE_GROUPED = ops.USE_MOE_TC = True
            assert (out.cpu().double() - ref).abs().max() <= tol * max(1.0, float(ref.abs().max())), (T, K, F, N, E, top, grouped, tc)
        ops.check_wait_failures()
