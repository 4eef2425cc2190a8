"""Gavipel (layer-list decoder with a repeated span, windowed gated attention and group-limited experts) against the plain
oracle of oracle/gavipel.py.

Small configurations with their own random weights; the oracle runs in float64.  The engine's "f32" precision is held to a
tight bar (a lost key, a window that is one token off, a missing sink or a page of the wrong pass shows), the serving
precision to the bar its operand rounding allows.
"""
import copy
import math

import numpy as np
import pytest
import torch

from oracle import gavipel as G

T64 = torch.float64


# ---------------------------------------------------------------------------------------------------- configurations
def mixer(heads=6, kv_heads=2, dim=40, vdim=24, scale=0.2, window=50, rot_dims=12, base=900.0, scaling=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 24}
    return m


def moe(ff=36, experts=6, top=2, count=3, keep=2, shared=52):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def layer(mx=None, mlp="default"):
    return {"type": "attention", "mixer": mx or mixer(), "mlp": moe() if mlp == "default" else mlp}


def config(layers, loop=None, width=112, vocab=211, scale=5.0, eps=1e-5):
    c = {"architecture": "Gavipel", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
         "layers": copy.deepcopy(layers)}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# five layers of unequal geometry; layers 1-2 run three times
FULL = config([layer(mixer(window=37)),
               layer(mixer(heads=4, kv_heads=4, dim=18, vdim=36, scale=0.35, window=64, rot_dims=18, scaling=False), moe(ff=20, experts=8, top=3, count=2, keep=1, shared=0)),
               layer(mixer(heads=8, kv_heads=1, dim=32, vdim=16, window=33, rot_dims=8), moe(ff=40, experts=4, top=1, count=4, keep=2, shared=24)),
               layer(mixer(window=0), None),
               layer(mixer(heads=3, kv_heads=3, dim=24, vdim=40, window=129, rot_dims=0), moe(ff=28, experts=9, top=4, count=1, keep=1))],
              loop=(1, 3, 3))
SINGLE = {
    "attention_only": config([layer(mlp=None)]),
    "no_rotation_no_window": config([layer(mixer(window=0, rot_dims=0), None)], width=96, vocab=128),
    "full_rotation_odd_widths": config([layer(mixer(heads=5, kv_heads=5, dim=22, vdim=9, rot_dims=22, window=7), None)], width=72, vocab=90),
    "window_of_one": config([layer(mixer(window=1), None)]),
    "experts_grouped": config([layer(mixer(window=40), moe())]),
    "experts_top1_no_shared": config([layer(mixer(window=40), moe(ff=30, experts=5, top=1, count=5, keep=1, shared=0))]),
    "experts_one_group": config([layer(mixer(window=40), moe(ff=44, experts=7, top=7, count=1, keep=1, shared=16))]),
    "loop_from_the_first_layer": config([layer(), layer(mixer(window=20))], loop=(0, 2, 2)),
    "loop_once": config([layer(), layer(mixer(window=20), None)], loop=(1, 2, 1)),
    "no_loop": config([layer(), layer(mixer(window=20), None)]),
}


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


F32_TOL, SPLIT_TOL = 2e-5, 2e-3


def oracle_logits(cfg, w, ids, cache=None):
    return G.forward(cfg, w, ids, cache).numpy()


# ---------------------------------------------------------------------------------------------------- CPU: the oracle itself
def test_oracle_prefill_equals_token_by_token():
    w = G.random_weights(FULL, 1)
    ids = tokens(90, FULL["vocab"], 2)
    whole = oracle_logits(FULL, w, ids)
    c = G.Cache(FULL)
    parts = [oracle_logits(FULL, w, ids[a:b], c) for a, b in ((0, 7), (7, 9), (9, 10), (10, 70), (70, 71), (71, 90))]
    assert rel(np.concatenate(parts), whole) < 1e-11


def test_oracle_mechanisms_on_known_answers():
    # one key with score 0 beside the valueless unit term: half the value
    q = torch.zeros(1, 1, 4, dtype=T64); k = torch.ones(1, 1, 4, dtype=T64); v = torch.full((1, 1, 3), 2.0, dtype=T64)
    assert torch.allclose(G.windowed_attention(q, k, v, torch.tensor([0]), 1.0, 5, 1), torch.full((1, 1, 3), 1.0, dtype=T64))
    # window 2 at position 3 sees keys 2 and 3 only: values 0, 1, 2, 3 with equal scores -> (2 + 3) / (1 + 2)
    k = torch.zeros(4, 1, 2, dtype=T64); v = torch.arange(4, dtype=T64).reshape(4, 1, 1)
    out = G.windowed_attention(torch.zeros(1, 1, 2, dtype=T64), k, v, torch.tensor([3]), 1.0, 2, 1)
    assert abs(float(out) - 5.0 / 3.0) < 1e-12
    # rotation: pairs (0, 1) and (2, 3) turn, the rest passes; a quarter turn maps (1, 0) to (0, 1)
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 7.0, 9.0]]], dtype=T64)
    y = G.rotate(x, torch.tensor([1]), torch.tensor([math.pi / 2, math.pi], dtype=T64))
    assert torch.allclose(y, torch.tensor([[[0.0, 1.0, 0.0, -2.0, 7.0, 9.0]]], dtype=T64), atol=1e-12)
    # frequency bands: wavelengths 2 pi (short: kept), 2 pi * 10^4 (long: divided), and 2 pi * 100 in between (blended)
    f = G.rotary_frequencies(6, 100.0 ** 3, {"factor": 5.0, "low": 1.0, "high": 4.0, "original": 2000.0})
    raw = [1.0, 1e-2, 1e-4]
    assert abs(float(f[0]) - raw[0]) < 1e-15 and abs(float(f[2]) - raw[2] / 5.0) < 1e-18
    s = (2000.0 / (2 * math.pi / raw[1]) - 1.0) / 3.0
    assert 0.0 < s < 1.0 and abs(float(f[1]) - ((1 - s) * raw[1] / 5.0 + s * raw[1])) < 1e-15
    # norms
    assert torch.allclose(G.norm_one_plus(torch.tensor([[3.0, 3.0]], dtype=T64), torch.tensor([0.5, -1.0], dtype=T64), 0.0), torch.tensor([[1.5, 0.0]], dtype=T64))
    assert torch.allclose(G.head_norm(torch.tensor([[2.0, 2.0]], dtype=T64), torch.tensor([3.0, 0.0], dtype=T64), 0.0), torch.tensor([[3.0, 0.0]], dtype=T64))
    # routing: the bias moves the choice but not the weight; a group is ranked by its two best; losers count as minus infinity
    h = torch.ones(1, 1, dtype=T64)
    wr = torch.tensor([[0.0], [2.0], [-1.0], [1.0]], dtype=T64)                    # scores .5, .88, .27, .73
    idx, wt = G.route(h, wr, torch.tensor([0.0, 0.0, 0.0, 0.0], dtype=T64), 1, 1, 1)
    assert idx.tolist() == [[1]] and abs(float(wt) - 1 / (1 + math.exp(-2.0))) < 1e-12
    idx, wt = G.route(h, wr, torch.tensor([1.0, 0.0, 0.0, 0.0], dtype=T64), 1, 1, 1)
    assert idx.tolist() == [[0]] and abs(float(wt) - 0.5) < 1e-12                  # chosen through the bias, weighted without it
    # groups {0, 1} and {2, 3}: sums 1.38 and 1.0 -> group 0 only, although expert 3 beats expert 0
    idx, _ = G.route(h, wr, torch.zeros(4, dtype=T64), 2, 2, 1)
    assert sorted(idx.tolist()[0]) == [0, 1]
    # negative choice values: the kept group's experts still beat the dropped group's
    idx, _ = G.route(h, wr, torch.tensor([-5.0, -5.0, -9.0, -9.0], dtype=T64), 2, 2, 1)
    assert sorted(idx.tolist()[0]) == [0, 1]
    # run order and pass starts
    c = config([layer()] * 5, loop=(1, 3, 2))
    assert [i for i, _ in G.layer_runs(c)] == [0, 1, 2, 1, 2, 3, 4] and G.pass_starts(c) == [1, 3]
    assert [i for i, _ in G.layer_runs(config([layer()] * 2))] == [0, 1] and G.pass_starts(config([layer()] * 2)) == []


def test_oracle_sees_what_the_sharp_tests_are_about(monkeypatch):
    cfg, w = sharp_model(3)
    ids = tokens(150, cfg["vocab"], 4)
    want = oracle_logits(cfg, w, ids)
    orig = G.windowed_attention
    for dw in (-1, 1):                                                           # a window one token off
        monkeypatch.setattr(G, "windowed_attention", lambda q, k, v, p, s, win, n, dw=dw: orig(q, k, v, p, s, win + dw, n))
        assert rel(oracle_logits(cfg, w, ids)[40:], want[40:]) > 1e-2
    monkeypatch.setattr(G, "windowed_attention", no_sink)                        # the unit term of the denominator left out
    assert rel(oracle_logits(cfg, w, ids), want) > 1e-2
    monkeypatch.setattr(G, "windowed_attention", orig)
    c = G.Cache(cfg)
    oracle_logits(cfg, w, ids[:120], c)
    assert [i for i, _ in G.layer_runs(cfg)] == [0, 1, 1, 2]
    c.k[1], c.k[2] = c.k[2], c.k[1]                                              # keys of one pass handed to the other
    assert rel(oracle_logits(cfg, w, ids[120:], c), want[120:]) > 1e-3


def no_sink(q, k, v, q_pos, scale, window, n_rep):
    S, H, _ = q.shape
    out = torch.zeros(S, H, v.shape[-1], dtype=q.dtype)
    j = torch.arange(k.shape[0])[None, :]
    hidden = (j > q_pos[:, None]) | (q_pos[:, None] - j >= window)
    for h in range(H):
        s = ((q[:, h, :] @ k[:, h // n_rep, :].T) * scale).masked_fill(hidden, float("-inf"))
        out[:, h, :] = torch.softmax(s, -1) @ v[:, h // n_rep, :]
    return out


def sharp_model(seed):
    """Scores with a spread of several units: a query looks at one or two keys anywhere in its window and the unit term of the
    denominator is a real competitor, so a lost key, a shifted edge or a missing sink moves the logits by O(1).  The windows
    (70 and 45) put their edges inside pages, on a page border (position 64 + 70 - 1) and across 32-key tiles."""
    cfg = config([layer(mixer(scale=0.45, window=70, rot_dims=12), None),
                  layer(mixer(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.5, window=45, rot_dims=32, scaling=False)),
                  layer(mixer(scale=0.4, window=128, rot_dims=0), None)], loop=(1, 2, 2), width=128, vocab=200)
    return cfg, G.random_weights(cfg, seed)


# ---------------------------------------------------------------------------------------------------- GPU
def make(cfg, seed=0, **opts):
    import crane_b200
    w = G.random_weights(cfg, seed)
    opts.setdefault("max_tokens", 1024)
    opts.setdefault("max_batch", 4)
    m = crane_b200.GavipelModel(cfg, device=0, **opts)
    m.load_checkpoint((k, t.to(torch.float32).numpy()) for k, t in w.items())
    return m, w


def all_rows(n):
    return list(range(n))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(name):
    cfg = SINGLE[name]
    m, w = make(cfg, 3, precision="f32")
    ids = tokens(100, cfg["vocab"], 4)
    assert rel(m.step_batch([(0, ids, all_rows(100))]), oracle_logits(cfg, w, ids)) < F32_TOL
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_whole_model_prefill_and_token_by_token_decoding(precision, tol):
    m, w = make(FULL, 5, precision=precision)
    ids = tokens(170, FULL["vocab"], 6)
    want = oracle_logits(FULL, w, ids)
    got = m.step_batch([(0, ids, all_rows(len(ids)))])
    assert rel(got, want) < tol
    m.clear_kv_cache()
    rows = [m.step_batch([(0, ids[:3], [0, 1, 2])])]
    rows += [m.step_batch([(0, [t], [0])]) for t in ids[3:]]       # long decoding: every window passes over decoded tokens, two page borders
    step = np.concatenate(rows)
    assert rel(step, want) < tol
    if precision == "f32":
        assert rel(step, got) < 1e-5
    m.close()


@pytest.mark.gpu
def test_plain_bf16_precision_is_close():
    m, w = make(FULL, 7, precision="bf16")
    ids = tokens(90, FULL["vocab"], 8)
    assert rel(m.step_batch([(0, ids, all_rows(90))]), oracle_logits(FULL, w, ids)) < 5e-2
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("cuts", [[2, 2, 2, 61, 3, 64, 1, 1, 30, 2], [63, 1, 1, 63, 2, 36], [1] * 5 + [95, 66], [31, 33, 32, 64, 6]])
def test_portions_of_any_size_match_the_whole_prompt(cuts):
    m, w = make(FULL, 9, precision="f32")
    n = sum(cuts)
    ids = tokens(n, FULL["vocab"], 10)
    want = oracle_logits(FULL, w, ids)
    at, rows = 0, []
    for c in cuts:
        rows.append(m.step_batch([(0, ids[at:at + c], all_rows(c))]))
        at += c
    assert rel(np.concatenate(rows), want) < F32_TOL
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_unequal_requests_in_one_batch_match_each_alone(precision, tol):
    m, w = make(FULL, 11, precision=precision, max_tokens=1024)
    lens = [97, 5, 130, 64]
    prompts = [tokens(n, FULL["vocab"], 20 + i) for i, n in enumerate(lens)]
    want = [oracle_logits(FULL, w, p) for p in prompts]
    seqs = [0] + [m.seq_create() for _ in range(3)]
    got = [[] for _ in lens]
    at = [0] * 4
    # a different mixture every step: portions of some beside single tokens of others, one request sitting a step out
    plan = [[(0, 40), (1, 2), (2, 1)], [(2, 64), (3, 63), (0, 1)], [(1, 1), (3, 1), (0, 56), (2, 2)], [(1, 2), (2, 63)]]
    for stepn in plan:
        entries = [(seqs[i], prompts[i][at[i]:at[i] + c], all_rows(c)) for i, c in stepn]
        lg = m.step_batch(entries)
        r = 0
        for i, c in stepn:
            got[i].append(lg[r:r + c]); r += c; at[i] += c
    for i in range(4):
        g = np.concatenate(got[i])
        assert rel(g, want[i][:len(g)]) < tol, i
    m.close()


@pytest.mark.gpu
def test_pages_and_slots_are_used_again():
    m, w = make(FULL, 13, precision="f32", max_tokens=256, max_batch=2)        # 4 pages, 2 slots
    a, b, c = (tokens(n, FULL["vocab"], 30 + i) for i, n in enumerate((130, 120, 100)))
    s1 = m.seq_create()
    m.step_batch([(0, a, []), (s1, b[:60], [])])                # 3 + 1 pages: the pool is full
    with pytest.raises(Exception):
        m.step_batch([(s1, b[60:], [])])                        # needs a fifth page: refused, nothing changes
    assert m.seq_len(s1) == 60
    m.clear_kv_cache()                                          # sequence 0 gives its three pages back
    got_b = m.step_batch([(s1, b[60:], [len(b) - 61])])
    assert rel(got_b[0], oracle_logits(FULL, w, b)[-1]) < F32_TOL
    m.seq_free(s1)
    s2 = m.seq_create()                                         # same slot, pages that still hold b's keys in every pass
    assert s2 == s1
    got_c = m.step_batch([(s2, c[:50], []), (0, a[:64], [63])])
    got_c2 = m.step_batch([(s2, c[50:], [49])])
    assert rel(got_c2[0], oracle_logits(FULL, w, c)[-1]) < F32_TOL
    assert rel(got_c[0], oracle_logits(FULL, w, a[:64])[-1]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_window_edges_page_borders_and_the_sink_with_sharp_scores():
    import crane_b200
    cfg, w = sharp_model(41)
    m = crane_b200.GavipelModel(cfg, device=0, max_tokens=1024, max_batch=2, precision="f32")
    m.load_checkpoint((k, t.to(torch.float32).numpy()) for k, t in w.items())
    ids = tokens(330, cfg["vocab"], 42)
    want = oracle_logits(cfg, w, ids)
    got = m.step_batch([(0, ids, all_rows(330))])
    assert rel(got, want) < F32_TOL
    # decode over the borders of 32-key tiles and 64-token pages and over the places where a window's far edge leaves a page,
    # after a prompt that ends just before / on / after them
    for start in (31, 32, 33, 44, 45, 46, 63, 64, 65, 69, 70, 71, 108, 109, 110, 127, 128, 129, 133, 134, 255, 257):
        m.clear_kv_cache()
        m.step_batch([(0, ids[:start], [])])
        rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in ids[start:start + 4]])
        assert rel(rows, want[start:start + 4]) < F32_TOL, start
    # the same edges inside portions of a prompt
    for cut in (45, 70, 109, 134):
        m.clear_kv_cache()
        a = m.step_batch([(0, ids[:cut - 1], [cut - 2])])
        b = m.step_batch([(0, ids[cut - 1:cut + 40], all_rows(41))])
        assert rel(np.concatenate([a, b]), want[cut - 2:cut + 40]) < F32_TOL, cut
    m.close()


@pytest.mark.gpu
def test_first_tokens_of_a_sequence():
    m, w = make(FULL, 15, precision="f32")
    ids = tokens(6, FULL["vocab"], 16)
    want = oracle_logits(FULL, w, ids)
    assert rel(m.step_batch([(0, ids[:1], [0])]), want[:1]) < F32_TOL           # a one-token prompt: one key beside the unit term
    assert rel(m.step_batch([(0, ids[1:2], [0])]), want[1:2]) < F32_TOL
    assert rel(m.step_batch([(0, ids[2:], [0, 1, 2, 3])]), want[2:]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_long_context_decode_with_and_without_a_window():
    cfg = config([layer(mixer(scale=0.4, window=0), None), layer(mixer(scale=0.4, window=300))], loop=(0, 1, 2), width=128, vocab=150)
    m, w = make(cfg, 17, precision="f32", max_tokens=2048)
    ids = tokens(1500, cfg["vocab"], 18)
    want = oracle_logits(cfg, w, ids)
    m.step_batch([(0, ids[:1490], [])])
    rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in ids[1490:]])
    assert rel(rows, want[1490:]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_greedy_generation_through_generate_and_the_scheduler():
    from crane_b200.scheduler import BatchScheduler
    m, w = make(FULL, 19, precision="f32", max_tokens=512)

    def oracle_greedy(prompt, n):
        c = G.Cache(FULL)
        lg = oracle_logits(FULL, w, prompt, c)[-1]
        out, margins = [], []
        for _ in range(n):
            top = np.sort(lg)[-2:]
            margins.append(top[1] - top[0])
            out.append(int(lg.argmax()))
            lg = oracle_logits(FULL, w, [out[-1]], c)[-1]
        return out, min(margins)

    prompts = [tokens(n, FULL["vocab"], 50 + i) for i, n in enumerate((70, 9, 33, 130, 20, 64))]
    want = [oracle_greedy(p, 12) for p in prompts]
    assert min(mg for _, mg in want) > 1e-4                     # no decision of this test is a close call
    assert m.generate(prompts[0], max_new_tokens=12).tolist() == want[0][0]
    m.clear_kv_cache()
    sch = BatchScheduler(m, chunk=48, max_live=3, token_budget=80)
    rids = [sch.add(p, 12) for p in prompts]
    out = sch.run()
    for rid, (toks, _) in zip(rids, want):
        assert out[rid] == toks, rid
    sch = BatchScheduler(m, chunk=32, max_live=2)
    rid = sch.add(prompts[1], 6, temperature=0.8, top_k=1, seed=3)         # top-k 1 is greedy whatever the draw
    assert sch.run()[rid] == want[1][0][:6]
    m.clear_kv_cache()
    s1 = m.seq_create()
    m.step_batch([(0, prompts[2], []), (s1, prompts[4], [])])
    first = [want[2][0][0], want[4][0][0]]
    toks, _ = m.decode_batch([0, s1], first, n_steps=5)                     # the graph-replayed loop, two sequences side by side
    assert toks[0].tolist() == want[2][0][1:6] and toks[1].tolist() == want[4][0][1:6]
    m.close()


@pytest.mark.gpu
def test_wide_heads_and_many_rows_take_the_tensor_core_paths():
    # 128-wide heads, enough (row, expert) pairs for the per-expert GEMMs, a window shorter than the prompt
    cfg = config([layer(mixer(heads=4, kv_heads=2, dim=128, vdim=128, scale=0.08, window=150, rot_dims=64),
                        moe(ff=64, experts=4, top=2, count=2, keep=2, shared=96))], loop=(0, 1, 2), width=256, vocab=300)
    m, w = make(cfg, 21, precision="split")
    ids = tokens(400, cfg["vocab"], 22)
    want = oracle_logits(cfg, w, ids)
    assert rel(m.step_batch([(0, ids, all_rows(400))]), want) < SPLIT_TOL
    m.clear_kv_cache()
    a = m.step_batch([(0, ids[:333], all_rows(333))])
    b = m.step_batch([(0, ids[333:], all_rows(67))])
    assert rel(np.concatenate([a, b]), want) < SPLIT_TOL
    m.close()


def random_config(seed):
    """A layer list drawn at random: every grouping of query heads, widths that are and are not multiples of 8, windows around
    tile and page sizes, rotation of none / some / all dimensions, every shape of expert choice, every form of repeated span."""
    r = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(r.integers(len(xs)))]
    layers = []
    for _ in range(int(r.integers(1, 5))):
        g, rep = pick(1, 2, 3), pick(1, 2, 3, 5)
        d, dv = (64, 64) if r.random() < 0.3 else (pick(16, 18, 24, 40, 66), pick(8, 20, 24, 64, 70))
        rot = pick(0, 2, d // 2 * 2, (d // 4) * 2)
        mx = mixer(heads=g * rep, kv_heads=g, dim=d, vdim=dv, scale=float(pick(0.5, 1.0, 2.0)) / math.sqrt(d), window=pick(0, 1, 5, 31, 32, 33, 64, 100),
                   rot_dims=rot, base=float(pick(50.0, 1e4)), scaling=bool(r.integers(2)))
        f = None
        if r.random() < 0.75:
            E, count = pick((4, 2), (6, 3), (8, 4), (9, 1), (5, 5), (12, 3))
            keep = int(r.integers(1, count + 1))
            top = int(r.integers(1, keep * (E // count) + 1))
            f = moe(ff=pick(12, 30, 64), experts=E, top=top, count=count, keep=keep, shared=pick(0, 20, 64))
        layers.append(layer(mx, f))
    n = len(layers)
    loop = None
    if r.random() < 0.8:
        a = int(r.integers(0, n)); b = int(r.integers(a + 1, n + 1))
        loop = (a, b, pick(1, 2, 3))
    return config(layers, loop=loop, width=pick(72, 100, 136, 160), vocab=pick(90, 211, 300), scale=float(pick(1.0, 6.0)), eps=float(pick(1e-6, 1e-5)))


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(10))
def test_random_layer_lists(seed):
    cfg = random_config(100 + seed)
    r = np.random.default_rng(seed)
    ids, other = tokens(150, cfg["vocab"], 200 + seed), tokens(70, cfg["vocab"], 300 + seed)
    for precision, tol in (("f32", F32_TOL), ("split", SPLIT_TOL)):
        m, w = make(cfg, 400 + seed, precision=precision)
        want, want2 = oracle_logits(cfg, w, ids), oracle_logits(cfg, w, other)
        assert rel(m.step_batch([(0, ids, all_rows(150))]), want) < tol, (precision, "whole")
        m.clear_kv_cache()
        s1 = m.seq_create()
        at, at2, rows, rows2 = 0, 0, [], []
        while at < 150:                                      # random cuts, the second request beside some of them
            c = int(min(150 - at, r.choice([1, 2, 3, 17, 40, 64])))
            entries = [(0, ids[at:at + c], all_rows(c))]
            c2 = int(min(70 - at2, r.choice([0, 1, 2, 30])))
            if c2:
                entries.append((s1, other[at2:at2 + c2], all_rows(c2)))
            lg = m.step_batch(entries)
            rows.append(lg[:c]); rows2.append(lg[c:]); at += c; at2 += c2
        assert rel(np.concatenate(rows), want) < tol, (precision, "cuts")
        got2 = np.concatenate(rows2)
        assert rel(got2, want2[:len(got2)]) < tol, (precision, "beside")
        m.close()


@pytest.mark.gpu
def test_model_folder_loader_and_trace_runner(tmp_path):
    import json, os, subprocess, sys
    cfg = SINGLE["loop_from_the_first_layer"]
    w = G.random_weights(cfg, 23)
    hdr, blob = {}, b""
    for k, t in w.items():
        bits = G.to_numpy_bf16_bits(t).tobytes()
        hdr[k] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [len(blob), len(blob) + len(bits)]}
        blob += bits
    mdir = tmp_path / "model"; mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    h = json.dumps(hdr).encode()
    (mdir / "model.safetensors").write_bytes(len(h).to_bytes(8, "little") + h + blob)
    a, b = tokens(80, cfg["vocab"], 24), tokens(70, cfg["vocab"], 25)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [49]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [0, 67]}, {"id": "a", "tokens": a[50:51], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[51:], "want": []}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [69]}], "end": ["c"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    wa, wb = oracle_logits(cfg, w, a), oracle_logits(cfg, w, b)
    read = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    assert rel(read(0), wa[49:50]) < F32_TOL
    assert rel(read(1), np.stack([wb[2], wb[69], wa[50]])) < F32_TOL
    assert not (out / "2.f32").exists()
    assert rel(read(3), wb[69:70]) < F32_TOL                    # request c runs on the slot and pages b gave back
