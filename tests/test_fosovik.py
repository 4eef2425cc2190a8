"""Fosovik (layer-list decoder on ragged-batch steps) against the plain oracle of oracle/fosovik.py.

Small configurations with their own random weights; the oracle runs in float64.  The engine's "f32" precision is held to a
tight bar (any lost key, wrong edge or stale state shows), the serving precisions to the bar their operand rounding allows.
"""
import numpy as np
import pytest
import torch

from oracle.fosovik import (FosovikOracle, causal_conv, dense_ff, dyt_norm, grouped_rms, moe_ff, query_temperature, random_weights,
                            sink_attention, ssm_scan, unit_rms)

# ---------------------------------------------------------------------------------------------------- configurations
ATT = {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 40, "vdim": 24, "scale": 0.9,
                                      "q_temp": {"coef": 0.4, "every": 16}}, "mlp": None}
ATT_PLAIN = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 18, "vdim": 36, "scale": 0.3}, "mlp": None}
SSM = {"type": "mamba2", "mixer": {"heads": 6, "vdim": 20, "state": 24, "groups": 3, "conv": 4, "norm_groups": 2}, "mlp": None}
SSM1 = {"type": "mamba2", "mixer": {"heads": 2, "vdim": 34, "state": 9, "groups": 1, "conv": 2, "norm_groups": 4}, "mlp": None}
DENSE = {"kind": "dense", "ff": 200, "limit": 1.5}
MOE = {"kind": "moe", "expert": {"ff": 48}, "router": {"experts": 6, "top": 2}}
MOE1 = {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 5, "top": 1}}


def layer(mixer, mlp=None, **mixer_extra):
    m = dict(mixer["mixer"], **mixer_extra)
    return {"type": mixer["type"], "mixer": m, "mlp": mlp}


def config(layers, width=160, vocab=300, scale=7.0, eps=1e-5):
    return {"architecture": "Fosovik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": layers}


FULL = config([layer(ATT, MOE), layer(SSM, DENSE), layer(SSM1, MOE1), layer(ATT, None, kv_from=0), layer(ATT_PLAIN, DENSE),
               layer(SSM, MOE)])
SINGLE = {
    "attention": config([layer(ATT)]),
    "attention_plain": config([layer(ATT_PLAIN)], width=96, vocab=128),
    "mamba2": config([layer(SSM)]),
    "mamba2_one_group": config([layer(SSM1)], width=64, vocab=77),
    "dense": config([layer(ATT_PLAIN, DENSE)]),
    "moe": config([layer(ATT_PLAIN, MOE)]),
    "moe_top1": config([layer(SSM1, MOE1)]),
    "shared_kv": config([layer(ATT, DENSE), layer(SSM1), layer(ATT, MOE, kv_from=0)]),
}


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


F32_TOL, SPLIT_TOL = 2e-5, 2e-3


# ---------------------------------------------------------------------------------------------------- CPU: the oracle itself
def test_oracle_prefill_equals_token_by_token():
    cfg = FULL
    o = FosovikOracle(cfg, random_weights(cfg, 1))
    ids = tokens(41, cfg["vocab"], 2)
    whole = o.forward(ids, o.new_state()).numpy()
    st = o.new_state()
    parts = [o.forward(ids[a:b], st).numpy() for a, b in ((0, 7), (7, 9), (9, 10), (10, 33), (33, 41))]
    assert rel(np.concatenate(parts), whole) < 1e-11


def test_oracle_mechanisms_on_known_answers():
    # sink: one key, zero score, sink 0 -> half the value
    q = torch.zeros(1, 1, 4, dtype=torch.float64); k = torch.ones(1, 1, 4, dtype=torch.float64); v = torch.full((1, 1, 3), 2.0, dtype=torch.float64)
    out = sink_attention(q, k, v, torch.tensor([0]), 1.0, torch.zeros(1, dtype=torch.float64), 1)
    assert torch.allclose(out, torch.full((1, 1, 3), 1.0, dtype=torch.float64))
    # temperature steps every `every` positions, starting from 1
    t = query_temperature(torch.tensor([0, 14, 15, 31]), 0.5, 16)
    assert torch.allclose(t, torch.tensor([1.0, 1.0, 1 + 0.5 * np.log(2.0), 1 + 0.5 * np.log(3.0)], dtype=torch.float64))
    # conv: last column is the current token's tap
    y, win = causal_conv(torch.tensor([[1.0], [2.0], [3.0]]), torch.tensor([[10.0, 1.0]]), torch.zeros(1), torch.zeros(1, 1))
    assert y.flatten().tolist() == [1.0, 12.0, 23.0] and win.flatten().tolist() == [3.0]
    # scan with zero decay rate keeps everything: A_log -> -inf
    x = torch.ones(3, 1, 2, dtype=torch.float64); B = torch.ones(3, 1, 1, dtype=torch.float64)
    y, s = ssm_scan(x, B, B, torch.ones(3, 1, dtype=torch.float64), torch.tensor([-50.0], dtype=torch.float64), torch.zeros(1, dtype=torch.float64),
                    torch.zeros(1, 1, 2, dtype=torch.float64), 1)
    assert torch.allclose(y[:, 0, 0], torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64))
    assert torch.allclose(grouped_rms(torch.tensor([[3.0, 3.0, 1.0, 1.0]]), 2, 0.0), torch.ones(1, 4))
    assert torch.allclose(unit_rms(torch.tensor([[2.0, 2.0]]), 0.0), torch.ones(1, 2))
    assert float(dyt_norm(torch.tensor(100.0), 1.0, 2.0, 0.5)) == 2.5
    # clamp: gate above the limit saturates, up is clamped on both sides
    h = torch.eye(2, dtype=torch.float64)
    out = dense_ff(h, torch.tensor([[9.0, 0.0]], dtype=torch.float64), torch.tensor([[-9.0, 9.0]], dtype=torch.float64), torch.ones(1, 1, dtype=torch.float64), 2.0)
    g = 2.0 / (1 + np.exp(-1.702 * 2.0))
    assert abs(float(out[0]) - g * (-2.0 + 1.0)) < 1e-12 and float(out[1]) == 0.0
    # top-1 of two experts: weight is the softmax score itself, not 1
    r = torch.tensor([[2.0], [0.0]], dtype=torch.float64)
    one = [torch.ones(1, 1, dtype=torch.float64)] * 2
    out = moe_ff(torch.ones(1, 1, dtype=torch.float64), r, one, one, 1)
    s = np.exp(2.0) / (np.exp(2.0) + 1.0)
    gl = 0.5 * (1 + float(torch.erf(torch.tensor(1.0 / np.sqrt(2.0)))))
    assert abs(float(out) - s * gl) < 1e-12


# ---------------------------------------------------------------------------------------------------- GPU
def make(cfg, seed=0, **opts):
    import crane_b200
    w = random_weights(cfg, seed)
    opts.setdefault("max_tokens", 1024)
    opts.setdefault("max_batch", 4)
    m = crane_b200.FosovikModel(cfg, device=0, **opts)
    m.load_checkpoint(w.items())
    return m, FosovikOracle(cfg, w)


def all_rows(n):
    return list(range(n))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(name):
    cfg = SINGLE[name]
    m, o = make(cfg, 3, precision="f32")
    ids = tokens(70, cfg["vocab"], 4)
    got = m.step_batch([(0, ids, all_rows(70))])
    want = o.forward(ids, o.new_state()).numpy()
    assert rel(got, want) < F32_TOL
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_whole_model_prefill_and_token_by_token_decoding(precision, tol):
    m, o = make(FULL, 5, precision=precision)
    ids = tokens(150, FULL["vocab"], 6)
    want = o.forward(ids, o.new_state()).numpy()
    got = m.step_batch([(0, ids, all_rows(len(ids)))])
    assert rel(got, want) < tol
    m.clear_kv_cache()
    rows = [m.step_batch([(0, ids[:3], [0, 1, 2])])]
    rows += [m.step_batch([(0, [t], [0])]) for t in ids[3:]]       # long decoding: 147 single-token steps across two page borders
    step = np.concatenate(rows)
    assert rel(step, want) < tol
    if precision == "f32":
        assert rel(step, got) < 1e-5
    m.close()


@pytest.mark.gpu
def test_plain_bf16_precision_is_close():
    cfg = config([layer(ATT, DENSE), layer(SSM, DENSE), layer(ATT_PLAIN)])
    m, o = make(cfg, 7, precision="bf16")
    ids = tokens(90, cfg["vocab"], 8)
    got = m.step_batch([(0, ids, all_rows(90))])
    assert rel(got, o.forward(ids, o.new_state()).numpy()) < 5e-2
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("cuts", [[2, 2, 2, 61, 3, 64, 1, 1, 30, 2], [63, 1, 1, 63, 2, 36], [1] * 5 + [95, 66], [31, 33, 32, 64, 6]])
def test_portions_of_any_size_match_the_whole_prompt(cuts):
    m, o = make(FULL, 9, precision="f32")
    n = sum(cuts)
    ids = tokens(n, FULL["vocab"], 10)
    want = o.forward(ids, o.new_state()).numpy()
    at, rows = 0, []
    for c in cuts:
        rows.append(m.step_batch([(0, ids[at:at + c], all_rows(c))]))
        at += c
    assert rel(np.concatenate(rows), want) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_unequal_requests_in_one_batch_match_each_alone():
    m, o = make(FULL, 11, precision="f32", max_tokens=1024)
    lens = [97, 5, 130, 64]
    prompts = [tokens(n, FULL["vocab"], 20 + i) for i, n in enumerate(lens)]
    want = [o.forward(p, o.new_state()).numpy() for p in prompts]
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
        assert rel(g, want[i][:len(g)]) < F32_TOL, i
    m.close()


@pytest.mark.gpu
def test_pages_and_slots_are_used_again():
    m, o = make(FULL, 13, precision="f32", max_tokens=256, max_batch=2)        # 4 pages, 2 slots
    a, b, c = (tokens(n, FULL["vocab"], 30 + i) for i, n in enumerate((130, 120, 100)))
    s1 = m.seq_create()
    m.step_batch([(0, a, []), (s1, b[:60], [])])                # 3 + 1 pages: the pool is full
    with pytest.raises(Exception):
        m.step_batch([(s1, b[60:], [])])                        # needs a fifth page: refused, nothing changes
    assert m.seq_len(s1) == 60
    m.clear_kv_cache()                                          # sequence 0 gives its three pages back
    got_b = m.step_batch([(s1, b[60:], [len(b) - 61])])
    assert rel(got_b[0], o.forward(b, o.new_state()).numpy()[-1]) < F32_TOL
    m.seq_free(s1)
    s2 = m.seq_create()                                         # same slot, dirty pages and state from b
    assert s2 == s1
    got_c = m.step_batch([(s2, c[:50], []), (0, a[:64], [63])])
    got_c2 = m.step_batch([(s2, c[50:], [49])])
    assert rel(got_c2[0], o.forward(c, o.new_state()).numpy()[-1]) < F32_TOL
    assert rel(got_c[0], o.forward(a[:64], o.new_state()).numpy()[-1]) < F32_TOL
    m.close()


def sharp_attention_model(seed, **opts):
    """Scores with a spread of several units: every query looks at one or two keys anywhere in the context, and the sink is a
    real competitor, so a lost key, a shifted edge or a missing sink moves the logits by O(1)."""
    att = layer(ATT, None, scale=1.6, q_temp={"coef": 0.7, "every": 8})
    cfg = config([att, layer(ATT, DENSE, kv_from=0, scale=1.2)], width=128, vocab=200)
    import crane_b200
    w = random_weights(cfg, seed)
    w["l0.mix.sink"] = np.asarray([6.0, -2.0, 4.0, 0.5, 8.0, 2.0, -5.0, 3.0], np.float32)
    w["l1.mix.sink"] = w["l0.mix.sink"][::-1].copy()
    m = crane_b200.FosovikModel(cfg, device=0, max_tokens=1024, max_batch=2, **opts)
    m.load_checkpoint(w.items())
    return cfg, w, m, FosovikOracle(cfg, w)


@pytest.mark.gpu
def test_far_keys_page_borders_and_the_sink_with_sharp_scores():
    cfg, w, m, o = sharp_attention_model(41, precision="f32")
    ids = tokens(330, cfg["vocab"], 42)
    want = o.forward(ids, o.new_state()).numpy()
    # the oracle itself must see the effects this test is about
    no_sink = dict(w); no_sink["l0.mix.sink"] = np.full(8, -60.0, np.float32)
    assert rel(FosovikOracle(cfg, no_sink).forward(ids[:40], o.new_state()).numpy(), want[:40]) > 1e-2
    st = o.new_state(); o.forward(ids[:200], st)
    st.k[0][5] = 0; st.v[0][5] = 0                                # lose one far key
    assert rel(o.forward(ids[200:], st).numpy(), want[200:]) > 1e-3
    got = m.step_batch([(0, ids, all_rows(330))])
    assert rel(got, want) < F32_TOL
    # decode over the borders of 32-key tiles and 64-token pages, after a prompt that ends just before / on / after them
    for start in (31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 257):
        m.clear_kv_cache()
        m.step_batch([(0, ids[:start], [])])
        rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in ids[start:start + 4]])
        assert rel(rows, want[start:start + 4]) < F32_TOL, start
    m.close()


@pytest.mark.gpu
def test_first_tokens_of_a_sequence():
    m, o = make(FULL, 15, precision="f32")
    ids = tokens(6, FULL["vocab"], 16)
    want = o.forward(ids, o.new_state()).numpy()
    assert rel(m.step_batch([(0, ids[:1], [0])]), want[:1]) < F32_TOL           # a one-token prompt: empty conv window, one key
    assert rel(m.step_batch([(0, ids[1:2], [0])]), want[1:2]) < F32_TOL
    assert rel(m.step_batch([(0, ids[2:], [0, 1, 2, 3])]), want[2:]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_long_context_decode_uses_split_keys():
    cfg = config([layer(ATT, DENSE, scale=1.4), layer(SSM)], width=128, vocab=150)
    m, o = make(cfg, 17, precision="f32", max_tokens=2048)
    ids = tokens(1500, cfg["vocab"], 18)
    want = o.forward(ids, o.new_state()).numpy()
    m.step_batch([(0, ids[:1490], [])])
    rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in ids[1490:]])
    assert rel(rows, want[1490:]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_greedy_generation_through_generate_and_the_scheduler():
    from crane_b200.scheduler import BatchScheduler
    m, o = make(FULL, 19, precision="f32", max_tokens=512)

    def oracle_greedy(prompt, n):
        st = o.new_state()
        lg = o.forward(prompt, st).numpy()[-1]
        out, margins = [], []
        for _ in range(n):
            top = np.sort(lg)[-2:]
            margins.append(top[1] - top[0])
            out.append(int(lg.argmax()))
            lg = o.forward([out[-1]], st).numpy()[-1]
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
    # sampling through the same path: temperature with top-k 1 is greedy whatever the draw
    sch = BatchScheduler(m, chunk=32, max_live=2)
    rid = sch.add(prompts[1], 6, temperature=0.8, top_k=1, seed=3)
    assert sch.run()[rid] == want[1][0][:6]
    # batched decode entry point: two sequences side by side
    m.clear_kv_cache()
    s1 = m.seq_create()
    m.step_batch([(0, prompts[2], []), (s1, prompts[4], [])][:2])
    first = [want[2][0][0], want[4][0][0]]
    toks, _ = m.decode_batch([0, s1], first, n_steps=5)
    assert toks[0].tolist() == want[2][0][1:6] and toks[1].tolist() == want[4][0][1:6]
    m.close()


@pytest.mark.gpu
def test_model_folder_loader_and_trace_runner(tmp_path):
    import json, os, struct, subprocess, sys
    cfg = SINGLE["shared_kv"]
    w = random_weights(cfg, 23)
    hdr, blob = {}, b""
    for k, a in w.items():
        bits = (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
        hdr[k] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [len(blob), len(blob) + len(bits)]}
        blob += bits
    mdir = tmp_path / "model"; mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    h = json.dumps(hdr).encode()
    (mdir / "model.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + blob)
    o = FosovikOracle(cfg, w)
    a, b = tokens(75, cfg["vocab"], 24), tokens(20, cfg["vocab"], 25)
    wa, wb = o.forward(a, o.new_state()).numpy(), o.forward(b, o.new_state()).numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": []}, {"id": "a", "tokens": a[70:71], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[71:], "want": [3]}, {"id": "b", "tokens": b[2:], "want": [17]}], "end": ["a", "b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [19]}], "end": ["c"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", SPLIT_TOL)):
        out = tmp_path / dtype
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(mdir), "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done %d" % i for i in range(4)]
        V = cfg["vocab"]
        rd = lambda i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
        assert rel(rd(0), wa[[0, 69]]) < tol and rel(rd(1), wa[[70]]) < tol
        assert rel(rd(2), np.stack([wa[74], wb[19]])) < tol and rel(rd(3), wb[[19]]) < tol


# ---------------------------------------------------------------------------------------------------- the wide paths
ATT_W = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.45,
                                        "q_temp": {"coef": 0.3, "every": 32}}, "mlp": None}
SSM_W = {"type": "mamba2", "mixer": {"heads": 4, "vdim": 64, "state": 64, "groups": 2, "conv": 4, "norm_groups": 4}, "mlp": None}
MOE_W = {"kind": "moe", "expert": {"ff": 96}, "router": {"experts": 4, "top": 2}}
WIDE = config([layer(ATT_W, MOE_W), layer(SSM_W, DENSE), layer(ATT_W, DENSE, kv_from=0)], width=256, vocab=512)


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("split", SPLIT_TOL), ("f32", F32_TOL)])
def test_tensor_core_attention_and_expert_gemms(precision, tol):
    """128-wide heads and enough (row, expert) pairs: the serving precisions take the flash kernel (sink, per-sequence pages and
    offsets) and per-expert tensor-core GEMMs; the exact mode stays on the f32 kernels.  Both against the oracle."""
    m, o = make(WIDE, 61, precision=precision, max_tokens=1024)
    a, b = tokens(400, WIDE["vocab"], 62), tokens(150, WIDE["vocab"], 63)
    wa, wb = o.forward(a, o.new_state()).numpy(), o.forward(b, o.new_state()).numpy()
    got = m.step_batch([(0, a[:300], all_rows(300))])                 # 600 pairs: expert GEMMs; 300 rows: flash
    assert rel(got, wa[:300]) < tol
    s1 = m.seq_create()
    got = m.step_batch([(0, a[300:], all_rows(100)), (s1, b[:149], all_rows(149))])   # cached prefix + a second sequence, ragged
    assert rel(got[:100], wa[300:]) < tol and rel(got[100:], wb[:149]) < tol
    # a single decoded token of one sequence (399 cached keys) beside a fresh 40-row prompt: still the many-row kernels
    c = tokens(40, WIDE["vocab"], 64)
    wc = o.forward(c, o.new_state()).numpy()
    s2 = m.seq_create()
    got = m.step_batch([(s1, b[149:], [0]), (s2, c, all_rows(40))])
    assert rel(got[:1], wb[149:]) < tol and rel(got[1:], wc) < tol
    m.close()


@pytest.mark.gpu
def test_on_device_greedy_loop_equals_step_by_step():
    m, o = make(FULL, 71, precision="f32", max_tokens=1024)
    pa, pb = tokens(50, FULL["vocab"], 72), tokens(70, FULL["vocab"], 73)

    def by_steps(p, n):
        m.clear_kv_cache()
        lg = m.step_batch([(0, p, [len(p) - 1])])
        out = []
        for _ in range(n):
            out.append(int(lg[0].argmax()))
            lg = m.step_batch([(0, [out[-1]], [0])])
        return out

    wa, wb = by_steps(pa, 40), by_steps(pb, 40)
    m.clear_kv_cache()
    assert m.generate(pa, max_new_tokens=40).tolist() == wa         # prefill + 39 replays of the decode graph across a page border
    m.clear_kv_cache()
    s1 = m.seq_create()
    m.step_batch([(0, pa, []), (s1, pb, [])])
    toks, lg = m.decode_batch([0, s1], [wa[0], wb[0]], n_steps=30, want_logits=True)
    assert toks[0].tolist() == wa[1:31] and toks[1].tolist() == wb[1:31]
    st = o.new_state(); ref = o.forward(pb + wb[:30], st).numpy()[-1]
    assert rel(lg[1], ref) < F32_TOL
    assert m.seq_len(s1) == 100 and m.kv_len() == 80
    m.close()


# ---------------------------------------------------------------------------------------------------- CPU: the scheduler's bookkeeping
class _FakeEngine:
    """Stands in for a model handle: counts pages as the engine does and hands out token t + 1 for every wanted row."""

    def __init__(self, max_tokens, max_batch):
        self.config = {"engine": {"max_tokens": max_tokens, "max_batch": max_batch}}
        self.pool, self.max_batch = max_tokens // 64, max_batch
        self.len = {0: 0}
        self.steps, self.last = [], []

    def _pages(self):
        return sum((n + 63) // 64 for n in self.len.values())

    def seq_create(self):
        s = min(i for i in range(self.max_batch) if i not in self.len)
        self.len[s] = 0
        return s

    def seq_free(self, s):
        del self.len[s]

    def seq_select(self, s):
        pass

    def clear_kv_cache(self):
        self.len[0] = 0

    def step_batch(self, entries, copy=True):
        assert len({e[0] for e in entries}) == len(entries) <= self.max_batch
        for s, toks, want in entries:
            assert s in self.len and len(toks) > 0
            self.len[s] += len(toks)
        assert self._pages() <= self.pool
        self.steps.append([(s, len(t), list(w)) for s, t, w in entries])
        self.last = [t[w_] + 1 for s, t, w in entries for w_ in w]

    def sample_rows(self, params):
        assert len(params) == len(self.last)
        return np.asarray(self.last, np.uint32)


def test_scheduler_admission_chunking_and_page_accounting():
    from crane_b200.scheduler import BatchScheduler
    eng = _FakeEngine(max_tokens=512, max_batch=3)                     # 8 pages, 3 slots
    sch = BatchScheduler(eng, chunk=50, max_live=3, token_budget=70)
    prompts = [[10] * 130, [20] * 60, [30] * 200, [40] * 5]
    rids = [sch.add(p, 4) for p in prompts]
    out = sch.run()
    # every request got its tokens: the fake feeds back last + 1, so a prompt of value v yields v + 1, v + 2, ...
    for rid, p in zip(rids, prompts):
        assert out[rid] == [p[0] + 1 + i for i in range(4)]
    for st in eng.steps:
        assert sum(n for _, n, _ in st) <= 70                          # the token budget holds in every iteration
        assert all(n <= 50 for _, n, _ in st)
    # prompt portions and single decoded tokens do share iterations
    assert any(any(n > 1 for _, n, _ in st) and any(n == 1 for _, n, _ in st) for st in eng.steps)
    assert eng.len == {0: 0}                                           # every slot but the handle's own is free again, pages returned
    with pytest.raises(ValueError):
        BatchScheduler(eng).add([], 3)
    big = BatchScheduler(eng, chunk=64)
    big.add([1] * 600, 8)                                              # larger than the whole pool
    with pytest.raises(ValueError):
        big.run()


# ---------------------------------------------------------------------------------------------------- random geometries
def random_config(seed):
    """A layer list drawn at random: widths that are and are not multiples of 8, every grouping of query heads, shared keys / values,
    one to five taps, layers without a feed-forward, experts with top-1 .. top-all."""
    r = np.random.default_rng(1000 + seed)
    pick = lambda *xs: xs[int(r.integers(len(xs)))]
    width, vocab = int(pick(72, 96, 136, 200, 264)), int(pick(61, 150, 257, 512))
    layers, att_at = [], []
    for i in range(int(r.integers(3, 7))):
        if r.random() < 0.5:
            G = int(pick(1, 2, 3)); rep = int(pick(1, 2, 3, 4, 6, 8))
            m = {"heads": G * rep, "kv_heads": G, "dim": int(pick(8, 12, 16, 24, 40, 64)), "vdim": int(pick(8, 10, 16, 24, 48)),
                 "scale": float(pick(0.2, 0.5, 1.0))}
            if r.random() < 0.6:
                m["q_temp"] = {"coef": float(pick(0.1, 0.5, 1.0)), "every": int(pick(1, 7, 32, 100))}
            same = [j for j in att_at if layers[j]["mixer"].get("kv_from") is None]
            if same and r.random() < 0.4:
                src = layers[int(pick(*same))]["mixer"]
                m.update(kv_heads=src["kv_heads"], dim=src["dim"], vdim=src["vdim"], heads=src["kv_heads"] * rep,
                         kv_from=int(next(j for j in same if layers[j]["mixer"] is src)))
            L = {"type": "attention", "mixer": m}
            att_at.append(i)
        else:
            groups = int(pick(1, 2, 3)); hp = int(pick(1, 2, 4))
            P = int(pick(4, 12, 16, 20, 40))
            ng = int(pick(1, 2, groups * hp))
            while (groups * hp * P) % ng:
                ng -= 1
            L = {"type": "mamba2", "mixer": {"heads": groups * hp, "vdim": P, "state": int(pick(4, 8, 16, 33, 64)), "groups": groups,
                                             "conv": int(pick(1, 2, 3, 4, 5)), "norm_groups": ng}}
        k = r.random()
        if k < 0.2:
            L["mlp"] = None
        elif k < 0.55:
            L["mlp"] = {"kind": "dense", "ff": int(pick(24, 100, 256, 300)), "limit": float(pick(0.5, 2.0, 7.0))}
        else:
            E = int(pick(2, 3, 8, 11))
            L["mlp"] = {"kind": "moe", "expert": {"ff": int(pick(8, 36, 64))}, "router": {"experts": E, "top": int(r.integers(1, E + 1))}}
        layers.append(L)
    return {"architecture": "Fosovik", "vocab": vocab, "width": width, "embedding": {"scale": float(pick(1.0, 4.0, 11.0))},
            "norm": {"eps": float(pick(1e-6, 1e-5, 1e-3))}, "layers": layers}


def test_random_configs_are_valid_for_the_oracle():
    for seed in range(10):
        cfg = random_config(seed)
        o = FosovikOracle(cfg, random_weights(cfg, seed))
        ids = tokens(9, cfg["vocab"], seed)
        st = o.new_state()
        a = o.forward(ids, o.new_state()).numpy()
        b = np.concatenate([o.forward(ids[:4], st).numpy(), o.forward(ids[4:], st).numpy()])
        assert np.isfinite(a).all() and rel(b, a) < 1e-10


def rows_close(got, want, tol, cfg):
    """Exact mode: every row within tol.  Serving precision: operand rounding may flip a router choice that was nearly a tie, which
    moves that row by O(1) in either implementation -- a model with experts may have a few such rows, all others must hold the bar."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want).max(-1) / np.abs(want).max()
    has_experts = any((L.get("mlp") or {}).get("kind") == "moe" for L in cfg["layers"])
    if tol <= F32_TOL or not has_experts:
        return bool((err < tol).all())
    return float((err < tol).mean()) >= 0.9


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
@pytest.mark.parametrize("seed", range(10))
def test_random_geometries_whole_chunked_and_mixed(seed, precision, tol):
    cfg = random_config(seed)
    m, o = make(cfg, seed, precision=precision, max_tokens=768, max_batch=3)
    r = np.random.default_rng(seed)
    pa, pb, pc = (tokens(int(n), cfg["vocab"], 100 * seed + i) for i, n in enumerate((r.integers(70, 200), r.integers(2, 90), r.integers(65, 140))))
    wa, wb, wc = (o.forward(p, o.new_state()).numpy() for p in (pa, pb, pc))
    assert rows_close(m.step_batch([(0, pa, all_rows(len(pa)))]), wa, tol, cfg)               # whole
    s1, s2 = m.seq_create(), m.seq_create()
    at, got = {s1: 0, s2: 0}, {s1: [], s2: []}
    src = {s1: pb, s2: pc}
    while any(at[s] < len(src[s]) for s in src):                                              # random cuts, both sequences side by side
        entries = []
        for s in src:
            left = len(src[s]) - at[s]
            if left and r.random() < 0.8:
                n = int(min(left, r.choice([1, 1, 2, 3, 17, 40, 64])))
                entries.append((s, src[s][at[s]:at[s] + n], all_rows(n)))
        if not entries:
            continue
        lg = m.step_batch(entries)
        k = 0
        for s, t, w in entries:
            got[s].append(lg[k:k + len(t)]); k += len(t); at[s] += len(t)
    assert rows_close(np.concatenate(got[s1]), wb, tol, cfg) and rows_close(np.concatenate(got[s2]), wc, tol, cfg)
    m.seq_free(s1)
    m.clear_kv_cache()                                                                        # pages and slots again, with one token at a time
    rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in pb[:20]])
    assert rows_close(rows, wb[:min(20, len(pb))], tol, cfg)
    m.close()


# ---------------------------------------------------------------------------------------------------- the ends of the supported ranges
@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_widest_heads_largest_state_many_experts(precision, tol):
    att = {"type": "attention", "mixer": {"heads": 6, "kv_heads": 1, "dim": 256, "vdim": 256, "scale": 0.3, "q_temp": {"coef": 0.2, "every": 50}}}
    ssm = {"type": "mamba2", "mixer": {"heads": 2, "vdim": 136, "state": 256, "groups": 2, "conv": 4, "norm_groups": 1}}
    ssm2 = {"type": "mamba2", "mixer": {"heads": 3, "vdim": 8, "state": 130, "groups": 1, "conv": 3, "norm_groups": 3}}
    moe = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 70, "top": 5}}
    cfg = config([dict(att, mlp=dict(DENSE)), dict(ssm, mlp=None), dict(ssm2, mlp=moe if precision == "f32" else dict(DENSE)),
                  layer(att, None, kv_from=0)], width=192, vocab=333)
    m, o = make(cfg, 81, precision=precision, max_tokens=512, max_batch=2)
    a, b = tokens(200, cfg["vocab"], 82), tokens(90, cfg["vocab"], 83)
    wa, wb = o.forward(a, o.new_state()).numpy(), o.forward(b, o.new_state()).numpy()
    s1 = m.seq_create()
    got = m.step_batch([(0, a[:150], all_rows(150)), (s1, b[:30], all_rows(30))])
    assert rel(got[:150], wa[:150]) < tol and rel(got[150:], wb[:30]) < tol
    got = m.step_batch([(0, a[150:151], [0]), (s1, b[30:], all_rows(60))])               # one decoded token beside a 60-row portion
    assert rel(got[:1], wa[150:151]) < tol and rel(got[1:], wb[30:]) < tol
    rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in a[151:160]])
    assert rel(rows, wa[151:160]) < tol
    m.close()


@pytest.mark.gpu
def test_step_batch_rejects_bad_requests_and_stays_usable():
    import crane_b200
    m, o = make(SINGLE["dense"], 91, precision="f32", max_tokens=128, max_batch=2)
    V = SINGLE["dense"]["vocab"]
    ids = tokens(10, V, 92)
    for bad in ([(0, ids, [10])],                       # wanted position past the portion
                [(0, [V], [0])],                        # token outside the vocabulary
                [(0, ids, [0]), (0, ids, [0])],         # the same sequence twice
                [(1, ids, [0])],                        # a slot nobody created
                [(0, [], [])],                          # nothing to run
                [(0, tokens(200, V, 93), [])]):         # more pages than the pool has
        with pytest.raises(crane_b200.CraneB200Error):
            m.step_batch(bad)
    assert m.seq_len(0) == 0
    assert rel(m.step_batch([(0, ids, all_rows(10))]), o.forward(ids, o.new_state()).numpy()) < F32_TOL
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_long_portions_scan_in_segments(precision, tol):
    """From 512 rows in the longest entry the Mamba-2 scan runs as four segments joined by their decay products: a long entry on a
    carried state, a short one beside it (one segment), then more rows on the states both left."""
    cfg = config([layer(SSM, DENSE), layer(SSM1), layer(ATT_PLAIN)], width=96, vocab=211)
    m, o = make(cfg, 95, precision=precision, max_tokens=1536, max_batch=2)
    a, b = tokens(900, cfg["vocab"], 96), tokens(120, cfg["vocab"], 97)
    wa, wb = o.forward(a, o.new_state()).numpy(), o.forward(b, o.new_state()).numpy()
    s1 = m.seq_create()
    m.step_batch([(0, a[:37], [])])                                                  # a state to start from
    want = [36, 37, 300, 511, 512, 700]
    got = m.step_batch([(0, a[37:740], [w - 37 for w in want[1:]]), (s1, b[:5], [4])])      # 703 rows: segments of 176
    assert rel(got[:-1], wa[want[1:]]) < tol and rel(got[-1:], wb[4:5]) < tol
    got = m.step_batch([(s1, b[5:], [114]), (0, a[740:], [0, 159])])                 # short portions again: one segment
    assert rel(got[:1], wb[119:]) < tol and rel(got[1:], wa[[740, 899]]) < tol
    m.close()
