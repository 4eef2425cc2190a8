"""CPU oracle for the Gavipel decoder -- TEST INFRASTRUCTURE ONLY (plain, slow, one function per mechanism).

Gavipel is a decoder-only model whose layer list comes from config.json.  A span of the list may be run several
times in a row with the same weights (every pass keeps keys / values of its own), and before each pass the stream is
mixed with the embedding output by one linear.  A layer adds `ls1 * mixer(norm1(x)) + ls2 * ff(norm2(x))` to the stream,
both branches reading the same x.  The mixer is windowed softmax attention over rotated, RMS-normalised queries and keys
with an extra `1` in the softmax denominator and a sigmoid gate on its output; the feed-forward is a mixture of
SiLU-gated experts routed by sigmoid scores with a selection bias and a limit on the groups of experts a token may use,
plus one expert that every token uses.

Notation (weights W are [out, in], applied as W x):
  rms(x)            = x / sqrt(mean(x^2) + eps)
  norm(x)           = rms(x) * (1 + w)                          (layer norms, final norm)
  head_norm(x)      = rms(x) * w                                (queries and keys, per head)
  rot(x, p)         : (x[2i], x[2i+1]) <- (x[2i] c - x[2i+1] s, x[2i+1] c + x[2i] s),  c, s = cos, sin(p f_i),  i < dims/2
  attention row i   = sum_j e^{s_ij} v_j / (1 + sum_j e^{s_ij}),  j in (i - window, i],  s_ij = scale q_i . k_j
  expert(h)         = W_down (silu(W_gate h) * (W_up h))

Everything runs in the dtype of the weights handed in (float64 in the tests), whole prompts or token by token;
`Cache` makes the two forms comparable.
"""
from __future__ import annotations

import math

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------- mechanisms
def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def head_norm(x, w, eps):
    """x [..., d]: RMS norm over the last axis with a plain weight shared by all heads."""
    return rms(x, eps) * w


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; then, per frequency, by its wavelength l = 2 pi / f against the original
    context length L: short waves (l < L/high) stay, long waves (l > L/low) are divided by `factor`, the band between
    is blended linearly in L/l."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < orig / high:
                out.append(fi)
            elif wave > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=torch.float64)


def rotate(x, pos, freqs):
    """x [S, heads, d], pos [S]; neighbouring pairs of the first 2 * len(freqs) dimensions are rotated."""
    n = 2 * freqs.numel()
    ang = pos.to(torch.float64)[:, None] * freqs[None, :]                  # [S, n/2]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def windowed_attention(q, k, v, q_pos, scale, window, n_rep):
    """q [S, H, d] at absolute positions q_pos [S]; k [T, G, d], v [T, G, dv] are the rows of positions 0..T-1.
    Row i sees j with 0 <= i - j < window.  The denominator carries one extra term e^0 that has no value."""
    S, H, _ = q.shape
    T = k.shape[0]
    out = torch.zeros(S, H, v.shape[-1], dtype=q.dtype)
    j = torch.arange(T)[None, :]
    hidden = (j > q_pos[:, None]) | (q_pos[:, None] - j >= window)
    for h in range(H):
        g = h // n_rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(hidden, float("-inf"))
        m = torch.clamp(s.max(-1).values, min=0.0)
        e = torch.exp(s - m[:, None])
        out[:, h, :] = (e @ v[:, g, :]) / (e.sum(-1) + torch.exp(-m))[:, None]
    return out


def silu(z):
    return z * torch.sigmoid(z)


def expert(h, w_gate, w_up, w_down):
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def route(h, w_router, correction, top, n_groups, keep):
    """-> (indices [S, top], weights [S, top]).  Scores are sigmoids; selection uses score + correction, restricted to the
    `keep` groups (of E / n_groups neighbouring experts) whose two largest selection scores sum highest; the weights are the
    plain scores of the chosen experts."""
    s = torch.sigmoid(h @ w_router.T)                                       # [S, E]
    c = s + correction
    S, E = c.shape
    per = E // n_groups
    gs = c.reshape(S, n_groups, per)
    gscore = torch.topk(gs, min(2, per), dim=-1).values.sum(-1)             # [S, n_groups]
    kept = torch.topk(gscore, keep, dim=-1).indices
    allowed = torch.zeros(S, n_groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    c = c.masked_fill(~allowed[:, :, None].expand(S, n_groups, per).reshape(S, E), float("-inf"))
    idx = torch.topk(c, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def moe(h, p, pre, cfg):
    r = cfg["router"]
    idx, wts = route(h, p[pre + "router"], p[pre + "correction"], r["top"], r["groups"]["count"], r["groups"]["keep"])
    out = torch.zeros(h.shape[0], p[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for kk in range(idx.shape[1]):
            e = int(idx[t, kk])
            out[t] += wts[t, kk] * expert(h[t:t + 1], p[f"{pre}e{e}.gate"], p[f"{pre}e{e}.up"], p[f"{pre}e{e}.down"])[0]
    if cfg.get("shared"):
        out = out + expert(h, p[pre + "shared.gate"], p[pre + "shared.up"], p[pre + "shared.down"])
    return out


# ---------------------------------------------------------------------------------------------- the model
def layer_runs(config):
    """The order in which layers run: [(layer index, pass index)]; layers outside the repeated span run once (pass 0)."""
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, 0) for i in range(a)]
    for t in range(times):
        runs += [(i, t) for i in range(a, b)]
    runs += [(i, 0) for i in range(b, n)]
    return runs


def pass_starts(config):
    """Indices into layer_runs() before which the stream is mixed with the embedding output: the first run of every pass
    over the repeated span (the first pass too).  Layers before and after the span are not passes."""
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return [a + t * (b - a) for t in range(times)] if b > a else []


class Cache:
    """Keys / values per layer RUN (a repeated layer keeps one set per pass)."""

    def __init__(self, config):
        self.k = [None] * len(layer_runs(config))
        self.v = [None] * len(layer_runs(config))
        self.len = 0


def attention_mixer(h, pos, p, pre, mc, eps, cache, slot):
    H, G, d, dv = mc["heads"], mc.get("kv_heads", mc["heads"]), mc["dim"], mc["vdim"]
    S = h.shape[0]
    q = (h @ p[pre + "q"].T).reshape(S, H, d)
    k = (h @ p[pre + "k"].T).reshape(S, G, d)
    v = (h @ p[pre + "v"].T).reshape(S, G, dv)
    q, k = head_norm(q, p[pre + "q.norm"], eps), head_norm(k, p[pre + "k.norm"], eps)
    rot = mc.get("rot")
    if rot and rot.get("dims", 0) > 0:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate(q, pos, f), rotate(k, pos, f)
    if cache.k[slot] is not None:
        k, v = torch.cat([cache.k[slot], k], 0), torch.cat([cache.v[slot], v], 0)
    cache.k[slot], cache.v[slot] = k, v
    window = (mc.get("mask") or {}).get("size") or (1 << 60)
    o = windowed_attention(q, k, v, pos, mc["scale"], window, H // G).reshape(S, H * dv)
    o = o * torch.sigmoid(h @ p[pre + "g"].T)
    return o @ p[pre + "o"].T


def forward(config, p, tokens, cache=None, trace=None):
    """tokens: the next tokens of one sequence -> logits [S, vocab].  `p`: name -> tensor.  `trace`, a list, receives the
    stream after every layer run."""
    cache = cache or Cache(config)
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(cache.len, cache.len + ids.numel())
    x0 = p["embed"][ids] * config["embedding"]["scale"]
    x = x0
    starts = set(pass_starts(config))
    for slot, (li, _) in enumerate(layer_runs(config)):
        if slot in starts:
            x = torch.cat([x, x0], -1) @ p["loop.in"].T
        lc, pre = config["layers"][li], f"l{li}."
        y = attention_mixer(norm_one_plus(x, p[pre + "norm1"], eps), pos, p, pre + "mix.", lc["mixer"], eps, cache, slot) * p[pre + "ls1"]
        if lc.get("mlp"):
            y = y + moe(norm_one_plus(x, p[pre + "norm2"], eps), p, pre + "mlp.", lc["mlp"]) * p[pre + "ls2"]
        x = x + y
        if trace is not None:
            trace.append(x.clone())
    cache.len += ids.numel()
    return norm_one_plus(x, p["final.norm"], eps) @ p["embed"].T


# ---------------------------------------------------------------------------------------------- random models for tests
def tensor_shapes(config):
    W, V = config["width"], config["vocab"]
    out = {"embed": (V, W), "loop.in": (W, 2 * W), "final.norm": (W,)}
    for i, lc in enumerate(config["layers"]):
        m, pre = lc["mixer"], f"l{i}."
        H, G, d, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
        out.update({pre + "norm1": (W,), pre + "ls1": (W,), pre + "mix.q": (H * d, W), pre + "mix.k": (G * d, W), pre + "mix.v": (G * dv, W),
                    pre + "mix.q.norm": (d,), pre + "mix.k.norm": (d,), pre + "mix.g": (H * dv, W), pre + "mix.o": (W, H * dv)})
        f = lc.get("mlp")
        if f:
            F, E = f["expert"]["ff"], f["router"]["experts"]
            out.update({pre + "norm2": (W,), pre + "ls2": (W,), pre + "mlp.router": (E, W), pre + "mlp.correction": (E,)})
            for e in range(E):
                out.update({f"{pre}mlp.e{e}.gate": (F, W), f"{pre}mlp.e{e}.up": (F, W), f"{pre}mlp.e{e}.down": (W, F)})
            if f.get("shared"):
                Fs = f["shared"]["ff"]
                out.update({pre + "mlp.shared.gate": (Fs, W), pre + "mlp.shared.up": (Fs, W), pre + "mlp.shared.down": (W, Fs)})
    return out


def random_weights(config, seed=0):
    """bf16-representable float64 tensors; norms and scales around their neutral values, projections ~ 1/sqrt(in)."""
    g = torch.Generator().manual_seed(seed)
    p = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = torch.randn(shape, generator=g) * 0.5
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = torch.randn(shape, generator=g) * 0.1
        elif last == "norm":
            t = 1.0 + torch.randn(shape, generator=g) * 0.1
        elif last in ("ls1", "ls2"):
            t = 0.6 + torch.rand(shape, generator=g) * 0.4
        elif last == "correction":
            t = torch.randn(shape, generator=g) * 0.3
        elif last == "router":
            t = torch.randn(shape, generator=g) * (2.0 / math.sqrt(shape[-1]))
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        p[name] = t.to(torch.bfloat16).to(torch.float64)
    return p


def to_numpy_bf16_bits(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
