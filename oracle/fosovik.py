"""CPU oracle for the Fosovik decoder -- TEST INFRASTRUCTURE ONLY (plain, slow, one function per mechanism).

Fosovik is a decoder-only model whose layer list comes from config.json: every layer normalises the residual
stream once with a Dynamic-Tanh norm and feeds that one output to a token mixer and (optionally) a feed-forward,
whose sum is added back.  Mixers: softmax attention with an attention sink, weightless QK RMS norm, a
position-dependent query temperature and no rotation (optionally reading another layer's keys / values), or a
Mamba-2 state-space layer.  Feed-forwards: a clamped gated unit or a softmax-routed mixture of GELU experts.

Notation used below (weights W are [out, in], applied as W x):
  dyt(x)          = tanh(a x) * w + b
  unit_rms(x)     = x / sqrt(mean(x^2) + eps)
  temp(p)         = 1 + c * ln(floor((p + 1) / m) + 1)
  attention row i = sum_{j<=i} e^{s_ij} v_j / (e^{sink} + sum_{j<=i} e^{s_ij}),  s_ij = scale * temp(i) q_i . k_j
  ssm             : S_t = exp(-exp(A) dt_t) S_{t-1} + dt_t B_t x_t^T ;  y_t = S_t^T C_t + D x_t

Everything runs in the dtype of the weights handed in (float64 by default in the tests), token by token or as
whole prompts; the state objects make the two forms comparable.
"""
from __future__ import annotations

import math

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------- mechanisms
def dyt_norm(x, alpha, w, b):
    """Dynamic Tanh: no mean, no variance."""
    return torch.tanh(alpha * x) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def query_temperature(pos, coef, every):
    """[S] factors for positions `pos` (integer tensor)."""
    return 1.0 + coef * torch.log(torch.floor((pos.to(torch.float64) + 1.0) / every) + 1.0)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def sink_attention(q, k, v, q_pos, scale, sink, n_rep):
    """q [S, H, d] at absolute positions q_pos [S]; k [T, G, d], v [T, G, dv] are the cached rows 0..T-1.
    Query head h reads key/value head h // n_rep.  The sink is one extra term exp(sink_h) of the denominator."""
    S, H, _ = q.shape
    T = k.shape[0]
    out = torch.zeros(S, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // n_rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale                       # [S, T]
        j = torch.arange(T)[None, :]
        s = s.masked_fill(j > q_pos[:, None], float("-inf"))
        m = torch.maximum(s.max(-1).values, sink[h].expand(S))
        e = torch.exp(s - m[:, None])
        den = e.sum(-1) + torch.exp(sink[h] - m)
        out[:, h, :] = (e @ v[:, g, :]) / den[:, None]
    return out


def causal_conv(u, w, b, window):
    """u [S, C] new inputs, window [taps-1, C] the inputs before them (zeros at the start of a sequence);
    w [C, taps] with the LAST column multiplying the current token.  -> (y [S, C], new window)."""
    taps = w.shape[1]
    full = torch.cat([window, u], 0)                                   # [taps-1+S, C]
    S = u.shape[0]
    y = torch.zeros_like(u)
    for t in range(S):
        seg = full[t:t + taps]                                         # [taps, C], last row = current token
        y[t] = (seg * w.T).sum(0) + b
    return y, full[full.shape[0] - (taps - 1):].clone() if taps > 1 else window


def ssm_scan(x, B, C, dt, A_log, D, state, heads_per_group):
    """x [S, Hm, P], B, C [S, G, N], dt [S, Hm] (after softplus), state [Hm, N, P] -> (y [S, Hm, P], state)."""
    S, Hm, P = x.shape
    st = state.clone()
    ys = []
    for t in range(S):
        y = torch.zeros(Hm, P, dtype=x.dtype)
        for h in range(Hm):
            g = h // heads_per_group
            decay = torch.exp(-torch.exp(A_log[h]) * dt[t, h])
            st[h] = decay * st[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[h] = st[h].T @ C[t, g] + D[h] * x[t, h]
        ys.append(y)
    return torch.stack(ys, 0), st


def grouped_rms(y, parts, eps):
    """y [S, inner] normalised in `parts` equal slices, each by its own root mean square."""
    S, n = y.shape
    return unit_rms(y.reshape(S, parts, n // parts), eps).reshape(S, n)


def dense_ff(h, w_gate, w_up, w_down, limit):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def route(h, w_router, top):
    """-> (indices [S, top], weights [S, top]): softmax over all experts, the `top` largest, not renormalised."""
    s = torch.softmax(h @ w_router.T, -1)
    wts, idx = torch.topk(s, top, dim=-1)
    return idx, wts


def moe_ff(h, w_router, ups, downs, top):
    idx, wts = route(h, w_router, top)
    out = torch.zeros(h.shape[0], downs[0].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            out[t] += wts[t, k] * (gelu_erf(h[t] @ ups[e].T) @ downs[e].T)
    return out


# ---------------------------------------------------------------------------------------------- the model
class SeqState:
    """What one sequence carries from call to call."""

    def __init__(self):
        self.n = 0          # tokens so far
        self.k = {}         # layer -> [T, G, d]
        self.v = {}
        self.conv = {}      # layer -> [taps-1, C]
        self.ssm = {}       # layer -> [Hm, N, P]


class FosovikOracle:
    def __init__(self, config: dict, weights: dict, dtype=torch.float64):
        self.cfg = config
        self.dt = dtype
        self.w = {}
        for k, v in weights.items():
            a = np.asarray(v)
            if a.dtype == np.uint16:                                   # raw bf16 bits
                a = (a.astype(np.uint32) << 16).view(np.float32)
            self.w[k] = torch.from_numpy(np.ascontiguousarray(a)).to(dtype if a.dtype.kind == "f" else torch.int64)
        self.eps = float(config["norm"]["eps"])
        self.layers = config["layers"]

    def new_state(self):
        return SeqState()

    def _norm(self, x, name):
        return dyt_norm(x, self.w[name + ".alpha"], self.w[name], self.w[name + ".b"])

    def _attention(self, li, h, st, pos):
        L, m, w = self.layers[li], self.layers[li]["mixer"], self.w
        p = f"l{li}.mix."
        S = h.shape[0]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        q = unit_rms((h @ w[p + "q"].T).reshape(S, H, d), self.eps)
        if "q_temp" in m and m["q_temp"]:
            q = q * query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"]).to(self.dt)[:, None, None]
        src = m.get("kv_from")
        if src is None:
            k = unit_rms((h @ w[p + "k"].T).reshape(S, G, d), self.eps)
            v = (h @ w[p + "v"].T).reshape(S, G, dv)
            st.k[li] = torch.cat([st.k[li], k], 0) if li in st.k else k
            st.v[li] = torch.cat([st.v[li], v], 0) if li in st.v else v
            src = li
        sink = w[p + "sink"] if (p + "sink") in w else torch.full((H,), float("-inf"), dtype=self.dt)
        o = sink_attention(q, st.k[src], st.v[src], pos, m["scale"], sink, H // G)
        return o.reshape(S, H * dv) @ w[p + "o"].T

    def _mamba2(self, li, h, st):
        m, w = self.layers[li]["mixer"], self.w
        p = f"l{li}.mix."
        S = h.shape[0]
        Hm, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
        inner = Hm * P
        proj = h @ w[p + "in"].T
        z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
        C_ = xbc.shape[1]
        win = st.conv.get(li, torch.zeros(taps - 1, C_, dtype=self.dt))
        cw = w[p + "conv"].reshape(C_, taps)
        xbc, st.conv[li] = causal_conv(xbc, cw, w[p + "conv.b"], win)
        xbc = silu(xbc)
        x = xbc[:, :inner].reshape(S, Hm, P)
        B = xbc[:, inner:inner + G * N].reshape(S, G, N)
        Cc = xbc[:, inner + G * N:].reshape(S, G, N)
        dt = softplus(dt + w[p + "dt_bias"])
        s0 = st.ssm.get(li, torch.zeros(Hm, N, P, dtype=self.dt))
        y, st.ssm[li] = ssm_scan(x, B, Cc, dt, w[p + "A_log"], w[p + "D"], s0, Hm // G)
        y = y.reshape(S, inner) * silu(z)
        y = grouped_rms(y, m["norm_groups"], self.eps) * w[p + "norm"]
        return y @ w[p + "o"].T

    def _ff(self, li, h):
        f, w = self.layers[li].get("mlp"), self.w
        if not f:
            return None
        p = f"l{li}.mlp."
        if f["kind"] == "dense":
            return dense_ff(h, w[p + "gate"], w[p + "up"], w[p + "down"], f["limit"])
        E = f["router"]["experts"]
        return moe_ff(h, w[p + "router"], [w[f"{p}e{e}.up"] for e in range(E)], [w[f"{p}e{e}.down"] for e in range(E)],
                      f["router"]["top"])

    def forward(self, tokens, st: SeqState, residuals: list | None = None):
        """Feeds `tokens` after what `st` already holds; -> logits [S, vocab]."""
        ids = torch.as_tensor(np.asarray(tokens, dtype=np.int64))
        S = ids.shape[0]
        pos = torch.arange(st.n, st.n + S)
        x = self.w["embed"][ids] * self.cfg["embedding"]["scale"]
        for li, L in enumerate(self.layers):
            h = self._norm(x, f"l{li}.norm1")
            mix = self._attention(li, h, st, pos) if L["type"] == "attention" else self._mamba2(li, h, st)
            ff = self._ff(li, h)
            x = x + (mix + ff if ff is not None else mix)
            if residuals is not None:
                residuals.append(x.clone())
        st.n += S
        return self._norm(x, "final.norm") @ self.w["head"].T


# ---------------------------------------------------------------------------------------------- synthetic checkpoints
def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor a Fosovik checkpoint with this config holds."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,), "final.norm.b": (W,), "final.norm.alpha": ()}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out.update({p + "norm1": (W,), p + "norm1.b": (W,), p + "norm1.alpha": ()})
        if L["type"] == "attention":
            out[p + "mix.q"] = (m["heads"] * m["dim"], W)
            if m.get("kv_from") is None:
                out[p + "mix.k"] = (m["kv_heads"] * m["dim"], W)
                out[p + "mix.v"] = (m["kv_heads"] * m["vdim"], W)
            out[p + "mix.sink"] = (m["heads"],)
            out[p + "mix.o"] = (W, m["heads"] * m["vdim"])
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out[p + "mix.in"] = (2 * inner + 2 * gn + m["heads"], W)
            out[p + "mix.conv"] = (inner + 2 * gn, m["conv"])
            out[p + "mix.conv.b"] = (inner + 2 * gn,)
            for n in ("dt_bias", "A_log", "D"):
                out[p + "mix." + n] = (m["heads"],)
            out[p + "mix.norm"] = (inner,)
            out[p + "mix.o"] = (W, inner)
        f = L.get("mlp")
        if f and f["kind"] == "dense":
            out.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        elif f:
            for e in range(f["router"]["experts"]):
                out[f"{p}mlp.e{e}.up"] = (f["expert"]["ff"], W)
                out[f"{p}mlp.e{e}.down"] = (W, f["expert"]["ff"])
            out[p + "mlp.router"] = (f["router"]["experts"], W)
    return out


def _bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return (u.astype(np.uint32) << 16).view(np.float32).reshape(np.shape(a))


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """bf16-representable float32 arrays; scales chosen so activations stay O(1) and routers / sinks / decays matter."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shp in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith(".alpha"):
            a = np.float32(rng.uniform(0.4, 0.9))
        elif leaf == "b" and "norm" in name:
            a = rng.normal(0, 0.1, shp)
        elif leaf in ("norm1", "norm") or name == "final.norm":
            a = 1.0 + rng.normal(0, 0.1, shp)
        elif leaf == "sink":
            a = rng.normal(0, 1.0, shp)
        elif leaf == "dt_bias":
            a = rng.uniform(-3.0, 0.5, shp)
        elif leaf == "A_log":
            a = rng.uniform(-1.5, 1.0, shp)
        elif leaf == "D":
            a = rng.normal(1.0, 0.3, shp)
        elif leaf == "conv":
            a = rng.normal(0, 0.5, shp)
        elif name.endswith("conv.b"):
            a = rng.normal(0, 0.1, shp)
        elif name == "embed":
            a = rng.normal(0, 1.0 / cfg["embedding"]["scale"], shp)
        elif leaf == "router":
            a = rng.normal(0, 3.0 / math.sqrt(shp[-1]), shp)
        else:
            a = rng.normal(0, 1.0 / math.sqrt(shp[-1]), shp)
        out[name] = _bf16_round(np.asarray(a, dtype=np.float32))
    return out
