"""Plain, slow restatement of the Dibulix decoder LM in float64: one function per mechanism, written from the equations and
sharing no code with ``moshi_b200``.  Everything runs token by token on explicit per-request state (lists of past latents, keys
and values, the last inputs of the short convolutions, the vectors and matrices of the recurrences), with no tiling, folding,
chunking or fused step of any kind, so agreement with the product path checks its kernels, its cache and its state handling alike.

The design: pre-norm sublayers (mixer, then an optional dense feed-forward) on ``streams`` residual streams.  A sublayer reads
``u = sum_s a[s] x_s``, computes ``y = f(rms(u) * w)`` and every stream becomes ``x_t <- sum_s M[s, t] x_s + b[t] y`` (all from
the old streams).  Mixers: ``latent_attention`` (keys and values expanded from a cached latent, one rotated key part shared by
the heads, a sliding window, a sigmoid gate per head), ``parallel`` (sliding-window attention whose softmax denominator holds
one extra unit, beside a minGRU) and ``channel_delta`` (the gated delta rule with one decay per key channel, behind short
convolutions).  The logits come from the embedding table itself, times a constant.

Notation: W width; per head q, k [dim], v [vdim]; S matrix memory [dim, vdim]; c latent [rank].
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def rotary_table(dims, base, scaling=None):
    """(frequencies [dims / 2], amplitude).  f_i = base^(-2i/dims).  With ``scaling`` = {factor, original, fast, slow}: the index at
    which a wave makes t turns over ``original`` positions is d(t) = dims ln(original / (2 pi t)) / (2 ln base); between
    lo = floor(d(fast)) and hi = ceil(d(slow)) (clipped to 0 .. dims - 1) a ramp goes from 0 to 1; the frequency becomes
    f_i / factor where the ramp is 1, stays f_i where it is 0, and cos and sin are both multiplied by 0.1 ln(factor) + 1."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    amp = 1.0
    if scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def d(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(d(float(scaling["fast"]))), 0)
        hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=F64), amp


def rotate_adjacent(u, pos, freqs, amp=1.0):
    """u [heads, dim]: dimension 2i turns with 2i + 1 by the angle pos * f_i, for the first 2 * len(freqs) dimensions of a head."""
    n = freqs.shape[0]
    ang = pos * freqs
    c, s = torch.cos(ang) * amp, torch.sin(ang) * amp
    out = u.clone()
    a, b = u[:, 0:2 * n:2], u[:, 1:2 * n:2]
    out[:, 0:2 * n:2] = a * c - b * s
    out[:, 1:2 * n:2] = b * c + a * s
    return out


def rotate_halves(u, pos, freqs, amp=1.0):
    """u [heads, dim]: dimension i turns with i + len(freqs)."""
    n = freqs.shape[0]
    ang = pos * freqs
    c, s = torch.cos(ang) * amp, torch.sin(ang) * amp
    out = u.clone()
    a, b = u[:, :n], u[:, n:2 * n]
    out[:, :n] = a * c - b * s
    out[:, n:2 * n] = b * c + a * s
    return out


def window_softmax(scores, extra_one):
    """Softmax over the given scores; ``extra_one`` adds a unit to the denominator (a key of score 0 that carries no value)."""
    m = scores.max(-1, keepdim=True).values
    if extra_one:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(scores - m)
    den = e.sum(-1, keepdim=True)
    if extra_one:
        den = den + torch.exp(-m)
    return e / den


def visible(pos, n_keys, window):
    """Indices j of the cached keys that position pos sees: 0 <= pos - j < window (window None: all up to pos)."""
    lo = 0 if not window else max(0, pos - window + 1)
    return slice(lo, min(pos + 1, n_keys))


def short_conv(history, taps_w):
    """history [taps, C] (zeros in front of the sequence, the current token last), taps_w [C, taps] -> [C]."""
    return (history.t() * taps_w).sum(-1)


# ---------------------------------------------------------------------------------------------------------------------------
# mixers: each takes the layer's tensors p (name after '<layer>.mix.' -> float64 tensor), the mixer's configuration m, the
# normed input h [W], the position, and the request's state for this layer (a dict that it fills)
# ---------------------------------------------------------------------------------------------------------------------------
def window_attention_sink1(p, m, h, pos, st):
    """Grouped-query sliding-window attention with biased projections, rotation of adjacent pairs, and 1 + sum in the denominator."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (p["q"] @ h + p["q.b"]).view(H, d)
    k = (p["k"] @ h + p["k.b"]).view(G, d)
    v = (p["v"] @ h + p["v.b"]).view(G, dv)
    rot = m.get("rot")
    if rot and rot.get("dims", 0) > 0:
        f, amp = rotary_table(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        q, k = rotate_adjacent(q, pos, f, amp), rotate_adjacent(k, pos, f, amp)
    st.setdefault("k", []).append(k)
    st.setdefault("v", []).append(v)
    sl = visible(pos, len(st["k"]), (m.get("mask") or {}).get("size"))
    K, V = torch.stack(st["k"][sl]), torch.stack(st["v"][sl])         # [n, G, d], [n, G, dv]
    out = torch.zeros(H, dv, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        w = window_softmax((K[:, g] @ q[hh]) * m["scale"], extra_one=True)
        out[hh] = w @ V[:, g]
    return p["o"] @ out.reshape(-1)


def min_gru(p, m, h, pos, st):
    """S <- (1 - z) S + z c, z = sigmoid(W_z h + b_z), c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0), u = W_x h + b_x;
    out = W_o (S * silu(W_g h))."""
    z = sigmoid(p["z"] @ h + p["z.b"])
    u = p["x"] @ h + p["x.b"]
    cand = torch.where(u >= 0, u + 0.5, sigmoid(u))
    S = st.get("S")
    if S is None:
        S = torch.zeros(m["width"], dtype=F64)
    S = (1.0 - z) * S + z * cand
    st["S"] = S
    return p["o"] @ (S * silu(p["g"] @ h))


def parallel_pair(p, m, h, pos, st):
    left = {k[5:]: v for k, v in p.items() if k.startswith("left.")}
    right = {k[6:]: v for k, v in p.items() if k.startswith("right.")}
    a = window_attention_sink1(left, m["left"], h, pos, st.setdefault("left", {}))
    b = min_gru(right, m["right"], h, pos, st.setdefault("right", {}))
    return m["left_scale"] * a + m["right_scale"] * b


def latent_attention(p, m, h, pos, st, eps):
    """Keys and values of every head are expanded from one cached latent; one rotated key part is shared by the heads."""
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (p["q"] @ h).view(H, d + dr)
    q_plain, q_rot = q[:, :d], q[:, d:]
    dkv = p["dkv"] @ h
    c = rms_norm(dkv[:r], p["dkv.norm"], eps)
    k_rot = dkv[r:].view(1, dr)
    rot = m.get("rot") or {}
    if dr > 0:
        f, amp = rotary_table(dr, float(rot["base"]), rot.get("scaling"))
        q_rot, k_rot = rotate_halves(q_rot, pos, f, amp), rotate_halves(k_rot, pos, f, amp)
    st.setdefault("c", []).append(c)
    st.setdefault("kr", []).append(k_rot[0])
    sl = visible(pos, len(st["c"]), (m.get("mask") or {}).get("size"))
    C, KR = torch.stack(st["c"][sl]), torch.stack(st["kr"][sl])      # [n, r], [n, dr]
    gate = sigmoid(p["g"] @ h)
    uk, uv = p["uk"].view(H, d, r), p["uv"].view(H, dv, r)
    out = torch.zeros(H, dv, dtype=F64)
    for hh in range(H):
        keys = C @ uk[hh].t()                                         # [n, d]
        vals = C @ uv[hh].t()                                         # [n, dv]
        s = (keys @ q_plain[hh] + KR @ q_rot[hh]) * m["scale"]
        out[hh] = (window_softmax(s, extra_one=False) @ vals) * gate[hh]
    return p["o"] @ out.reshape(-1)


def channel_delta(p, m, h, pos, st, eps):
    """Gated delta rule with one decay per head and key channel: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    raw = torch.cat([p["q"] @ h, p["k"] @ h, p["v"] @ h])
    hist = st.get("conv")
    if hist is None:
        hist = torch.zeros(taps, raw.shape[0], dtype=F64)
    hist = torch.cat([hist[1:], raw[None]])
    st["conv"] = hist
    w = torch.cat([p["q.conv"], p["k.conv"], p["v.conv"]])
    act = silu(short_conv(hist, w))
    q, k, v = act[:G * d].view(G, d), act[G * d:2 * G * d].view(G, d), act[2 * G * d:].view(H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigmoid(p["b"] @ h)
    g = torch.exp(-torch.exp(p["A_log"])[:, None] * softplus(p["a2"] @ (p["a1"] @ h) + p["dt_bias"]).view(H, d))
    gate = sigmoid(p["g2"] @ (p["g1"] @ h)).view(H, dv)
    S = st.get("S")
    if S is None:
        S = torch.zeros(H, d, dv, dtype=F64)
    S = S.clone()
    out = torch.zeros(H, dv, dtype=F64)
    for hh in range(H):
        gi = hh // (H // G)
        S[hh] = g[hh][:, None] * S[hh]
        u = beta[hh] * (v[hh] - S[hh].t() @ k[gi])
        S[hh] = S[hh] + torch.outer(k[gi], u)
        out[hh] = S[hh].t() @ q[gi]
    st["S"] = S
    out = rms_unit(out, eps) * p["norm"] * gate
    return p["o"] @ out.reshape(-1)


def dense_relu2(p, h):
    return p["down"] @ relu_squared(p["up"] @ h)


def hyper_read(xs, a):
    """u = sum_s a[s] x_s."""
    return (a[:, None] * xs).sum(0)


def hyper_write(xs, M, b, y):
    """x_t <- sum_s M[s, t] x_s + b[t] y, all streams from the old ones."""
    return M.t() @ xs + b[:, None] * y[None]


# ---------------------------------------------------------------------------------------------------------------------------
class Oracle:
    """cfg: the dict of config.json; tensors: name -> tensor (any float type).  ``new_state()`` per request, ``step(state, token)``
    returns (logits [vocab], [the sum of the streams after every layer])."""

    def __init__(self, cfg: dict, tensors: dict):
        self.cfg = cfg
        self.t = {k: v.detach().to("cpu", F64) for k, v in tensors.items()}
        self.eps = float(cfg["norm"]["eps"])
        self.streams = int(cfg["streams"]) if "streams" in cfg else 0

    def new_state(self):
        return {"pos": 0, "layers": [dict() for _ in self.cfg["layers"]]}

    def _sub(self, i):
        pre = f"l{i}.mix."
        return {k[len(pre):]: v for k, v in self.t.items() if k.startswith(pre)}

    def _mixer(self, i, L, h, pos, st):
        p, m = self._sub(i), L["mixer"]
        if L["type"] == "parallel":
            return parallel_pair(p, m, h, pos, st)
        if L["type"] == "latent_attention":
            return latent_attention(p, m, h, pos, st, self.eps)
        if L["type"] == "channel_delta":
            return channel_delta(p, m, h, pos, st, self.eps)
        raise ValueError(L["type"])

    def step(self, state, token):
        t, eps, pos = self.t, self.eps, state["pos"]
        x0 = t["embed"][token]
        xs = x0[None].repeat(max(self.streams, 1), 1)
        trace = []
        for i, L in enumerate(self.cfg["layers"]):
            subs = [(1, lambda h: self._mixer(i, L, h, pos, state["layers"][i]))]
            if L.get("mlp") is not None:
                subs.append((2, lambda h: dense_relu2({"up": t[f"l{i}.mlp.up"], "down": t[f"l{i}.mlp.down"]}, h)))
            for q, f in subs:
                if self.streams:
                    u = hyper_read(xs, t[f"l{i}.hc{q}.in"])
                    y = f(rms_norm(u, t[f"l{i}.norm{q}"], eps))
                    xs = hyper_write(xs, t[f"l{i}.hc{q}.mix"], t[f"l{i}.hc{q}.out"], y)
                else:
                    xs = xs + f(rms_norm(xs[0], t[f"l{i}.norm{q}"], eps))[None]
            trace.append(xs.sum(0))
        x = xs.sum(0)
        logits = (t["embed"] @ rms_norm(x, t["final.norm"], eps)) * float(self.cfg.get("logit_scale", 1.0))
        state["pos"] = pos + 1
        return logits, trace

    def run(self, tokens, state=None):
        """All tokens of one request in order -> (logits [n, vocab], layers [n_layers, n, W])."""
        state = state if state is not None else self.new_state()
        lg, tr = [], []
        for tok in tokens:
            a, b = self.step(state, int(tok))
            lg.append(a)
            tr.append(torch.stack(b))
        return torch.stack(lg), torch.stack(tr, 1)

    def forward(self, tokens, return_layers=False):
        lg, tr = self.run(tokens)
        return (lg, tr) if return_layers else lg

    def greedy(self, prompt, n_new):
        """(tokens, gap between the two largest logits at every choice)."""
        st = self.new_state()
        lg, _ = self.run(prompt, st)
        out, gaps = [], []
        for _ in range(n_new):
            top = lg[-1].topk(2).values
            nxt = int(lg[-1].argmax())
            out.append(nxt)
            gaps.append(float(top[0] - top[1]))
            lg, _ = self.run([nxt], st)
        return out, gaps
