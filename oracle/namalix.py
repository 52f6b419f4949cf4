"""Plain, slow restatement of the Namalix decoder LM in float64: one function per mechanism, written from the equations and
sharing no code with ``moshi_b200``.  Everything runs token by token on explicit per-request state (lists of past keys and
values, the last inputs of the short convolutions, the matrices of the two recurrences), with no tiling, chunking or fused step
of any kind, so agreement with the product path checks its kernels, its cache and its state handling alike.

The design: every layer is a PARALLEL block, ``x <- x + mixer(h) + ff(h)`` with one norm ``h = rms(x) * (1 + w)`` feeding both
sublayers.  Mixers: ``attention`` (causal attention whose weights are sigmoids, not a softmax, mixed over heads after the
sigmoid, with values blended with those of the first such layer, and a gate per head), ``retention`` (a matrix memory with a
fixed decay per head) and ``delta`` (the gated delta rule behind short convolutions).  Feed-forwards: a gated dense layer
(tanh-GELU) or a routed mixture of clamped gated experts with a sigmoid router.

Notation: x residual stream [W]; h what both sublayers read; per head q, k [dim], v [vdim]; S matrix memory [dim, vdim].
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_zero_centered(x, w, eps):
    """RMS norm whose weight is stored around zero: rms_unit(x) * (1 + w)."""
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_table(dims, base, scaling):
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


def rotate_interleaved(u, pos, freqs, amp):
    """u [heads, dim]: dimension 2i turns with 2i + 1 by the angle pos * f_i, for the first 2 * len(freqs) dimensions of a head."""
    n = freqs.shape[0]
    ang = pos * freqs
    c, s = torch.cos(ang) * amp, torch.sin(ang) * amp
    out = u.clone()
    a, b = u[:, 0:2 * n:2], u[:, 1:2 * n:2]
    out[:, 0:2 * n:2] = a * c - b * s
    out[:, 1:2 * n:2] = b * c + a * s
    return out


def rotate_halves(u, pos, freqs, amp):
    """u [heads, dim]: dimension i turns with i + len(freqs)."""
    n = freqs.shape[0]
    ang = pos * freqs
    c, s = torch.cos(ang) * amp, torch.sin(ang) * amp
    out = u.clone()
    a, b = u[:, :n], u[:, n:2 * n]
    out[:, :n] = a * c - b * s
    out[:, n:2 * n] = b * c + a * s
    return out


def sigmoid_attention(q, keys, values, scale, softcap, bias, talk):
    """One query token.  q [H, dim]; keys / values: lists of [G, dim] / [G, vdim] for positions 0 .. pos (all are seen).
    score = q . k * scale, capped by softcap * tanh(. / softcap) when a cap is given; weight = sigmoid(score + bias[h]), no
    normalisation over keys; the weights are then mixed over heads, w'[h] = sum_g talk[h, g] w[g], and head h applies its mixed
    weights to the values of its own key/value head."""
    H, G = q.shape[0], keys[0].shape[0]
    rep = H // G
    k, v = torch.stack(keys), torch.stack(values)                               # [n, G, dim], [n, G, vdim]
    s = torch.stack([(k[:, h // rep] @ q[h]) * scale for h in range(H)])        # [H, n]
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    w = talk @ torch.sigmoid(s + bias[:, None])
    return torch.stack([w[h] @ v[:, h // rep] for h in range(H)])               # [H, vdim]


def retention_step(S, q, k, v, decay):
    """S [heads, dim, vdim] <- decay[h] S + k v^T;  o = S^T q."""
    S = decay[:, None, None] * S + k[:, :, None] * v[:, None, :]
    return S, torch.einsum("hdv,hd->hv", S, q)


def short_conv_step(history, u, w):
    """One step of a per-channel causal convolution.  ``history``: the earlier inputs (newest last; what lies in front of the
    sequence is zero); w [C, taps], the newest input meets the last tap."""
    taps = w.shape[1]
    y = w[:, taps - 1] * u
    for back in range(1, taps):
        if back <= len(history):
            y = y + w[:, taps - 1 - back] * history[-back]
    return y


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule_step(S, q, k, v, beta, g):
    """Gated delta rule per head: S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q (the read sees the new write)."""
    S = g[:, None, None] * S
    u = beta[:, None] * (v - torch.einsum("hdv,hd->hv", S, k))
    S = S + k[:, :, None] * u[:, None, :]
    return S, torch.einsum("hdv,hd->hv", S, q)


def dense_ff(h, gate, up, down):
    return down @ (gelu_tanh(gate @ h) * (up @ h))


def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(gate @ h, max=limit)
    u = torch.clamp(up @ h, -limit, limit)
    return down @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def sigmoid_router(h, router, correction, top, out_scale):
    """Scores s = sigmoid(router h).  The ``top`` experts with the largest s + correction are chosen (ties: the lower index); their
    weights are their s (without the correction) divided by the sum of the chosen s, times ``out_scale``."""
    s = torch.sigmoid(router @ h)
    choice = s + correction
    order = sorted(range(s.shape[0]), key=lambda e: (-float(choice[e]), e))[:top]
    den = sum(s[e] for e in order) + 1e-20
    return [(e, s[e] / den * out_scale) for e in order]


class NamalixOracle:
    """Whole model.  ``cfg`` is the raw ``config.json`` dictionary; ``forward`` takes new tokens of ONE request on top of ``state``."""

    def __init__(self, cfg: dict, tensors):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in dict(tensors).items()}
        self.eps = float(cfg["norm"]["eps"])
        self.rot = {}
        self.vmix_first = None
        for i, L in enumerate(cfg["layers"]):
            rot = L["mixer"].get("rot")
            if rot and int(rot.get("dims", 0)) > 0:
                self.rot[i] = rotary_table(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
            if L["type"] == "attention" and L["mixer"].get("v_mix") and self.vmix_first is None:
                self.vmix_first = i

    def new_state(self):
        st = {"pos": 0, "layers": []}
        for L in self.cfg["layers"]:
            m = L["mixer"]
            if L["type"] == "attention":
                st["layers"].append({"keys": [], "values": []})
            elif L["type"] == "retention":
                st["layers"].append({"S": torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=F64)})
            else:
                st["layers"].append({"S": torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=F64), "q": [], "k": [], "v": []})
        return st

    def _attention(self, i, m, h, pos, st, shared):
        W, p = self.W, f"l{i}.mix."
        H, G, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        q, k, v = (W[p + "q"] @ h).view(H, dim), (W[p + "k"] @ h).view(G, dim), (W[p + "v"] @ h).view(G, vdim)
        if i in self.rot:
            f, amp = self.rot[i]
            q, k = rotate_interleaved(q, pos, f, amp), rotate_interleaved(k, pos, f, amp)
        if m.get("v_mix"):
            if i == self.vmix_first:
                shared["v_first"] = v
            else:
                lam = W[p + "vmix"]
                v = (1.0 - lam) * v + lam * shared["v_first"]
        st["keys"].append(k)
        st["values"].append(v)
        o = sigmoid_attention(q, st["keys"], st["values"], float(m["scale"]), float(m.get("softcap") or 0.0), W[p + "pb"], W[p + "talk"])
        o = o * torch.sigmoid(W[p + "g"] @ h)[:, None]
        return W[p + "o"] @ o.reshape(-1)

    def _retention(self, i, m, h, pos, st):
        W, p = self.W, f"l{i}.mix."
        H, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        q, k, v = (W[p + "q"] @ h).view(H, dim), (W[p + "k"] @ h).view(H, dim), (W[p + "v"] @ h).view(H, vdim)
        if i in self.rot:
            f, amp = self.rot[i]
            q, k = rotate_halves(q, pos, f, amp), rotate_halves(k, pos, f, amp)
        k = k * dim ** -0.5
        st["S"], o = retention_step(st["S"], q, k, v, torch.tensor([float(d) for d in m["decay"]], dtype=F64))
        o = rms_unit(o, self.eps).reshape(-1) * torch.nn.functional.silu(W[p + "g"] @ h)
        return W[p + "o"] @ o

    def _delta(self, i, m, h, st):
        W, p = self.W, f"l{i}.mix."
        H, G, dim, vdim, taps = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"])
        proj = {}
        for name in ("q", "k", "v"):
            u = W[p + name] @ h
            proj[name] = torch.nn.functional.silu(short_conv_step(st[name], u, W[p + name + ".conv"]))
            st[name].append(u)
            while len(st[name]) > taps - 1:
                del st[name][0]
        rep = H // G
        q = unit_vector(proj["q"].view(G, dim)) * dim ** -0.5
        k = unit_vector(proj["k"].view(G, dim))
        q, k = q.repeat_interleave(rep, 0), k.repeat_interleave(rep, 0)          # head h reads q/k head h // rep
        v = proj["v"].view(H, vdim)
        beta = torch.sigmoid(W[p + "b"] @ h)
        g = torch.exp(-torch.exp(W[p + "A_log"]) * torch.nn.functional.softplus(W[p + "a"] @ h + W[p + "dt_bias"]))
        st["S"], o = delta_rule_step(st["S"], q, k, v, beta, g)
        o = (rms_unit(o, self.eps) * W[p + "norm"]).reshape(-1) * torch.nn.functional.silu(W[p + "g"] @ h)
        return W[p + "o"] @ o

    def _ff(self, i, mlp, h):
        W, p = self.W, f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return dense_ff(h, W[p + "gate"], W[p + "up"], W[p + "down"])
        r = mlp["router"]
        picks = sigmoid_router(h, W[p + "router"], W[p + "correction"], int(r["top"]), float(r["scale"]))
        lim = float(mlp["expert"]["limit"])
        return sum(w * clamped_expert(h, W[p + f"e{e}.gate"], W[p + f"e{e}.up"], W[p + f"e{e}.down"], lim) for e, w in picks)

    def _token(self, tok, state, layers_out):
        cfg, W, eps = self.cfg, self.W, self.eps
        pos = state["pos"]
        x = W["embed"][tok] * float(cfg["embedding"]["scale"])
        shared = {}
        for i, L in enumerate(cfg["layers"]):
            st = state["layers"][i]
            h = norm_zero_centered(x, W[f"l{i}.norm1"], eps)
            if L["type"] == "attention":
                y = self._attention(i, L["mixer"], h, pos, st, shared)
            elif L["type"] == "retention":
                y = self._retention(i, L["mixer"], h, pos, st)
            else:
                y = self._delta(i, L["mixer"], h, st)
            if L.get("mlp") is not None:
                y = y + self._ff(i, L["mlp"], h)
            x = x + y
            layers_out.append(x)
        state["pos"] = pos + 1
        return W["head"] @ norm_zero_centered(x, W["final.norm"], eps)

    def forward(self, tokens, state=None, return_layers=False):
        state = self.new_state() if state is None else state
        logits, layers = [], []
        for t in tokens:
            per = []
            logits.append(self._token(int(t), state, per))
            layers.append(torch.stack(per))
        logits = torch.stack(logits)
        return (logits, torch.stack(layers, 1)) if return_layers else logits          # layers: [layer, token, W]

    def greedy(self, prompt, n_new):
        """(tokens, top-2 logit gaps) of greedy decoding."""
        st = self.new_state()
        lg = self.forward(prompt, st)[-1]
        out, gaps = [], []
        for _ in range(n_new):
            top = torch.topk(lg, 2).values
            out.append(int(lg.argmax()))
            gaps.append(float(top[0] - top[1]))
            lg = self.forward([out[-1]], st)[-1]
        return out, gaps
