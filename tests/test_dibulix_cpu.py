"""Host-side checks of the Dibulix design (no GPU): configuration reader and registry, tensor names and shapes, synthetic
weights, and the oracle's mechanisms against closed forms written out in the tests themselves."""
import json
import math

import pytest
import torch

from moshi_b200.config import DECODER_ARCHITECTURES, DecoderLMConfig, DibulixConfig
from moshi_b200.synth import iter_synth_decoder_tensors
from oracle import dibulix as D

F64 = torch.float64


def small_cfg():
    lat = {"dim": 6, "heads": 3, "kv_rank": 10, "mask": {"size": 5}, "rot_dim": 4, "scale": 0.3, "vdim": 5,
           "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "fast": 4.0, "original": 64, "slow": 0.5}}}
    left = {"dim": 6, "heads": 4, "kv_heads": 2, "mask": {"size": 7}, "rot": {"base": 50.0, "dims": 4}, "scale": 0.4, "vdim": 3}
    return {"architecture": "Dibulix", "logit_scale": 0.5, "norm": {"eps": 1e-5}, "streams": 3, "vocab": 31, "width": 12,
            "layers": [{"type": "channel_delta", "mixer": {"conv": 3, "dim": 4, "heads": 4, "kv_heads": 2, "vdim": 3}, "mlp": {"ff": 9, "kind": "dense"}},
                       {"type": "latent_attention", "mixer": lat, "mlp": None},
                       {"type": "parallel", "mixer": {"left": left, "left_scale": 1.3, "right": {"width": 14}, "right_scale": 0.7}, "mlp": {"ff": 11, "kind": "dense"}}]}


def test_configuration_round_trip_and_registry():
    raw = small_cfg()
    cfg = DecoderLMConfig.from_dict(raw)
    assert isinstance(cfg, DibulixConfig) and DECODER_ARCHITECTURES["Dibulix"] is DibulixConfig
    assert cfg.block == "pre_norm_streams" and cfg.streams == 3 and cfg.logit_scale == 0.5 and cfg.tied_head
    d, l, p = cfg.layers
    assert d.a.kind == "channel_delta" and d.a.conv == 3 and d.a.kv_heads == 2 and d.mlp_kind == "dense" and d.ff == 9
    assert l.a.kind == "latent_attention" and l.a.rot_dims == 4 and l.a.window == 5 and l.a.sink == "none" and l.a.head_gate and l.a.rot_pairing == "halves"
    assert l.a.rot_scaling_kind == "ramp" and l.mlp_kind is None
    assert p.a.kind == "window_attention" and p.a.bias and p.a.sink == "unit" and p.a.rot_pairing == "adjacent" and p.a.window == 7
    assert p.b.kind == "mingru" and p.b.dim == 14 and p.a_scale == 1.3 and p.b_scale == 0.7
    assert json.loads(json.dumps(cfg.to_dict())) == raw
    from moshi_b200.models.loaders import model_class
    assert model_class(raw).__name__ == "DecoderLM"
    plain = small_cfg()
    del plain["streams"]
    assert DecoderLMConfig.from_dict(plain).streams == 0 and "streams" not in DecoderLMConfig.from_dict(plain).to_dict()
    for bad_type in ("mlstm", "delta"):
        bad = small_cfg()
        bad["layers"][0]["type"] = bad_type
        with pytest.raises((ValueError, KeyError)):
            DecoderLMConfig.from_dict(bad)
    bad = small_cfg()
    bad["layers"][1]["mixer"]["rot"]["dims"] = 2
    with pytest.raises(ValueError):
        DecoderLMConfig.from_dict(bad)


def test_tensor_names_and_synthetic_weights():
    cfg = DecoderLMConfig.from_dict(small_cfg())
    cfg.layers[0].a.decay_rank, cfg.layers[0].a.gate_rank = 5, 6
    s = cfg.tensor_shapes()
    assert s["l0.mix.q"] == (8, 12) and s["l0.mix.v"] == (12, 12) and s["l0.mix.k.conv"] == (8, 3) and s["l0.mix.a1"] == (5, 12) and s["l0.mix.a2"] == (16, 5)
    assert s["l0.mix.dt_bias"] == (16,) and s["l0.mix.g1"] == (6, 12) and s["l0.mix.g2"] == (12, 6) and s["l0.mix.b"] == (4, 12) and s["l0.mix.norm"] == (3,)
    assert s["l1.mix.q"] == (30, 12) and s["l1.mix.dkv"] == (14, 12) and s["l1.mix.dkv.norm"] == (10,) and s["l1.mix.uk"] == (18, 10) and s["l1.mix.uv"] == (15, 10)
    assert s["l1.mix.g"] == (3, 12) and "l1.norm2" not in s and "l1.hc2.in" not in s and s["l1.hc1.mix"] == (3, 3)
    assert s["l2.mix.left.q"] == (24, 12) and s["l2.mix.left.k.b"] == (12,) and s["l2.mix.left.v"] == (6, 12) and s["l2.mix.right.z"] == (14, 12)
    assert s["l2.mix.right.x.b"] == (14,) and s["l2.mix.right.o"] == (12, 14) and s["l2.hc2.out"] == (3,) and s["l2.mlp.down"] == (12, 11)
    assert "head" not in s and s["final.norm"] == (12,)
    t = dict(iter_synth_decoder_tensors(cfg, seed=1))
    assert set(t) == set(s) and all(tuple(t[k].shape) == s[k] for k in s)
    assert abs(float(t["l0.hc1.in"].float().sum()) - 1.0) < 0.4 and float((t["l0.hc1.mix"].float() - torch.eye(3)).abs().max()) < 0.2
    o = D.Oracle(cfg.to_dict(), t)
    lg, layers = o.run([3, 1, 4, 1, 5, 9, 2, 6])
    assert lg.shape == (8, 31) and layers.shape == (3, 8, 12) and bool(torch.isfinite(lg).all())


def test_softmax_with_a_unit_in_the_denominator():
    s = torch.tensor([0.3, -1.2, 2.0], dtype=F64)
    w = D.window_softmax(s, extra_one=True)
    want = torch.exp(s) / (1.0 + torch.exp(s).sum())
    assert torch.allclose(w, want, atol=1e-15) and float(w.sum()) < 1.0
    assert torch.allclose(D.window_softmax(s, extra_one=False), torch.softmax(s, 0), atol=1e-15)
    # very negative scores: the unit takes all the weight; very large ones: it vanishes
    assert float(D.window_softmax(s - 50.0, True).sum()) < 1e-18 * 1e3 + 1e-15
    assert abs(float(D.window_softmax(s + 50.0, True).sum()) - 1.0) < 1e-12


def test_window_and_first_tokens():
    assert D.visible(0, 1, 5) == slice(0, 1) and D.visible(4, 5, 5) == slice(0, 5) and D.visible(5, 6, 5) == slice(1, 6)
    assert D.visible(9, 10, 1) == slice(9, 10) and D.visible(9, 10, None) == slice(0, 10) and D.visible(9, 10, 0) == slice(0, 10)


def test_rotations_depend_on_distance_only_and_the_ramp_by_hand():
    f, amp = D.rotary_table(8, 100.0)
    assert amp == 1.0 and torch.allclose(f, torch.tensor([100.0 ** (-2 * i / 8) for i in range(4)], dtype=F64))
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 10, generator=g, dtype=F64), torch.randn(1, 10, generator=g, dtype=F64)
    for rot in (D.rotate_adjacent, D.rotate_halves):
        a = (rot(q, 17, f) * rot(k, 11, f)).sum()
        b = (rot(q, 106, f) * rot(k, 100, f)).sum()
        assert abs(float(a - b)) < 1e-10
        assert torch.equal(rot(q, 5, f)[:, 8:], q[:, 8:])                                   # beyond the rotated dimensions
    # adjacent: (0, 1) is a pair; halves: (0, 4) is a pair
    e0 = torch.zeros(1, 10, dtype=F64)
    e0[0, 0] = 1.0
    assert abs(float(D.rotate_adjacent(e0, 1, f)[0, 1]) - math.sin(1.0)) < 1e-12 and abs(float(D.rotate_halves(e0, 1, f)[0, 4]) - math.sin(1.0)) < 1e-12
    # the ramp: base 100, 8 dims, original 64: d(t) = 8 ln(64 / (2 pi t)) / (2 ln 100)
    sc = {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 0.5}
    fs, amp = D.rotary_table(8, 100.0, sc)
    d = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(d(4.0)), 0), min(math.ceil(d(0.5)), 7)
    for i in range(4):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert abs(float(fs[i]) - (float(f[i]) / 4.0 * r + float(f[i]) * (1 - r))) < 1e-15
    assert abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-15


def test_min_gru_unrolled():
    g = torch.Generator().manual_seed(1)
    W, N = 5, 7
    p = {k: torch.randn(N, W, generator=g, dtype=F64) for k in ("z", "x", "g")}
    p.update({"z.b": torch.randn(N, generator=g, dtype=F64), "x.b": torch.randn(N, generator=g, dtype=F64), "o": torch.randn(W, N, generator=g, dtype=F64)})
    hs = torch.randn(4, W, generator=g, dtype=F64)
    st, outs = {}, []
    for t in range(4):
        outs.append(D.min_gru(p, {"width": N}, hs[t], t, st))
    # closed form of the last state: sum_t z_t c_t prod_{u > t} (1 - z_u)
    z = torch.sigmoid(hs @ p["z"].t() + p["z.b"])
    u = hs @ p["x"].t() + p["x.b"]
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = sum(z[t] * c[t] * torch.prod(1 - z[t + 1:], 0) for t in range(4))
    assert torch.allclose(st["S"], S, atol=1e-12)
    gate = hs[3] @ p["g"].t()
    assert torch.allclose(outs[3], p["o"] @ (S * gate * torch.sigmoid(gate)), atol=1e-12)
    assert bool((c > 0).all())                                                             # the candidate is positive on both branches, continuous at 0


def test_channel_delta_writes_overwrites_and_decays_per_channel():
    """Orthonormal keys, beta = 1, no decay: a write stores the value, a second write to the same key replaces it.  With a decay
    on one key channel only, what was stored under that channel's key fades while the others stay."""
    d, dv = 3, 2
    S = torch.zeros(d, dv, dtype=F64)

    def step(S, g, k, v, beta, q):
        S = g[:, None] * S
        u = beta * (v - S.t() @ k)
        S = S + torch.outer(k, u)
        return S, S.t() @ q
    e = torch.eye(d, dtype=F64)
    one = torch.ones(d, dtype=F64)
    S, o = step(S, one, e[0], torch.tensor([1.0, 2.0], dtype=F64), 1.0, e[0])
    assert torch.allclose(o, torch.tensor([1.0, 2.0], dtype=F64))
    S, o = step(S, one, e[1], torch.tensor([5.0, 6.0], dtype=F64), 1.0, e[0])
    assert torch.allclose(o, torch.tensor([1.0, 2.0], dtype=F64))
    S, o = step(S, one, e[0], torch.tensor([7.0, 8.0], dtype=F64), 1.0, e[0])
    assert torch.allclose(o, torch.tensor([7.0, 8.0], dtype=F64))                          # replaced, not added
    g = torch.tensor([0.5, 1.0, 1.0], dtype=F64)
    S, o = step(S, g, e[2], torch.zeros(dv, dtype=F64), 1.0, e[0] + e[1])
    assert torch.allclose(o, 0.5 * torch.tensor([7.0, 8.0], dtype=F64) + torch.tensor([5.0, 6.0], dtype=F64))
    # the oracle's mixer does the same steps: one head, identity-like projections are not needed, state carried in `st`
    cfg = DecoderLMConfig.from_dict(small_cfg())
    t = dict(iter_synth_decoder_tensors(cfg, seed=2))
    o1 = D.Oracle(cfg.to_dict(), t)
    toks = [3, 7, 7, 1, 0, 30, 12, 5, 9]
    whole, _ = o1.run(toks)
    st = o1.new_state()
    a, _ = o1.run(toks[:4], st)
    b, _ = o1.run(toks[4:], st)
    assert torch.equal(torch.cat([a, b]), whole)                                            # state carried over a cut


def test_streams_read_and_write():
    xs = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=F64)
    a = torch.tensor([0.5, 0.25, 0.25], dtype=F64)
    assert torch.allclose(D.hyper_read(xs, a), torch.tensor([2.5, 3.5], dtype=F64))
    M = torch.zeros(3, 3, dtype=F64)
    M[0, 1] = 1.0          # from stream 0 to stream 1
    M[2, 2] = 2.0
    y = torch.tensor([10.0, 20.0], dtype=F64)
    out = D.hyper_write(xs, M, torch.tensor([1.0, 0.0, -1.0], dtype=F64), y)
    assert torch.allclose(out, torch.tensor([[10.0, 20.0], [1.0, 2.0], [0.0, -8.0]], dtype=F64))


def test_latent_attention_equals_attention_over_expanded_keys():
    """One head, no rotation, a window of 2: the weights are a softmax over the last two positions of q . (W_uk c)."""
    g = torch.Generator().manual_seed(3)
    W, r, d, dv = 6, 4, 3, 2
    m = {"heads": 1, "dim": d, "rot_dim": 0, "vdim": dv, "kv_rank": r, "scale": 0.7, "mask": {"size": 2}}
    p = {"q": torch.randn(d, W, generator=g, dtype=F64), "dkv": torch.randn(r, W, generator=g, dtype=F64), "dkv.norm": torch.rand(r, generator=g, dtype=F64) + 0.5,
         "uk": torch.randn(d, r, generator=g, dtype=F64), "uv": torch.randn(dv, r, generator=g, dtype=F64), "g": torch.randn(1, W, generator=g, dtype=F64),
         "o": torch.eye(dv, dtype=F64)}
    hs = torch.randn(3, W, generator=g, dtype=F64)
    st = {}
    for t in range(3):
        out = D.latent_attention(p, m, hs[t], t, st, 1e-5)
    c = [D.rms_norm(p["dkv"] @ hs[t], p["dkv.norm"], 1e-5) for t in range(3)]
    q = p["q"] @ hs[2]
    s = torch.stack([q @ (p["uk"] @ c[j]) for j in (1, 2)]) * 0.7
    w = torch.softmax(s, 0)
    want = (w[0] * (p["uv"] @ c[1]) + w[1] * (p["uv"] @ c[2])) * torch.sigmoid(p["g"] @ hs[2])
    assert torch.allclose(out, want, atol=1e-12)
