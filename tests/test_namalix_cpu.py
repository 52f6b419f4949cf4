"""Host-side checks of the Namalix design (no GPU): configuration reader and registry, tensor names and shapes, synthetic
weights, and the oracle's mechanisms against closed forms written out in the tests themselves."""
import json
import math

import pytest
import torch

from moshi_b200.config import DECODER_ARCHITECTURES, DecoderLMConfig, NamalixConfig
from moshi_b200.synth import iter_synth_decoder_tensors
from oracle import namalix as N

F64 = torch.float64


def small_cfg():
    attn = {"dim": 6, "heads": 4, "kv_heads": 2, "scale": 0.4, "softcap": 3.0, "v_mix": True, "vdim": 5,
            "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "fast": 4.0, "original": 64, "slow": 0.5}}}
    moe = {"expert": {"ff": 7, "limit": 1.5}, "kind": "moe", "router": {"experts": 4, "scale": 1.5, "top": 2}}
    return {"architecture": "Namalix", "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "vocab": 31, "width": 12,
            "layers": [{"type": "delta", "mixer": {"conv": 3, "dim": 4, "heads": 4, "kv_heads": 2, "vdim": 3}, "mlp": {"ff": 9, "kind": "dense"}},
                       {"type": "attention", "mixer": attn, "mlp": moe},
                       {"type": "retention", "mixer": {"decay": [0.9, 0.99], "dim": 6, "heads": 2, "vdim": 4, "rot": {"base": 50.0, "dims": 6}}, "mlp": None},
                       {"type": "attention", "mixer": dict(attn, dim=8, scale=0.2), "mlp": None}]}


def test_configuration_round_trip_and_registry():
    raw = small_cfg()
    cfg = DecoderLMConfig.from_dict(raw)
    assert isinstance(cfg, NamalixConfig) and DECODER_ARCHITECTURES["Namalix"] is NamalixConfig
    assert cfg.block == "parallel_residual" and cfg.embedding_scale == 3.0
    a = cfg.layers[1].a
    assert a.kind == "sigmoid_attention" and a.rot_pairing == "adjacent" and a.rot_scaling_kind == "ramp" and a.softcap == 3.0 and a.v_mix
    assert cfg.layers[0].a.kind == "delta" and cfg.layers[0].a.conv == 3 and cfg.layers[0].mlp_kind == "gated_gelu"
    assert cfg.layers[2].a.decay == [0.9, 0.99] and cfg.layers[2].a.rot_pairing == "halves" and cfg.layers[2].mlp_kind is None
    assert cfg.layers[1].experts == 4 and cfg.layers[1].top == 2 and cfg.layers[1].expert_limit == 1.5 and cfg.layers[1].router_scale == 1.5
    assert cfg.first_v_mix_layer() == 1
    assert json.loads(json.dumps(cfg.to_dict())) == raw
    from moshi_b200.models.loaders import model_class
    assert model_class(raw).__name__ == "DecoderLM"
    for bad_type in ("mlstm", "window_attention"):
        bad = small_cfg()
        bad["layers"][0]["type"] = bad_type
        with pytest.raises((ValueError, KeyError)):
            DecoderLMConfig.from_dict(bad)
    bad = small_cfg()
    bad["layers"][2]["mixer"]["decay"] = [0.9]
    with pytest.raises(ValueError):
        DecoderLMConfig.from_dict(bad)


def test_tensor_names_and_synthetic_weights():
    cfg = DecoderLMConfig.from_dict(small_cfg())
    shapes = cfg.tensor_shapes()
    assert shapes["l0.mix.q"] == (8, 12) and shapes["l0.mix.v"] == (12, 12) and shapes["l0.mix.k.conv"] == (8, 3) and shapes["l0.mix.norm"] == (3,)
    assert shapes["l0.mix.b"] == (4, 12) and shapes["l0.mix.A_log"] == (4,) and shapes["l0.mlp.gate"] == (9, 12)
    assert shapes["l1.mix.q"] == (24, 12) and shapes["l1.mix.k"] == (12, 12) and shapes["l1.mix.v"] == (10, 12) and shapes["l1.mix.g"] == (4, 12)
    assert shapes["l1.mix.talk"] == (4, 4) and shapes["l1.mix.vmix"] == () and shapes["l1.mlp.e3.down"] == (12, 7) and shapes["l1.mlp.correction"] == (4,)
    assert shapes["l2.mix.g"] == (8, 12) and "l2.mlp.gate" not in shapes and "l2.mix.vmix" not in shapes and "final.norm.b" not in shapes
    t = dict(iter_synth_decoder_tensors(cfg, seed=1))
    assert set(t) == set(shapes) and all(tuple(t[k].shape) == tuple(shapes[k]) for k in shapes)
    assert float(t["l0.norm1"].float().abs().max()) < 0.25          # stored around zero
    orc = N.NamalixOracle(small_cfg(), t)
    lg, layers = orc.forward([1, 2, 3, 4, 5, 6, 7], return_layers=True)
    assert lg.shape == (7, 31) and layers.shape == (4, 7, 12) and torch.isfinite(lg).all()
    # state carried over a cut = the whole sequence
    st = orc.new_state()
    cut = torch.cat([orc.forward([1, 2, 3], st), orc.forward([4, 5, 6, 7], st)])
    assert torch.allclose(cut, lg, atol=1e-12)


def test_zero_centred_norm_and_gelu():
    x = torch.tensor([3.0, -4.0], dtype=F64)
    w = torch.tensor([0.5, -1.0], dtype=F64)
    y = N.norm_zero_centered(x, w, 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([3.0 / r * 1.5, 0.0], dtype=F64))
    z = torch.linspace(-4, 4, 33, dtype=F64)
    assert torch.allclose(N.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"), atol=1e-12)


def test_rotary_ramp_by_hand():
    # dims 10, base 300, original 200, fast 4, slow 0.5: index of 4 turns = 1.82 -> lo = 1; of half a turn = 3.64 -> hi = 4
    f, amp = N.rotary_table(10, 300.0, {"factor": 4.0, "original": 200, "fast": 4.0, "slow": 0.5})
    plain = [300.0 ** (-2.0 * i / 10) for i in range(5)]
    ramp = [0.0, 0.0, 1.0 / 3.0, 2.0 / 3.0, 1.0]
    want = [p / 4.0 * r + p * (1.0 - r) for p, r in zip(plain, ramp)]
    assert torch.allclose(f, torch.tensor(want, dtype=F64), rtol=1e-12)
    assert abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    f2, amp2 = N.rotary_table(6, 50.0, None)
    assert amp2 == 1.0 and torch.allclose(f2, torch.tensor([1.0, 50.0 ** (-1 / 3), 50.0 ** (-2 / 3)], dtype=F64))


def test_the_two_rotary_layouts():
    g = torch.Generator().manual_seed(0)
    u = torch.randn(2, 8, generator=g, dtype=F64)
    f = torch.tensor([1.0, 0.25], dtype=F64)
    a = N.rotate_interleaved(u, 3, f, 1.0)
    b = N.rotate_halves(u, 3, f, 1.0)
    # dimensions past the rotated ones pass unchanged; a rotation keeps the length of every pair
    assert torch.equal(a[:, 4:], u[:, 4:]) and torch.equal(b[:, 4:], u[:, 4:])
    assert torch.allclose(a[:, 0] ** 2 + a[:, 1] ** 2, u[:, 0] ** 2 + u[:, 1] ** 2)
    assert torch.allclose(b[:, 1] ** 2 + b[:, 3] ** 2, u[:, 1] ** 2 + u[:, 3] ** 2)
    c, s = math.cos(3.0), math.sin(3.0)
    assert torch.allclose(a[:, 0], u[:, 0] * c - u[:, 1] * s) and torch.allclose(a[:, 1], u[:, 1] * c + u[:, 0] * s)
    c, s = math.cos(0.75), math.sin(0.75)
    assert torch.allclose(b[:, 1], u[:, 1] * c - u[:, 3] * s) and torch.allclose(b[:, 3], u[:, 3] * c + u[:, 1] * s)
    # scores depend on the distance only: <rot(q, p), rot(k, j)> = <rot(q, p - j), k>
    q, k = u[:1], u[1:]
    for rot in (N.rotate_interleaved, N.rotate_halves):
        assert torch.allclose((rot(q, 9, f, 1.0) * rot(k, 4, f, 1.0)).sum(), (rot(q, 5, f, 1.0) * k).sum())
    # the amplitude multiplies the rotated part only
    assert torch.allclose(N.rotate_halves(u, 0, f, 1.3)[:, :4], 1.3 * u[:, :4]) and torch.equal(N.rotate_halves(u, 0, f, 1.3)[:, 4:], u[:, 4:])


def test_sigmoid_attention_by_hand():
    q = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=F64)                       # two heads on one key/value head
    keys = [torch.tensor([[1.0, 1.0]], dtype=F64), torch.tensor([[-3.0, 0.5]], dtype=F64)]
    values = [torch.tensor([[1.0, 0.0, 2.0]], dtype=F64), torch.tensor([[0.0, 4.0, -1.0]], dtype=F64)]
    bias = torch.tensor([0.1, -0.2], dtype=F64)
    talk = torch.tensor([[1.0, 0.5], [-0.25, 2.0]], dtype=F64)
    cap = 1.5
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    s = [[0.5 * 1.0, 0.5 * -3.0], [0.5 * 2.0, 0.5 * 1.0]]
    w = [[sig(cap * math.tanh(s[h][j] / cap) + float(bias[h])) for j in range(2)] for h in range(2)]
    mixed = [[sum(float(talk[h, g]) * w[g][j] for g in range(2)) for j in range(2)] for h in range(2)]
    want = torch.tensor([[mixed[h][0] * float(values[0][0, c]) + mixed[h][1] * float(values[1][0, c]) for c in range(3)] for h in range(2)], dtype=F64)
    got = N.sigmoid_attention(q, keys, values, 0.5, cap, bias, talk)
    assert torch.allclose(got, want, atol=1e-14)
    # no normalisation over keys: a second key adds to the first one's share, it does not take from it
    one = N.sigmoid_attention(q, keys[:1], values[:1], 0.5, cap, bias, talk)
    only_second = N.sigmoid_attention(q, keys[1:], values[1:], 0.5, cap, bias, talk)
    assert torch.allclose(got, one + only_second, atol=1e-14)
    # no cap: the raw score enters the sigmoid
    raw = N.sigmoid_attention(q, keys[:1], values[:1], 0.5, 0.0, bias, torch.eye(2, dtype=F64))
    assert torch.allclose(raw[0], sig(0.5 + 0.1) * values[0][0])


def test_retention_unrolled():
    g = torch.Generator().manual_seed(1)
    T, H, D, V = 7, 2, 3, 4
    q, k, v = (torch.randn(T, H, n, generator=g, dtype=F64) for n in (D, D, V))
    decay = torch.tensor([0.5, 0.9], dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64)
    for t in range(T):
        S, o = N.retention_step(S, q[t], k[t], v[t], decay)
        want = sum((decay ** (t - j))[:, None] * (q[t] * k[j]).sum(-1, keepdim=True) * v[j] for j in range(t + 1))
        assert torch.allclose(o, want, atol=1e-12)


def test_short_convolution_against_the_sum():
    g = torch.Generator().manual_seed(2)
    u = torch.randn(9, 3, generator=g, dtype=F64)
    w = torch.randn(3, 4, generator=g, dtype=F64)
    hist = []
    for t in range(9):
        y = N.short_conv_step(hist, u[t], w)
        want = sum(w[:, 3 - b] * u[t - b] for b in range(4) if t - b >= 0)
        assert torch.allclose(y, want, atol=1e-13)
        hist.append(u[t])
        hist = hist[-3:]


def test_delta_rule_writes_and_overwrites():
    # orthonormal keys, beta = 1, no decay: reading with a key returns the value last written under it
    k = torch.eye(3, dtype=F64)[None]                                           # [1 head, 3 keys, dim 3]
    S = torch.zeros(1, 3, 2, dtype=F64)
    one, g = torch.ones(1, dtype=F64), torch.ones(1, dtype=F64)
    vals = [torch.tensor([[1.0, 2.0]], dtype=F64), torch.tensor([[-1.0, 0.5]], dtype=F64), torch.tensor([[7.0, 7.0]], dtype=F64)]
    S, o = N.delta_rule_step(S, k[:, 0], k[:, 0], vals[0], one, g)
    assert torch.allclose(o, vals[0])                                           # the read-out sees the write of the same token
    S, o = N.delta_rule_step(S, k[:, 0], k[:, 1], vals[1], one, g)
    assert torch.allclose(o, vals[0])                                           # querying key 0 still returns its value
    S, o = N.delta_rule_step(S, k[:, 0], k[:, 0], vals[2], one, g)
    assert torch.allclose(o, vals[2])                                           # overwritten, not added
    # beta = 0.5 moves half way; the decay shrinks what was stored before the write
    S, o = N.delta_rule_step(S, k[:, 0], k[:, 0], torch.zeros(1, 2, dtype=F64), 0.5 * one, g)
    assert torch.allclose(o, 0.5 * vals[2])
    S, o = N.delta_rule_step(S, k[:, 1], k[:, 2], torch.zeros(1, 2, dtype=F64), one, 0.25 * g)
    assert torch.allclose(o, 0.25 * vals[1])
    u = N.unit_vector(torch.tensor([[3.0, 4.0]], dtype=F64))
    assert torch.allclose(u, torch.tensor([[0.6, 0.8]], dtype=F64), atol=1e-6)


def test_router_and_clamped_expert():
    h = torch.tensor([1.0, -1.0], dtype=F64)
    router = torch.tensor([[2.0, 0.0], [0.0, 0.0], [0.0, -1.0], [-3.0, 0.0]], dtype=F64)      # logits 2, 0, 1, -3
    s = [1 / (1 + math.exp(-z)) for z in (2.0, 0.0, 1.0, -3.0)]
    # without a correction: experts 0 and 2; the correction lifts expert 3 above expert 2 but its weight stays its own score
    picks = N.sigmoid_router(h, router, torch.zeros(4, dtype=F64), 2, 2.5)
    assert [e for e, _ in picks] == [0, 2]
    assert abs(float(picks[0][1]) - s[0] / (s[0] + s[2]) * 2.5) < 1e-12 and abs(sum(float(w) for _, w in picks) - 2.5) < 1e-12
    picks = N.sigmoid_router(h, router, torch.tensor([0.0, 0.0, 0.0, 0.9], dtype=F64), 2, 1.0)
    assert [e for e, _ in picks] == [3, 0] or [e for e, _ in picks] == [0, 3]
    w3 = dict(picks)[3]
    assert abs(float(w3) - s[3] / (s[0] + s[3])) < 1e-12
    # the expert: gate bounded above only, value on both sides, and the value enters as u + 1
    gate = torch.tensor([[5.0, 0.0], [-5.0, 0.0], [0.5, 0.0]], dtype=F64)
    up = torch.tensor([[9.0, 0.0], [-9.0, 0.0], [0.25, 0.0]], dtype=F64)
    down = torch.eye(3, dtype=F64)
    y = N.clamped_expert(h, gate, up, down, 2.0)
    sg = lambda g: g / (1 + math.exp(-1.702 * g))
    assert torch.allclose(y, torch.tensor([sg(2.0) * 3.0, sg(-5.0) * -1.0, sg(0.5) * 1.25], dtype=F64), atol=1e-12)


def test_value_blending_uses_the_first_layers_values():
    """Scaling the first blending layer's value projection changes what the later layer caches only through lambda."""
    raw = small_cfg()
    cfg = DecoderLMConfig.from_dict(raw)
    t = dict(iter_synth_decoder_tensors(cfg, seed=3))
    base = N.NamalixOracle(raw, t)
    toks = [3, 1, 4, 1, 5]
    st = base.new_state()
    base.forward(toks, st)
    t0 = dict(t)
    t0["l3.mix.vmix"] = torch.zeros(())
    st0 = N.NamalixOracle(raw, t0).new_state()
    N.NamalixOracle(raw, t0).forward(toks, st0)
    lam = float(t["l3.mix.vmix"].double())
    v1 = torch.stack(st["layers"][1]["values"])
    assert torch.allclose(torch.stack(st["layers"][3]["values"]), (1 - lam) * torch.stack(st0["layers"][3]["values"]) + lam * v1, atol=1e-9)
