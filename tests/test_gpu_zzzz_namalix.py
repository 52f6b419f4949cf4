"""The Namalix decoder LM on the GPU against its float64 oracle (``oracle/namalix.py``): every mechanism alone, whole prompts
with every layer's output, prompts in portions down to one and two tokens, token-by-token decoding, unequal batches, slots
given back and used again, sharp attention with the strongest key at tile and split edges and far back, far memories of the
recurrent mixers, the first tokens of a sequence, odd and aligned sizes, and greedy generation through the scheduler and the
command line."""
import copy
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from moshi_b200.config import DecoderLMConfig
from moshi_b200.synth import iter_synth_decoder_tensors
from oracle.decoder_lm import logit_error
from oracle.namalix import F64, NamalixOracle

from .test_gpu_zz_decoder_lm import gen_for, tokens, write_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {torch.float32: 3e-5, torch.bfloat16: 8e-2}


def attention(heads, kv, dim, vdim, scale, rot_dims=0, base=300.0, scaling=None, softcap=0.0, v_mix=False, mlp=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv, "scale": scale, "softcap": softcap, "v_mix": v_mix, "vdim": vdim}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": m, "mlp": mlp}


def retention(heads, dim, vdim, decay, rot_dims=0, base=1000.0, mlp=None):
    m = {"decay": decay, "dim": dim, "heads": heads, "vdim": vdim}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "retention", "mixer": m, "mlp": mlp}


def delta(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv, "vdim": vdim}, "mlp": mlp}


def moe(experts, top, ff, limit=1.5, scale=1.7):
    return {"expert": {"ff": ff, "limit": limit}, "kind": "moe", "router": {"experts": experts, "scale": scale, "top": top}}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def make_cfg(layers, vocab, width, emb=4.0, eps=1e-5):
    return DecoderLMConfig.from_dict({"architecture": "Namalix", "embedding": {"scale": emb}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width})


RAMP = {"factor": 4.0, "original": 200, "fast": 4.0, "slow": 0.5}      # with base 300 and 10 dims: two kept, two blended, one divided
# odd sizes: nothing is a multiple of 8; three query heads per key head and one; value size unlike key size; 1, 2 and all experts;
# a layer without feed-forward; attention layers with and without value blending, rotation over a part of the head, the whole head, none
ODD = make_cfg([attention(6, 2, 10, 12, 0.3, rot_dims=10, scaling=RAMP, softcap=5.0, v_mix=True, mlp=moe(5, 2, 24)),
                delta(4, 2, 9, 11, 3, mlp=dense(30)),
                retention(3, 10, 7, [0.9, 0.97, 0.995], rot_dims=6),
                attention(6, 2, 14, 12, 0.2, rot_dims=14, v_mix=True, mlp=moe(3, 3, 17, limit=0.7, scale=1.0)),
                attention(4, 4, 8, 5, 0.35, softcap=2.0, mlp=dense(21)),
                delta(2, 2, 17, 6, 1, mlp=moe(4, 1, 30)),
                retention(2, 5, 9, [0.8, 0.999], mlp=dense(13))], vocab=97, width=52)
# aligned sizes: in bfloat16 every linear takes the tcgen05 GEMM, the attention and the experts their tensor-core kernels; a layer
# order that starts with retention; one key head for all query heads; a delta rule with as many query/key heads as value heads
ALIGNED = make_cfg([retention(2, 32, 64, [0.96, 0.999], rot_dims=16, mlp=moe(8, 2, 48)),
                    attention(4, 1, 32, 16, 0.18, rot_dims=32, scaling={"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}, softcap=20.0, v_mix=True, mlp=dense(128)),
                    delta(4, 2, 16, 32, 4, mlp=moe(6, 3, 32, limit=3.0, scale=2.0)),
                    attention(8, 1, 16, 16, 0.25, rot_dims=8, v_mix=True, mlp=moe(8, 2, 48)),
                    delta(2, 2, 64, 16, 2, mlp=None)], vocab=200, width=96)


def build(cfg, dtype, seed=3, edit=None):
    from moshi_b200.models import DecoderLM
    tensors = dict(iter_synth_decoder_tensors(cfg, seed=seed))
    if dtype == torch.bfloat16:
        # a bf16 rounding can turn a router's close call and swap an expert for that token; with random weights that happens
        # every few dozen tokens.  Small expert outputs keep such a swap inside the bf16 tolerance (float32 runs as drawn).
        for k in tensors:
            if ".mlp.e" in k and k.endswith(".down"):
                tensors[k] = tensors[k] * 0.25
    if edit:
        edit(tensors)
    return DecoderLM(cfg, tensors, device="cuda:0", dtype=dtype), NamalixOracle(cfg.to_dict(), tensors)


def assert_close(got, want, dtype, what="", tol=None):
    """float32: every row within the tolerance.  bfloat16: a rounding can turn a router's close call, which changes that token
    as a whole, so up to a tenth of the rows may be off while the median stays well inside."""
    e = logit_error(got.cpu(), want)
    tol = tol or TOL[dtype]
    if dtype == torch.float32:
        assert float(e.max()) < tol, f"{what}: relative logit error {float(e.max()):.3g}"
    else:
        assert int((e > tol).sum()) <= max(1, e.numel() // 10) and float(e.median()) < tol, f"{what}: relative logit errors {e.tolist()}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
def test_whole_prompt_and_every_layer(cfg, dtype):
    model, orc = build(cfg, dtype)
    toks = tokens(90, cfg.vocab, 1)
    want, layers = orc.forward(toks, return_layers=True)
    with gen_for(model, trace_layers=True) as gen:
        got = gen.step([(1, toks)], list(range(len(toks))))
        lo = gen.layer_outputs().cpu()
        assert gen.error_flags() == 0
    scale = float(layers.abs().max())
    for i in range(len(cfg.layers)):
        err = (lo[i].to(F64) - layers[i]).abs().amax(-1) / scale              # per token
        if dtype == torch.float32:
            assert float(err.max()) < 2e-5, f"layer {i}: {float(err.max()):.3g}"
        else:
            assert int((err > 8e-2).sum()) <= err.numel() // 4 and float(err.median()) < 4e-2, f"layer {i}: {err.tolist()}"
    assert_close(got, want, dtype)


def one_layer(kind, **kw):
    mlp = kw.pop("mlp", None)
    if kind == "attention":
        layer = attention(kw.get("heads", 6), kw.get("kv", 3), kw.get("dim", 10), kw.get("vdim", 14), kw.get("scale", 0.3), rot_dims=kw.get("rot", 6),
                          scaling=kw.get("scaling"), softcap=kw.get("softcap", 4.0), mlp=mlp)
    elif kind == "retention":
        layer = retention(3, 12, 20, kw.get("decay", [0.9, 0.98, 0.999]), rot_dims=kw.get("rot", 8), mlp=mlp)
    else:
        layer = delta(kw.get("heads", 4), kw.get("kv", 2), 12, 10, kw.get("conv", 3), mlp=mlp)
    return make_cfg([layer], vocab=64, width=40)


MECHANISMS = {
    "attention": ("attention", {}),
    "attention_no_rotation": ("attention", {"rot": 0}),
    "attention_whole_head_rotated": ("attention", {"rot": 10}),
    "attention_ramp": ("attention", {"rot": 10, "scaling": RAMP}),
    "attention_one_kv_head": ("attention", {"kv": 1}),
    "attention_kv_per_head": ("attention", {"kv": 6}),
    "attention_no_cap": ("attention", {"softcap": 0.0}),
    "attention_tight_cap": ("attention", {"softcap": 0.4, "scale": 1.5}),
    "retention": ("retention", {}),
    "retention_no_rotation": ("retention", {"rot": 0}),
    "retention_whole_head_rotated": ("retention", {"rot": 12}),
    "delta": ("delta", {}),
    "delta_conv_1": ("delta", {"conv": 1}),
    "delta_conv_5": ("delta", {"conv": 5}),
    "delta_one_qk_head": ("delta", {"kv": 1}),
    "delta_qk_per_head": ("delta", {"kv": 4}),
    "dense": ("retention", {"mlp": dense(23)}),
    "moe_top1": ("delta", {"mlp": moe(7, 1, 12)}),
    "moe_all": ("attention", {"mlp": moe(3, 3, 20, limit=0.5, scale=0.8)}),
    "moe_top2_of_5": ("retention", {"mlp": moe(5, 2, 9, limit=5.0, scale=2.5)}),
}


@pytest.mark.parametrize("what", sorted(MECHANISMS))
def test_mechanisms_in_isolation(what):
    """One layer with one mixer (and one kind of feed-forward or none)."""
    kind, kw = MECHANISMS[what]
    cfg = one_layer(kind, **dict(kw))
    edit = None
    if what.startswith("moe"):      # corrections as large as the scores' spread: the choice is not the order of the scores
        edit = lambda t: t.update({"l0.mlp.correction": t["l0.mlp.correction"] * 2.0})
    model, orc = build(cfg, torch.float32, seed=11, edit=edit)
    toks = tokens(40, cfg.vocab, 2)
    want, layers = orc.forward(toks, return_layers=True)
    with gen_for(model, trace_layers=True) as gen:
        got = gen.step([(0, toks)], list(range(len(toks))))
        lo = gen.layer_outputs().cpu()
    assert float((lo[0].to(F64) - layers[0]).abs().max()) < 3e-5 * float(layers.abs().max())
    assert_close(got, want, torch.float32, what)


def test_value_blending_across_layers():
    """Three attention layers blend values (the first one gives, the others take) around one that does not; large lambdas."""
    layers = [attention(4, 2, 8, 6, 0.3, rot_dims=4, v_mix=True), attention(2, 1, 8, 6, 0.3), attention(6, 2, 6, 6, 0.3, v_mix=True, mlp=dense(16)),
              attention(2, 2, 10, 6, 0.3, rot_dims=10, v_mix=True)]
    cfg = make_cfg(layers, vocab=50, width=36)
    edit = lambda t: t.update({"l2.mix.vmix": torch.tensor(0.9), "l3.mix.vmix": torch.tensor(-0.6), "l0.mix.vmix": torch.tensor(55.0)})      # the giver's own is unused
    model, orc = build(cfg, torch.float32, seed=14, edit=edit)
    toks = tokens(50, cfg.vocab, 3)
    want = orc.forward(toks)
    flat = copy.deepcopy(cfg.to_dict())
    for L in flat["layers"]:
        L["mixer"]["v_mix"] = False
    assert float(logit_error(NamalixOracle(flat, orc.W).forward(toks), want).max()) > 100 * TOL[torch.float32], "the blend must matter"
    with gen_for(model) as gen:
        got = torch.cat([gen.step([(0, toks[:31])], list(range(31)))] + [gen.step([(0, [t])], [0]) for t in toks[31:]])
    assert_close(got, want, torch.float32)


def sharpen(t, layer=0, gain=6.0, bias=-7.0, self_key=False):
    """Large query weights and a low bias: almost every key's weight is next to zero and a few stand out near one, so a key that
    is wrongly seen or missed changes the result as a whole.  self_key: every key head copies the projection of the first query
    head that reads it, so that a token's own key scores |q|^2 for that head and always stands out."""
    p = f"l{layer}.mix."
    t[p + "q"] = t[p + "q"] * gain
    t[p + "pb"] = torch.full_like(t[p + "pb"], bias)
    if self_key:
        H, G = t[p + "pb"].shape[0], t[p + "k"].shape[0] * t[p + "pb"].shape[0] // t[p + "q"].shape[0]
        dim = t[p + "q"].shape[0] // H
        q = t[p + "q"].view(H, dim, -1)
        t[p + "k"] = q[::H // G].reshape(G * dim, -1).clone() / gain


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim", [(4, 2, 16, 16), (6, 3, 10, 14), (16, 4, 32, 128), (2, 1, 48, 32), (8, 8, 16, 80), (20, 4, 16, 16)])
def test_sharp_attention_at_tile_and_split_edges(heads, kv, dim, vdim, dtype, monkeypatch):
    """Sharp attention, so that a key wrongly seen or missed shows.  Fragment-sized heads with a bf16 cache take the tensor-core
    kernel (tiles of 16 tokens x 32 keys; 1, 2 or 4 accumulator items per warp; more than 16 heads mix from shared memory), the
    others the CUDA-core kernel (tiles of 4 tokens).  One prompt with keys split 1, 3 and 5 ways, portions whose edges fall
    inside tiles, single tokens (tiles of one token), and the tensor-core kernel on one-token tiles; all against the oracle, and
    bf16 also against the CUDA-core kernel on the same model.  The test first shows that the oracle's result moves by far more
    than the tolerance when the newest key is dropped."""
    cfg = make_cfg([attention(heads, kv, dim, vdim, dim ** -0.5, rot_dims=(dim // 4) * 2, softcap=30.0)], vocab=120, width=64)
    model, orc = build(cfg, dtype, seed=21, edit=lambda t: sharpen(t, self_key=True))
    toks = tokens(150, cfg.vocab, 70)
    want = orc.forward(toks)

    import oracle.namalix as NX
    full = NX.sigmoid_attention
    monkeypatch.setattr(NX, "sigmoid_attention", lambda q, keys, values, *rest: full(q, keys[:-1] or keys, values[:-1] or values, *rest))
    moved = NamalixOracle(cfg.to_dict(), orc.W).forward(toks)
    monkeypatch.undo()
    tol = {torch.float32: 3e-5, torch.bfloat16: 3e-2}[dtype]      # one layer and no router: bfloat16 stays well inside this
    assert float(logit_error(moved, want).median()) > 2.5 * tol, "the newest key must matter"
    with gen_for(model) as gen:
        plain = None
        if dtype == torch.bfloat16:
            gen.set_option("attn_tc", 0)
            plain = gen.step([(0, toks)], list(range(len(toks))))
            gen.set_option("attn_tc", 1)
        for split in (0, 1, 3, 5):
            gen.set_option("attn_split", split)
            whole = gen.step([(1, toks)], list(range(len(toks))))
            gen.release(1)
            assert_close(whole, want, dtype, f"split {split}", tol)
            if plain is not None:
                assert_close(whole, plain.cpu().to(F64), dtype, f"split {split}, against the CUDA-core kernel", tol)
        gen.set_option("attn_split", 0)
        parts = [gen.step([(2, toks[:37])], list(range(37))), gen.step([(2, toks[37:39])], [0, 1]), gen.step([(2, toks[39:100])], list(range(61)))]
        parts += [gen.step([(2, [t])], [0]) for t in toks[100:125]]         # single tokens: the CUDA-core kernel on one-token tiles
        gen.set_option("attn_tc", 2)                                            # and the tensor-core kernel on one-token tiles
        parts += [gen.step([(2, [t])], [0]) for t in toks[125:]]
        assert_close(torch.cat(parts), want, dtype, "portions and single tokens", tol)
        assert gen.error_flags() == 0


def test_a_far_key_among_hundreds():
    """Sharp attention over 760 tokens whose token 30 occurs nowhere else: the test first shows that the last 40 logits move when it
    is replaced, then reads them from a prompt portion and from single-token decoding (keys split over many CTAs)."""
    cfg = make_cfg([attention(4, 2, 16, 16, 0.25, softcap=50.0)], vocab=90, width=32)
    model, orc = build(cfg, torch.float32, seed=31, edit=lambda t: sharpen(t, gain=3.0, bias=-9.0))
    toks = tokens(760, cfg.vocab - 1, 5)
    marker = cfg.vocab - 1
    toks[30] = marker                                   # the only occurrence
    want = orc.forward(toks)[-40:]
    gone = list(toks)
    gone[30] = toks[31]
    assert float(logit_error(orc.forward(gone)[-40:], want).max()) > 30 * TOL[torch.float32], "token 30 must still matter at the end"
    with gen_for(model, capacity=1024, max_step_tokens=512) as gen:
        gen.step([(0, toks[:500])])
        gen.step([(0, toks[500:720])])
        got = gen.step([(0, toks[720:740])], list(range(20)))
        got = torch.cat([got] + [gen.step([(0, [t])], [0]) for t in toks[740:]])
    assert_close(got, want, torch.float32)


def keep_long(t):
    """Delta rule: decays next to one and small writes, so that what was stored hundreds of tokens ago still weighs."""
    for k in list(t):
        if k.endswith("A_log"):
            t[k] = torch.full_like(t[k], -7.0)
        if k.endswith("mix.b"):
            t[k] = t[k] * 0.1 - 0.0


@pytest.mark.parametrize("kind", ["retention", "delta"])
def test_far_tokens_reach_through_the_recurrent_state(kind):
    cfg = one_layer("retention", decay=[0.999, 0.9995, 0.99]) if kind == "retention" else one_layer("delta")
    model, orc = build(cfg, torch.float32, seed=6, edit=keep_long if kind == "delta" else None)
    toks = tokens(400, cfg.vocab, 4)
    want = orc.forward(toks)[-40:]
    swapped = [(toks[0] + 1) % cfg.vocab] + toks[1:]
    assert float(logit_error(orc.forward(swapped)[-40:], want).max()) > 30 * TOL[torch.float32], "token 0 must still matter at the end"
    with gen_for(model, capacity=512, max_step_tokens=512) as gen:
        gen.step([(0, toks[:150])])
        gen.step([(0, toks[150:360])])
        got = gen.step([(0, toks[360:380])], list(range(20)))
        got = torch.cat([got] + [gen.step([(0, [t])], [0]) for t in toks[380:]])
    assert_close(got, want, torch.float32)


@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_portions_and_single_tokens_equal_the_whole_prompt(dtype, cfg):
    model, orc = build(cfg, dtype)
    toks = tokens(130, cfg.vocab, 7)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        whole = gen.step([(0, toks)], list(range(len(toks))))
        for cuts in ([2, 3, 1, 7, 2, 40, 1, 1, 2, 9, 33, 2, 27], [64, 66], [1] * 12 + [118], [5, 4, 3, 2] * 9 + [4], [2] * 65):
            assert sum(cuts) == len(toks)
            gen.release(2)
            parts, at = [], 0
            for n in cuts:
                parts.append(gen.step([(2, toks[at:at + n])], list(range(n))))
                at += n
            got = torch.cat(parts)
            assert_close(got, want, dtype, f"cuts {cuts[:4]}")
            assert_close(got, whole.cpu().to(F64), dtype, "a cut changes at most the order of sums")


def test_the_first_tokens_of_a_sequence():
    """Positions 0 .. 5: convolutions with nothing in front, empty matrix memories, attention over a single key."""
    model, orc = build(ODD, torch.float32, seed=9)
    for n in (1, 2, 3, 6):
        toks = tokens(n, ODD.vocab, 20 + n)
        with gen_for(model) as gen:
            assert_close(gen.step([(0, toks)], list(range(n))), orc.forward(toks), torch.float32, f"{n} tokens at once")
            gen.release(0)
            one = torch.cat([gen.step([(0, [t])], [0]) for t in toks])
            assert_close(one, orc.forward(toks), torch.float32, f"{n} tokens one by one")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_token_by_token(dtype):
    cfg = ALIGNED
    model, orc = build(cfg, dtype, seed=4)
    toks = tokens(200, cfg.vocab, 8)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        gen.step([(1, toks[:20])])
        got = torch.cat([gen.step([(1, [t])], [0]) for t in toks[20:]])
        assert gen.error_flags() == 0
    assert_close(got, want[20:], dtype)


@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_batch_equals_each_request_alone(dtype, cfg):
    model, orc = build(cfg, dtype)
    reqs = [tokens(61, cfg.vocab, 30), tokens(9, cfg.vocab, 31), tokens(34, cfg.vocab, 32)]
    want = [orc.forward(r) for r in reqs]
    with gen_for(model) as gen:
        # different histories: 40 tokens, none, 33 tokens; then one step with 21 + 9 + 1 tokens
        gen.step([(2, reqs[0][:40]), (0, reqs[2][:33])])
        got = gen.step([(2, reqs[0][40:]), (1, reqs[1]), (0, reqs[2][33:])], list(range(31)))
    assert_close(got[:21], want[0][40:], dtype, "long history, many tokens")
    assert_close(got[21:30], want[1], dtype, "fresh request")
    assert_close(got[30:], want[2][33:], dtype, "single token")


def test_slots_are_given_back_and_used_again():
    """A shorter request in a slot that held a longer one: neither its cached keys and values, nor the carried convolution
    inputs, nor the matrix memories of the earlier request may show."""
    cfg = ODD
    model, orc = build(cfg, torch.float32)
    long_req, short_req = tokens(120, cfg.vocab, 50), tokens(11, cfg.vocab, 51)
    with gen_for(model, slots=1) as gen:
        gen.step([(0, long_req)])
        gen.release(0)
        assert gen.slot_length(0) == 0
        got = gen.step([(0, short_req[:2])], [0, 1])
        got = torch.cat([got, gen.step([(0, short_req[2:])], list(range(9)))])
        assert_close(got, orc.forward(short_req), torch.float32)
        gen.release(0)
        gen.step([(0, short_req)])
        with pytest.raises(Exception):
            gen.step([(0, tokens(300, cfg.vocab, 52))])             # would overflow the slot: refused whole
        assert gen.slot_length(0) == len(short_req)


@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_portions_run_as_parallel_segments(dtype, cfg):
    """A portion of at least two segments is cut for the retention (the delta rule takes portions whole): the segments run side
    by side from empty memories, are chained, and the later ones get the carried state's share added.  Segments of 16 tokens here
    (256 by default), so that portions of 33 .. 150 tokens take that path: one prompt, portions with a ragged last segment, a
    batch of long and short requests on different histories, then single tokens on the state the chain left in the slot."""
    from moshi_b200 import _lib
    model, orc = build(cfg, dtype)
    _lib.check(model._lib.b200_dlm_set_option(model._h, b"scan_segment", 16))
    reqs = [tokens(150, cfg.vocab, 80), tokens(9, cfg.vocab, 81), tokens(120, cfg.vocab, 82)]
    want = [orc.forward(r) for r in reqs]
    with gen_for(model) as gen:
        assert_close(gen.step([(0, reqs[0])], list(range(150))), want[0], dtype, "one portion of 150 tokens")
        gen.release(0)
        parts = [gen.step([(0, reqs[0][:70])], list(range(70))), gen.step([(0, reqs[0][70:73])], [0, 1, 2]), gen.step([(0, reqs[0][73:110])], list(range(37)))]
        parts += [gen.step([(0, [t])], [0]) for t in reqs[0][110:]]
        assert_close(torch.cat(parts), want[0], dtype, "70 + 3 + 37 tokens, then one by one")
        gen.release(0)
        gen.step([(2, reqs[0][:40]), (0, reqs[2][:33])])
        got = gen.step([(2, reqs[0][40:]), (1, reqs[1]), (0, reqs[2][33:])], list(range(110 + 9 + 87)))
        assert_close(got[:110], want[0][40:], dtype, "110 tokens on a history of 40")
        assert_close(got[110:119], want[1], dtype, "a short fresh request beside them")
        assert_close(got[119:], want[2][33:], dtype, "87 tokens on a history of 33")
        assert gen.error_flags() == 0


def test_segments_of_the_default_length():
    cfg = ALIGNED
    model, orc = build(cfg, torch.float32, seed=13)
    toks = tokens(700, cfg.vocab, 90)
    want = orc.forward(toks)
    with gen_for(model, capacity=1024, max_step_tokens=1024) as gen:
        got = torch.cat([gen.step([(0, toks[:600])], list(range(600))), gen.step([(0, toks[600:])], list(range(100)))])
    assert_close(got, want, torch.float32)


def test_greedy_generation_through_the_scheduler():
    from moshi_b200.serving import TokenScheduler
    cfg = ODD
    model, orc = build(cfg, torch.float32)
    prompts = {"a": tokens(23, cfg.vocab, 40), "b": tokens(3, cfg.vocab, 41), "c": tokens(40, cfg.vocab, 42)}
    with gen_for(model, slots=2, capacity=80, max_step_tokens=32) as gen:      # 3 requests over 2 slots, prompts cut at 32 tokens
        sched = TokenScheduler(gen)
        for k, p in prompts.items():
            sched.submit(k, p, 12)
        out = sched.run()
    for k, p in prompts.items():
        want, gaps = orc.greedy(p, 12)
        for i, (g, w, gap) in enumerate(zip(out[k], want, gaps)):
            if g != w:
                assert gap < 1e-3, f"request {k}: token {i} is {g}, the oracle says {w} with a gap of {gap}"
                break


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_command_line_replays_steps_and_generates(tmp_path, dtype):
    cfg = ODD
    tensors = dict(iter_synth_decoder_tensors(cfg, seed=8))
    if dtype == "bfloat16":
        for k in tensors:
            if ".mlp.e" in k and k.endswith(".down"):
                tensors[k] = tensors[k] * 0.25
    write_model(tmp_path / "m", cfg, tensors)
    orc = NamalixOracle(json.loads((tmp_path / "m" / "config.json").read_text()), tensors)
    a, b = tokens(30, cfg.vocab, 50), tokens(6, cfg.vocab, 51)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:21], "want": [0, 20]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[21:23], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[23:], "want": [6]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [5]}], "end": ["b"]}]
    (tmp_path / "out").mkdir()
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype, "--out", str(tmp_path / "out"),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    import numpy as np
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    read = lambda i, n: torch.from_numpy(np.fromfile(tmp_path / "out" / f"{i}.f32", dtype="<f4").reshape(n, cfg.vocab))
    fa = orc.forward(a)
    assert_close(read(0, 2), fa[[0, 20]], td)
    assert_close(read(2, 1), fa[[29]], td)
    assert_close(read(3, 1), orc.forward(b)[[5]], td)
    if dtype == "float32":
        r = subprocess.run([sys.executable, "-m", "moshi_b200.cli", "generate", "--model", str(tmp_path / "m"), "--dtype", dtype,
                            "--prompt", ",".join(map(str, b)), "--max-new", "5"], capture_output=True, text=True, timeout=600, cwd=ROOT)
        assert r.returncode == 0, r.stderr[-2000:]
        got = json.loads(r.stdout.strip().splitlines()[-1])["tokens"]
        want, gaps = orc.greedy(b, 5)
        for g, w, gap in zip(got, want, gaps):
            if g != w:
                assert gap < 1e-3
                break


def random_cfg(seed):
    """A configuration drawn from the design's whole space: layer order, head counts and sizes, rotation, cap, blending, taps,
    feed-forward kinds, expert counts; all blending layers share their key/value heads and value size."""
    import random
    r = random.Random(seed)
    width, vocab = r.choice([64, 96, 128, 160, 256, 320]), r.randrange(150, 700)
    bg, bv = r.choice([1, 2, 4]), r.choice([16, 32, 64])
    layers = []
    for i in range(r.randrange(3, 9)):
        kind = r.choice(["attention", "retention", "delta"]) if i > 2 else ["attention", "retention", "delta"][(i + seed) % 3]
        mlp = r.choice([None, dense(r.choice([48, 100, 256])), moe(r.choice([2, 4, 8, 12]), 1, r.choice([32, 64])), None])
        if mlp and mlp["kind"] == "moe":
            mlp["router"]["top"] = r.randrange(1, min(4, mlp["router"]["experts"]) + 1)
            mlp["expert"]["limit"], mlp["router"]["scale"] = r.choice([0.5, 1.0, 7.0]), r.choice([1.0, 2.5])
        if kind == "attention":
            blend = r.random() < 0.6
            g = bg if blend else r.choice([1, 2, 4])
            dim = r.choice([16, 32, 64, 128])
            rot = r.choice([0, dim // 2, dim])
            sc = r.choice([None, {"factor": r.choice([2.0, 4.0, 16.0]), "original": r.choice([64, 512, 4096]), "fast": r.choice([8.0, 32.0]), "slow": r.choice([0.5, 1.0, 2.0])}])
            layers.append(attention(g * r.choice([1, 2, 4]), g, dim, bv if blend else r.choice([16, 32, 48]), r.choice([dim ** -0.5, 0.09, 0.2]), rot_dims=rot,
                                    base=r.choice([100.0, 10000.0, 500000.0]), scaling=sc if rot else None, softcap=r.choice([0.0, 15.0, 30.0, 50.0]), v_mix=blend, mlp=mlp))
        elif kind == "retention":
            hh, dim = r.choice([1, 2, 4, 8]), r.choice([16, 32, 64])
            layers.append(retention(hh, dim, r.choice([16, 32, 64]), [1.0 - 2.0 ** -r.uniform(3, 10) for _ in range(hh)], rot_dims=r.choice([0, dim // 2, dim]),
                                    base=r.choice([1000.0, 1000000.0]), mlp=mlp))
        else:
            g = r.choice([1, 2, 4])
            layers.append(delta(g * r.choice([1, 2]), g, r.choice([16, 32, 64, 128]), r.choice([16, 32, 64]), r.choice([2, 3, 4]), mlp=mlp))
    return make_cfg(layers, vocab=vocab, width=width, emb=width ** 0.5, eps=r.choice([1e-6, 1e-5]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(seed, dtype):
    """Whole prompt, prompt + single tokens, and ragged portions of a drawn configuration against the oracle."""
    cfg = random_cfg(seed)
    model, orc = build(cfg, dtype, seed=100 + seed)
    toks = tokens(170, cfg.vocab, 200 + seed)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        assert_close(gen.step([(0, toks)], list(range(len(toks)))), want, dtype, "whole")
        got = torch.cat([gen.step([(1, toks[:138])], list(range(138)))] + [gen.step([(1, [t])], [0]) for t in toks[138:]])
        assert_close(got, want, dtype, "prompt, then single tokens")
        parts, at = [], 0
        for n in [2, 31, 3, 64, 1, 17, 2, 50]:
            parts.append(gen.step([(2, toks[at:at + n])], list(range(n))))
            at += n
        assert_close(torch.cat(parts), want, dtype, "portions")
        assert gen.error_flags() == 0


@pytest.mark.parametrize("heads,kv,dim,vdim,conv", [(3, 3, 9, 10, 2), (4, 2, 17, 33, 3), (2, 1, 40, 64, 4), (2, 2, 128, 48, 4), (1, 1, 200, 70, 2)])
def test_delta_rule_in_chunks_equals_token_by_token(heads, kv, dim, vdim, conv):
    """Portions of at least 16 tokens take the delta rule in chunks of 32 tokens (three products against the state and one forward
    substitution per chunk); shorter ones and single tokens the token-by-token kernel.  Both against the oracle, for every
    register layout of the chunk kernel (key sizes up to 16, 32, 64, 128, 256), with chunks that end ragged, portions that start
    on a carried state, a mixed batch, and decays near one so that the state carries across many chunks."""
    cfg = make_cfg([delta(heads, kv, dim, vdim, conv, mlp=dense(24))], vocab=80, width=48)
    model, orc = build(cfg, torch.float32, seed=41, edit=keep_long)
    reqs = [tokens(150, cfg.vocab, 91), tokens(20, cfg.vocab, 92), tokens(77, cfg.vocab, 93)]
    want = [orc.forward(r) for r in reqs]
    with gen_for(model) as gen:
        for chunked in (1, 0):
            gen.set_option("delta_chunk", chunked)
            for s in range(3):
                gen.release(s)
            assert_close(gen.step([(0, reqs[0])], list(range(150))), want[0], torch.float32, f"one portion (chunks {chunked})")
            gen.release(0)
            parts = [gen.step([(0, reqs[0][:70])], list(range(70))), gen.step([(0, reqs[0][70:73])], [0, 1, 2]), gen.step([(0, reqs[0][73:110])], list(range(37)))]
            parts += [gen.step([(0, [t])], [0]) for t in reqs[0][110:]]
            assert_close(torch.cat(parts), want[0], torch.float32, f"70 + 3 + 37 tokens, then one by one (chunks {chunked})")
            gen.release(0)
            gen.step([(2, reqs[0][:40]), (0, reqs[2][:33])])
            got = gen.step([(2, reqs[0][40:]), (1, reqs[1]), (0, reqs[2][33:34])], list(range(110 + 20 + 1)))
            assert_close(got[:110], want[0][40:], torch.float32, f"110 tokens on a history of 40 (chunks {chunked})")
            assert_close(got[110:130], want[1], torch.float32, f"a fresh request of 20 beside them (chunks {chunked})")
            assert_close(got[130:], want[2][33:34], torch.float32, f"a single token beside them (chunks {chunked})")
        assert gen.error_flags() == 0
