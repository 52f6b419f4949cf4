"""The Dibulix decoder LM on the GPU against its float64 oracle (``oracle/dibulix.py``): every mechanism alone, whole prompts
with every layer's output, prompts in portions down to two tokens, token-by-token decoding, unequal batches, slots given back
and used again, sharp attention at the windows' edges in prompts and in decoding, far memories of the recurrent mixers, the first
tokens of a sequence, odd and aligned sizes, stream counts from none to four, and greedy generation through the scheduler and
the command line."""
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
from oracle.dibulix import F64, Oracle

from .test_gpu_zz_decoder_lm import gen_for, tokens, write_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {torch.float32: 3e-5, torch.bfloat16: 8e-2}
RAMP = {"factor": 4.0, "original": 200, "fast": 4.0, "slow": 0.5}


def latent(heads, dim, rot_dim, vdim, rank, scale, window, base=300.0, scaling=None, mlp=None):
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling:
            m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def pair(heads, kv, dim, vdim, scale, window, width, rot_dims=0, base=1000.0, ls=1.0, rs=1.0, mlp=None):
    left = {"dim": dim, "heads": heads, "kv_heads": kv, "scale": scale, "vdim": vdim}
    if window:
        left["mask"] = {"size": window}
    if rot_dims:
        left["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": ls, "right": {"width": width}, "right_scale": rs}, "mlp": mlp}


def cdelta(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "channel_delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv, "vdim": vdim}, "mlp": mlp}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def make_cfg(layers, vocab, width, streams=2, logit_scale=0.5, eps=1e-5, ranks=(5, 7)):
    d = {"architecture": "Dibulix", "layers": layers, "logit_scale": logit_scale, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if streams is not None:
        d["streams"] = streams
    cfg = DecoderLMConfig.from_dict(d)
    for L in cfg.layers:             # the two bottlenecks' sizes are tensor shapes, not configuration keys
        if L.type == "channel_delta":
            L.a.decay_rank, L.a.gate_rank = ranks
    return cfg


# odd sizes: nothing is a multiple of 8; three query heads per key head and one; value size unlike key size; rotation over a part
# of the head and the whole head; windows shorter than the prompts; three streams; layers with and without feed-forward
ODD = make_cfg([cdelta(4, 2, 9, 11, 3, mlp=dense(30)),
                latent(3, 10, 6, 7, 13, 0.3, 17, scaling=RAMP, mlp=dense(21)),
                pair(6, 2, 10, 12, 0.3, 23, 37, rot_dims=6, ls=1.3, rs=0.8),
                cdelta(2, 2, 17, 6, 1),
                latent(5, 6, 10, 9, 21, 0.25, 40, mlp=None),
                pair(4, 4, 14, 5, 0.2, 9, 19, rot_dims=14, ls=0.7, rs=1.2, mlp=dense(13))], vocab=97, width=52, streams=3)
# aligned sizes: in bfloat16 every linear takes the tcgen05 GEMM and the window attention its tensor-core kernel; a layer order that
# starts with attention; one key head for all query heads; a delta rule whose query/key heads serve two value heads each
ALIGNED = make_cfg([pair(4, 1, 32, 16, 0.18, 48, 128, rot_dims=16, ls=1.25, rs=0.9, mlp=dense(128)),
                    latent(4, 32, 16, 32, 48, 0.15, 64, scaling={"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}, mlp=dense(64)),
                    cdelta(4, 2, 16, 32, 4),
                    pair(8, 2, 16, 16, 0.25, 33, 64, rot_dims=8),
                    cdelta(2, 2, 64, 16, 2, mlp=dense(96))], vocab=200, width=96, streams=2, ranks=(16, 16))


def build(cfg, dtype, seed=3, edit=None):
    from moshi_b200.models import DecoderLM
    tensors = dict(iter_synth_decoder_tensors(cfg, seed=seed))
    if edit:
        edit(tensors)
    return DecoderLM(cfg, tensors, device="cuda:0", dtype=dtype), Oracle(cfg.to_dict(), tensors)


def assert_close(got, want, dtype, what="", tol=None):
    e = logit_error(got.cpu(), want)
    tol = tol or TOL[dtype]
    assert float(e.max()) < tol, f"{what}: relative logit error {float(e.max()):.3g} at row {int(e.argmax())}"


def in_portions(gen, slot, toks, cuts):
    """The tokens in portions of the given sizes (the rest in one), every row wanted."""
    out, at = [], 0
    for n in list(cuts) + [len(toks)]:
        part = toks[at:at + n]
        if not part:
            break
        out.append(gen.step([(slot, part)], list(range(len(part)))))
        at += len(part)
    return torch.cat(out)


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
        err = float(((lo[i].to(F64) - layers[i]).abs().amax(-1) / scale).max())
        assert err < (2e-5 if dtype == torch.float32 else 8e-2), f"layer {i}: {err:.3g}"
    assert_close(got, want, dtype)


ALONE = {
    "latent": [latent(3, 10, 6, 7, 13, 0.3, 11, scaling=RAMP)],
    "latent_plain_rotation": [latent(2, 8, 12, 9, 20, 0.4, 25)],
    "latent_no_rotation_no_window": [latent(3, 10, 0, 7, 13, 0.3, 0)],
    "latent_one_head": [latent(1, 16, 4, 16, 8, 0.2, 5, mlp=dense(24))],
    "window_attention_alone": [pair(6, 2, 10, 12, 0.3, 13, 20, rot_dims=6, ls=1.4, rs=0.0)],
    "window_attention_all_rotated_one_kv_head": [pair(4, 1, 12, 5, 0.3, 7, 8, rot_dims=12, ls=1.0, rs=0.0)],
    "window_attention_unrotated": [pair(3, 3, 9, 9, 0.35, 30, 8, rot_dims=0, ls=1.0, rs=0.0)],
    "window_attention_without_a_mask": [pair(4, 2, 8, 6, 0.3, 0, 8, rot_dims=8, ls=1.0, rs=0.0)],
    "mingru_alone": [pair(2, 1, 4, 4, 0.3, 3, 45, ls=0.0, rs=0.9)],
    "pair": [pair(4, 2, 8, 8, 0.3, 12, 33, rot_dims=4, ls=0.85, rs=1.3, mlp=dense(40))],
    "delta_shared_heads": [cdelta(6, 2, 9, 11, 3)],
    "delta_one_tap": [cdelta(2, 2, 17, 6, 1)],
    "delta_five_taps_one_head": [cdelta(1, 1, 33, 20, 5, mlp=dense(16))],
    "delta_wide_key": [cdelta(2, 1, 130, 12, 2)],
}


@pytest.mark.parametrize("streams", [None, 1, 2, 4])
@pytest.mark.parametrize("what", sorted(ALONE))
def test_mechanisms_in_isolation(what, streams):
    if streams in (1, 4) and what not in ("latent", "pair", "delta_shared_heads"):
        pytest.skip("stream counts are covered on three mechanisms")
    cfg = make_cfg(copy.deepcopy(ALONE[what]), vocab=61, width=44, streams=streams, logit_scale=1.7)
    model, orc = build(cfg, torch.float32, seed=11)
    toks = tokens(50, cfg.vocab, 2)
    with gen_for(model) as gen:
        got = gen.step([(0, toks)], list(range(len(toks))))
    assert_close(got, orc.forward(toks), torch.float32, what)


def sharpen(names, by):
    def edit(t):
        for k in t:
            if k.endswith(names):
                t[k] = t[k] * by
    return edit


@pytest.mark.parametrize("window", [1, 2, 7, 32, 33, 40, 97, 128])
@pytest.mark.parametrize("kind", ["window", "latent"])
def test_sharp_attention_at_the_windows_edges(kind, window):
    """Large query and key weights make single keys dominate, so a window that is one token off shows; the oracle itself moves by
    far more than the tolerance when its window changes by one."""
    if kind == "window":
        layers, names = [pair(4, 2, 8, 8, 0.5, window, 8, rot_dims=4, ls=1.0, rs=0.0)], ("left.q", "left.k")
    else:
        layers, names = [latent(3, 8, 4, 8, 12, 0.5, window)], ("mix.q", "mix.uk", "mix.dkv")
    cfg = make_cfg(layers, vocab=53, width=40, streams=2)
    model, orc = build(cfg, torch.float32, seed=5, edit=sharpen(names, 3.0))
    n = max(100, 2 * window + 36)                      # the window passes over prompt tokens and over single tokens
    toks = tokens(n, cfg.vocab, 3)
    want = orc.forward(toks)
    for off in (-1, 1):
        if window + off < 1:
            continue
        d = cfg.to_dict()
        m = d["layers"][0]["mixer"]
        (m["left"] if kind == "window" else m)["mask"]["size"] = window + off
        other = Oracle(d, orc.t).forward(toks)
        assert float(logit_error(other, want).max()) > 50 * TOL[torch.float32]
    with gen_for(model, capacity=n + 8, max_step_tokens=max(256, n)) as gen:
        assert_close(gen.step([(0, toks)], list(range(n))), want, torch.float32, "whole")
        gen.release(0)
        got = in_portions(gen, 0, toks, [window + 1, 2, 3] + [1] * (window + 8 if window > 40 else 40) + [2] * 5)
        assert_close(got, want, torch.float32, "portions and single tokens")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["window", "latent"])
def test_a_far_key_without_a_mask(kind, dtype):
    """Without a mask every earlier key is seen: sharp scores over 600 tokens, so that single keys hundreds of positions back carry
    rows of the result, in a prompt whose keys are cut over CTAs, in portions, and in single tokens."""
    if kind == "window":
        layers, names = [pair(4, 2, 16, 16, 0.5, 0, 8, rot_dims=8, ls=1.0, rs=0.0)], ("left.q", "left.k")
    else:
        layers, names = [latent(2, 16, 16, 16, 16, 0.5, 0)], ("mix.q", "mix.uk", "mix.dkv")
    cfg = make_cfg(layers, vocab=53, width=48, streams=2)
    # bfloat16 rounds keys and queries: scores as sharp as float32 can take would turn that rounding into the result's error
    model, orc = build(cfg, dtype, seed=6, edit=sharpen(names, 3.0 if dtype == torch.float32 else 1.6))
    toks = tokens(600, cfg.vocab, 5)
    want = orc.forward(toks)
    short = orc.forward(toks[300:])                        # the same last tokens without the first 300: the far keys matter
    assert float(logit_error(short[-40:], want[-40:]).max()) > 50 * TOL[torch.float32]
    with gen_for(model, capacity=640, max_step_tokens=640) as gen:
        assert_close(gen.step([(0, toks)], list(range(600))), want, dtype, "whole")
        gen.release(0)
        got = in_portions(gen, 0, toks, [517, 2, 33] + [1] * 40)
        assert_close(got, want, dtype, "portions and single tokens")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_far_memories_of_the_recurrences(dtype):
    """Decays next to one and update gates next to zero: token 0 still moves the logits 300 tokens later."""
    cfg = make_cfg([cdelta(4, 2, 16, 16, 3), pair(2, 1, 8, 8, 0.3, 4, 48, ls=0.1, rs=1.5)], vocab=71, width=48, streams=2, ranks=(8, 8))

    def edit(t):
        for k in t:
            if k.endswith("A_log"):
                t[k] = torch.full_like(t[k], -7.0)
            if k.endswith("right.z.b"):
                t[k] = torch.full_like(t[k], -5.0)
    model, orc = build(cfg, dtype, seed=9, edit=edit)
    toks = tokens(300, cfg.vocab, 4)
    want = orc.forward(toks)
    moved = orc.forward([(toks[0] + 1) % cfg.vocab] + toks[1:])
    assert float(logit_error(moved[-1:], want[-1:]).max()) > 30 * TOL[torch.float32]
    with gen_for(model, capacity=320) as gen:
        got = in_portions(gen, 2, toks, [130, 2, 97, 3] + [1] * 30)
        assert_close(got, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
@pytest.mark.parametrize("cuts", [[2, 3, 1, 7, 2, 40], [1] * 12, [5, 4, 3, 2] * 6, [2] * 45, [64]], ids=["ragged", "ones", "cycle", "twos", "long"])
def test_portions_equal_the_whole_prompt(cfg, cuts, dtype):
    model, orc = build(cfg, dtype)
    toks = tokens(130, cfg.vocab, 6)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        assert_close(in_portions(gen, 1, toks, cuts), want, dtype)
        assert gen.error_flags() == 0


@pytest.mark.parametrize("n", [1, 2, 3, 6])
def test_first_tokens_at_once_and_one_by_one(n):
    model, orc = build(ODD, torch.float32)
    toks = tokens(n, ODD.vocab, 20 + n)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        assert_close(gen.step([(0, toks)], list(range(n))), want, torch.float32, "at once")
        assert_close(in_portions(gen, 1, toks, [1] * n), want, torch.float32, "one by one")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_token_by_token(dtype):
    cfg = ALIGNED if dtype == torch.bfloat16 else ODD
    model, orc = build(cfg, dtype)
    toks = tokens(190, cfg.vocab, 7)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        assert_close(in_portions(gen, 0, toks, [10] + [1] * 180), want, dtype)
        assert gen.error_flags() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [ODD, ALIGNED], ids=["odd", "aligned"])
def test_unequal_batch_equals_each_request_alone(cfg, dtype):
    model, orc = build(cfg, dtype)
    a, b, c = tokens(61, cfg.vocab, 8), tokens(9, cfg.vocab, 9), tokens(34, cfg.vocab, 10)
    wa, wb, wc = orc.forward(a), orc.forward(b), orc.forward(c)
    with gen_for(model) as gen:
        gen.step([(0, a[:40]), (2, c[:33])], [])
        got = gen.step([(0, a[40:]), (1, b), (2, c[33:])], list(range(21 + 9 + 1)))      # 21 + 9 + 1 tokens on histories of 40 / 0 / 33
        assert_close(got[:21], wa[40:], dtype, "a")
        assert_close(got[21:30], wb, dtype, "b")
        assert_close(got[30:], wc[33:], dtype, "c")
        got = gen.step([(1, [b[0]]), (0, [a[0]])], [0, 1])                                   # single tokens of two requests on their histories
        assert got.shape[0] == 2


def test_slots_are_given_back_and_used_again():
    model, orc = build(ODD, torch.float32)
    a, b = tokens(120, ODD.vocab, 12), tokens(11, ODD.vocab, 13)
    with gen_for(model, slots=1) as gen:
        gen.step([(0, a)], [])
        with pytest.raises(RuntimeError):
            gen.step([(0, tokens(200, ODD.vocab, 14))], [])                                 # would overflow the slot: refused whole
        gen.release(0)
        assert gen.slot_length(0) == 0
        assert_close(gen.step([(0, b)], list(range(11))), orc.forward(b), torch.float32)
        gen.release(0)
        assert_close(in_portions(gen, 0, a, [3, 50]), orc.forward(a), torch.float32, "again")


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
    cfg = ODD if dtype == "float32" else ALIGNED
    tensors = dict(iter_synth_decoder_tensors(cfg, seed=8))
    write_model(tmp_path / "m", cfg, tensors)
    orc = Oracle(cfg.to_dict(), tensors)
    a, b = tokens(30, cfg.vocab, 50), tokens(6, cfg.vocab, 51)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:21], "want": [0, 20]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[21:], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": b, "want": [5]}], "end": ["b"]}]
    (tmp_path / "out").mkdir()
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype, "--out", str(tmp_path / "out"),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    import numpy as np
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    got0 = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(2, cfg.vocab))
    got2 = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(1, cfg.vocab))
    assert_close(got0, orc.forward(a)[[0, 20]], td)
    assert_close(got2, orc.forward(b)[[5]], td)
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


def drawn_cfg(seed):
    """A configuration drawn from the design's space: layer order, head counts and sizes, windows, rotation, taps, streams."""
    g = torch.Generator().manual_seed(seed)

    def pick(*xs):
        return xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    layers = []
    for _ in range(pick(2, 3, 4)):
        kind, mlp = pick("latent", "pair", "delta"), pick(None, dense(pick(12, 32, 40)))
        if kind == "latent":
            rd = pick(0, 2, 4, 8)
            layers.append(latent(pick(1, 2, 4), pick(4, 8, 12), rd, pick(4, 8, 10), pick(6, 16, 24), pick(0.2, 0.35), pick(0, 3, 20, 64),
                                 base=pick(100.0, 10000.0), scaling=pick(None, RAMP) if rd else None, mlp=mlp))
        elif kind == "pair":
            kv, dim = pick(1, 2), pick(4, 8, 16)
            layers.append(pair(kv * pick(1, 2, 3), kv, dim, pick(4, 8, 16), pick(0.2, 0.4), pick(1, 5, 31, 70), pick(8, 24, 50),
                               rot_dims=pick(0, 2, dim), ls=pick(0.5, 1.0, 1.5), rs=pick(0.5, 1.0), mlp=mlp))
        else:
            kv = pick(1, 2)
            layers.append(cdelta(kv * pick(1, 2), kv, pick(4, 8, 24), pick(4, 8, 16), pick(1, 2, 4), mlp=mlp))
    return make_cfg(layers, vocab=pick(40, 80), width=pick(24, 32, 48), streams=pick(None, 1, 2, 3), logit_scale=pick(0.25, 1.0, 2.0), ranks=(pick(3, 8), pick(4, 16)))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_from_the_designs_space(seed):
    cfg = drawn_cfg(100 + seed)
    toks = tokens(80, cfg.vocab, seed)
    for dtype in (torch.float32, torch.bfloat16):
        model, orc = build(cfg, dtype, seed=seed)
        want = orc.forward(toks)
        with gen_for(model) as gen:
            assert_close(gen.step([(0, toks)], list(range(80))), want, dtype, "whole")
            assert_close(in_portions(gen, 1, toks, [37] + [1] * 20 + [2, 5, 2]), want, dtype, "portions")
            assert gen.error_flags() == 0


@pytest.mark.parametrize("dim,vdim,heads,kv", [(9, 11, 4, 2), (17, 6, 2, 2), (40, 33, 2, 1), (64, 64, 3, 3), (128, 32, 2, 2), (200, 16, 1, 1)])
def test_delta_rule_in_chunks_against_the_oracle_and_the_token_by_token_kernel(dim, vdim, heads, kv):
    """Portions of at least 16 tokens run in chunks of 32 (every register layout of the chunk kernel), shorter ones token by token:
    ragged last chunks, portions on a carried state, a mixed batch, and decays from next to one down to a tenth per token."""
    cfg = make_cfg([cdelta(heads, kv, dim, vdim, 3)], vocab=59, width=40, streams=2, ranks=(6, 6))

    def edit(t):
        a = t["l0.mix.A_log"].float()
        t["l0.mix.A_log"] = torch.linspace(-6.0, 1.0, a.numel()).to(t["l0.mix.A_log"].dtype)      # per head: g from ~1 to ~e^-2.7 per token
    model, orc = build(cfg, torch.float32, seed=21, edit=edit)
    a, b = tokens(150, cfg.vocab, 30), tokens(47, cfg.vocab, 31)
    wa, wb = orc.forward(a), orc.forward(b)
    with gen_for(model) as gen:
        got = in_portions(gen, 0, a, [70, 33, 5, 17])                                        # chunks, a ragged chunk, the scan, a short chunk, the rest
        assert_close(got, wa, torch.float32, "chunks on a carried state")
        gen.release(0)
        gen.step([(0, a[:100]), (1, b[:20])], [])
        got = gen.step([(1, b[20:]), (0, a[100:])], list(range(27 + 50)))                    # two requests of unequal length in one step
        assert_close(got[:27], wb[20:], torch.float32, "batch b")
        assert_close(got[27:], wa[100:], torch.float32, "batch a")
        gen.release(0)
        gen.set_option("delta_chunk", 0)
        assert_close(gen.step([(0, a)], list(range(150))), wa, torch.float32, "token by token")
        gen.set_option("delta_chunk", 1)


def drawn_small_model(seed):
    """Layer sizes of a small real model (widths of 128 to 384, heads of 32 to 128, windows of 48 to 257): every mixer kind at least once."""
    g = torch.Generator().manual_seed(seed)

    def pick(*xs):
        return xs[int(torch.randint(0, len(xs), (1,), generator=g))]

    def mlp():
        return pick(None, dense(pick(256, 320, 200)))
    kinds = ["latent", "pair", "delta"] + [pick("latent", "pair", "delta") for _ in range(pick(1, 2))]
    layers = []
    for i in torch.randperm(len(kinds), generator=g).tolist():
        if kinds[i] == "latent":
            rd = pick(16, 32, 64, 8)
            layers.append(latent(pick(2, 4, 8, 6), pick(32, 64, 96, 48), rd, pick(32, 64, 48), pick(64, 128, 192, 96), pick(0.1, 0.125), pick(0, 64, 100, 257),
                                 base=pick(1e4, 1e6), scaling=pick(None, {"factor": pick(4.0, 8.0), "original": pick(256, 1024), "fast": pick(32.0, 16.0), "slow": pick(1.0, 2.0)}),
                                 mlp=mlp()))
        elif kinds[i] == "pair":
            kv, dim = pick(1, 2, 4), pick(32, 64, 96, 128, 48)
            layers.append(pair(kv * pick(1, 2, 4), kv, dim, pick(32, 64, 96, 48), pick(0.1, 0.125), pick(0, 48, 130, 256), pick(128, 384, 200),
                               rot_dims=pick(0, 16, 24, dim), base=pick(1e4, 5e5), ls=pick(1.0, 1.3, 0.8), rs=pick(1.0, 0.9), mlp=mlp()))
        else:
            kv = pick(1, 2, 3, 4)
            layers.append(cdelta(kv * pick(1, 2), kv, pick(32, 48, 64, 128), pick(32, 64, 128, 48), pick(2, 3, 4), mlp=mlp()))
    return make_cfg(layers, vocab=pick(320, 1000, 777), width=pick(128, 160, 256, 320, 384, 200), streams=pick(None, 1, 2, 3, 4), logit_scale=pick(0.3, 0.5, 1.0),
                    eps=pick(1e-5, 1e-6), ranks=(pick(16, 24, 32), pick(16, 24, 32)))


@pytest.mark.parametrize("seed", range(4))
def test_drawn_models_at_a_small_models_sizes(seed):
    """Whole prompt, prompt + single tokens, and ragged portions with chunk-sized and two-token pieces, in both precisions."""
    cfg = drawn_small_model(40 + seed)
    toks = tokens(330, cfg.vocab, 60 + seed)
    for dtype in (torch.float32, torch.bfloat16):
        model, orc = build(cfg, dtype, seed=seed)
        want = orc.forward(toks)
        with gen_for(model, capacity=340, max_step_tokens=340) as gen:
            assert_close(gen.step([(0, toks)], list(range(330))), want, dtype, "whole")
            assert_close(in_portions(gen, 1, toks, [290] + [1] * 40), want, dtype, "prompt and single tokens")
            gen.release(1)
            assert_close(in_portions(gen, 1, toks, [2, 3, 17, 97, 2, 33, 64, 5, 31, 2, 16] + [1] * 20), want, dtype, "portions")
            assert gen.error_flags() == 0
