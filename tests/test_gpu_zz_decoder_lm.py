"""The text-only decoder LM (Likosun design) on the GPU against the float64 oracle (``oracle/decoder_lm.py``): every mechanism
alone, prompts whole / in portions / token by token, unequal batches, slot reuse, window edges of the kernels' own tiling, odd
sizes, and greedy generation through the scheduler and the command line."""
import ctypes as C
import json
import struct
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from moshi_b200.config import DecoderLMConfig
from moshi_b200.synth import iter_synth_decoder_tensors
from oracle.decoder_lm import F64, DecoderOracle, logit_error, sink_softmax

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def layer(heads, dim, vdim, rank, scale, ff):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def make_cfg(layers, vocab=130, width=72, emb=2.5, mult=0.7, eps=1e-5):
    return DecoderLMConfig.from_dict({"architecture": "Likosun", "vocab": vocab, "width": width, "embedding": {"scale": emb},
                                      "residual_mult": mult, "norm": {"eps": eps}, "layers": layers})


# odd sizes everywhere: nothing is a multiple of 8, heads and ranks differ per layer, one layer has no feed-forward
ODD = make_cfg([layer(3, 10, 7, 20, 0.4, 50), layer(5, 6, 9, 41, 0.21, None), layer(2, 13, 5, 33, 0.3, 37)], vocab=131, width=70)
# aligned sizes: in bfloat16 every linear takes the tcgen05 GEMM
ALIGNED = make_cfg([layer(4, 32, 24, 48, 0.2, 160), layer(4, 32, 24, 48, 0.15, 160)], vocab=200, width=96, emb=4.0, mult=0.5)


# latent sizes the tensor-core attention takes (bfloat16 only), heads differ per layer
TCATTN = make_cfg([layer(4, 32, 24, 64, 0.2, 160), layer(6, 16, 40, 128, 0.3, 96)], vocab=200, width=96, emb=4.0, mult=0.5)


def build(cfg, dtype, seed=3, edit=None, use_tc=True):
    from moshi_b200.models import DecoderLM
    tensors = dict(iter_synth_decoder_tensors(cfg, seed=seed))
    if edit:
        edit(tensors)
    return DecoderLM(cfg, tensors, device="cuda:0", dtype=dtype, use_tc=use_tc), DecoderOracle(cfg, tensors)


def gen_for(model, slots=3, capacity=256, **kw):
    from moshi_b200.models import DecoderLMGen
    return DecoderLMGen(model, slots=slots, capacity=capacity, max_step_tokens=kw.pop("max_step_tokens", 256), **kw)


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def assert_close(got, want, dtype, what=""):
    e = float(logit_error(got.cpu(), want).max())
    assert e < TOL[dtype], f"{what}: relative logit error {e:.3g}"


# ---- the attention kernel alone -------------------------------------------------------------------------------------------
def attn_oracle(qa, lat, sink, pos0):
    T, H, r = qa.shape
    out = torch.zeros(T, H, r, dtype=F64)
    for t in range(T):
        keys = lat[:pos0 + t + 1].to(F64)
        for h in range(H):
            p = sink_softmax((keys @ qa[t, h].to(F64))[None], sink[h].to(F64).reshape(1, 1))[0]
            out[t, h] = p @ keys
    return out


def run_attn(qa, lat, sink, pos0, nsplit=0, tensor_cores=1):
    from moshi_b200 import _lib
    T, H, r = qa.shape
    out = torch.empty(T, H, r, device="cuda", dtype=torch.float32)
    q, l, s = qa.cuda().contiguous(), lat.cuda().contiguous(), sink.cuda().contiguous()
    _lib.check(_lib.lib().b200_op_latent_attention(_lib.ptr(q), _lib.ptr(l), _lib.dtype_code(lat.dtype), _lib.ptr(s), _lib.ptr(out),
                                                   T, H, r, pos0, nsplit, tensor_cores, _lib.current_stream(torch.device("cuda:0"))))
    return out.cpu()


@pytest.mark.parametrize("T,H,r,pos0,nsplit", [
    (1, 1, 1, 0, 0), (1, 3, 40, 30, 0), (1, 3, 40, 31, 0), (1, 3, 40, 32, 2), (2, 3, 40, 63, 0), (5, 6, 96, 0, 0), (7, 5, 33, 250, 3),
    (3, 16, 64, 100, 0), (3, 17, 130, 40, 2), (2, 2, 520, 70, 0), (40, 2, 24, 0, 1), (1, 8, 300, 700, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_kernel(T, H, r, pos0, nsplit, dtype):
    g = torch.Generator().manual_seed(T * 1000 + r)
    qa = torch.randn(T, H, r, generator=g) * (1.5 / r ** 0.5)
    lat = torch.randn(pos0 + T, r, generator=g).to(dtype)
    sink = torch.randn(H, generator=g)
    got = run_attn(qa, lat, sink, pos0, nsplit, tensor_cores=0)
    want = attn_oracle(qa, lat, sink, pos0)
    assert (got.to(F64) - want).abs().max() < 2e-5


@pytest.mark.parametrize("T,H,r,pos0,nsplit", [
    (1, 16, 64, 0, 0), (1, 16, 512, 100, 0), (1, 16, 512, 2047, 7), (3, 5, 128, 30, 0), (3, 5, 128, 31, 2), (2, 8, 192, 63, 1), (40, 3, 320, 0, 1),
    (70, 2, 256, 500, 0), (1, 40, 448, 33, 3), (17, 1, 384, 15, 0)])
def test_latent_attention_on_tensor_cores(T, H, r, pos0, nsplit):
    """bf16 latents of 64 .. 512 elements: the mma kernel against the oracle and against the CUDA-core kernel.  Queries and
    softmax weights enter the tensor cores as bf16, hence the looser bound against the float64 oracle."""
    g = torch.Generator().manual_seed(T * 1000 + r + pos0)
    qa = torch.randn(T, H, r, generator=g) * (1.5 / r ** 0.5)
    lat = torch.randn(pos0 + T, r, generator=g).to(torch.bfloat16)
    sink = torch.randn(H, generator=g)
    got = run_attn(qa, lat, sink, pos0, nsplit, tensor_cores=1)
    ref = run_attn(qa, lat, sink, pos0, nsplit, tensor_cores=0)
    want = attn_oracle(qa, lat, sink, pos0)
    assert (ref.to(F64) - want).abs().max() < 2e-5
    assert (got.to(F64) - want).abs().max() < 2e-2 and (got.to(F64) - want).abs().mean() < 1.5e-3


@pytest.mark.parametrize("far", [0, 3, 31, 32, 33, 63, 64, 255, 256, 698, 699])
def test_one_key_stands_out_on_tensor_cores(far):
    g = torch.Generator().manual_seed(far)
    r, H, n = 64, 3, 700
    lat = (torch.randn(n, r, generator=g) * 0.3).to(torch.bfloat16)
    lf = lat.float()
    qa = torch.randn(2, H, r, generator=g) * 0.05 + 25.0 * lf[far] / (lf[far] @ lf[far])
    for nsplit in (0, 1, 5):
        got = run_attn(qa, lat, torch.zeros(H), n - 2, nsplit)
        want = attn_oracle(qa, lat, torch.zeros(H), n - 2)
        assert (got.to(F64) - want).abs().max() < 2e-2
    if far < n - 1:
        assert (got[0] - lf[far]).abs().max() < 2e-2 and (got[1] - lf[far]).abs().max() < 2e-2
    else:
        assert (got[1] - lf[far]).abs().max() < 2e-2 and (got[0] - lf[far]).abs().max() > 0.1


@pytest.mark.parametrize("far", [0, 3, 31, 32, 33, 63, 64, 255, 256, 698, 699])
def test_one_key_stands_out_wherever_it_sits(far):
    """One key among 700 carries nearly all the weight (its score is raised by 25): far back, at the edges of the kernel's
    32-key tiles and of its key splits, and the newest key itself.  Query 0 must NOT see the key of query 1 (position 699)."""
    g = torch.Generator().manual_seed(far)
    r, H, n = 48, 3, 700
    lat = torch.randn(n, r, generator=g) * 0.3
    qa = torch.randn(2, H, r, generator=g) * 0.05
    qa = qa + 25.0 * lat[far] / (lat[far] @ lat[far])          # score of key `far` += 25 for every row
    sink = torch.zeros(H)
    for nsplit in (0, 1, 5):
        got = run_attn(qa, lat, sink, n - 2, nsplit)
        want = attn_oracle(qa, lat, sink, n - 2)
        assert (got.to(F64) - want).abs().max() < 2e-5
    if far < n - 1:
        assert (got[0] - lat[far]).abs().max() < 1e-3 and (got[1] - lat[far]).abs().max() < 1e-3
    else:                                                       # only query 1 may see key 699
        assert (got[1] - lat[far]).abs().max() < 1e-3 and (got[0] - lat[far]).abs().max() > 0.1


def test_sink_takes_weight_but_gives_no_value():
    g = torch.Generator().manual_seed(0)
    lat, qa = torch.randn(50, 32, generator=g), torch.randn(1, 2, 32, generator=g) * 0.1
    got = run_attn(qa, lat, torch.tensor([30.0, -30.0]), 49)
    want = attn_oracle(qa, lat, torch.tensor([30.0, -30.0]), 49)
    assert (got.to(F64) - want).abs().max() < 2e-5
    assert got[0, 0].abs().max() < 1e-6 and got[0, 1].abs().max() > 1e-2       # head 0: the sink holds all the weight


# ---- whole model ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [ODD, ALIGNED, TCATTN], ids=["odd", "aligned", "tcattn"])
def test_whole_prompt_and_every_layer(cfg, dtype):
    model, orc = build(cfg, dtype)
    toks = tokens(45, cfg.vocab, 1)
    with gen_for(model, trace_layers=True) as gen:
        got = gen.step([(0, toks)], list(range(len(toks))))
        layers = gen.layer_outputs().cpu()
        assert gen.error_flags() == 0
    want, handed = orc.forward(toks, return_layers=True)
    for i in range(len(cfg.layers)):
        d = (layers[i].to(F64) - handed[i]).abs().max() / handed[i].abs().max()
        assert d < (1e-5 if dtype == torch.float32 else 2e-2), f"layer {i}: {d:.3g}"
    assert_close(got, want, dtype)


def test_bf16_linears_on_cuda_cores_and_on_tcgen05_agree():
    toks = tokens(300, ALIGNED.vocab, 2)              # more than 256 rows: the tensor-core GEMM runs in two row blocks
    outs = []
    for use_tc in (False, True):
        model, orc = build(ALIGNED, torch.bfloat16, use_tc=use_tc)
        with gen_for(model, capacity=512, max_step_tokens=512) as gen:
            outs.append(gen.step([(0, toks)], [0, 1, 100, 255, 256, 257, 299]).cpu())
    want = orc.forward(toks)[[0, 1, 100, 255, 256, 257, 299]]
    assert_close(outs[0], want, torch.bfloat16, "cuda cores")
    assert_close(outs[1], want, torch.bfloat16, "tcgen05")


@pytest.mark.parametrize("what", ["mixer_only", "gate_open", "gate_shut", "plain_residual", "scale_not_rsqrt_dim"])
def test_mechanisms_in_isolation(what):
    """One mechanism at a time through one- or two-layer models whose other parts are switched off by their weights."""
    lay = [layer(3, 8, 6, 12, 0.35, None if what == "mixer_only" else 30)]
    if what == "plain_residual":
        lay = lay * 3
    cfg = make_cfg(lay, vocab=60, width=40, emb=1.0, mult=1.0 if what == "plain_residual" else 0.6)

    def edit(t):
        if what in ("gate_open", "gate_shut"):
            for k in ("l0.rg1", "l0.rg2"):
                t[k] = torch.zeros_like(t[k])
                t[k + ".b"] = torch.full_like(t[k + ".b"], 30.0 if what == "gate_open" else -30.0)
        if what == "plain_residual":               # the average keeps only the newest result: an ordinary residual stream
            for i in range(3):
                a = torch.zeros(i + 2)
                a[-1] = 1.0
                t[f"l{i}.dwa"] = a.to(torch.bfloat16)
    model, orc = build(cfg, torch.float32, edit=edit)
    toks = tokens(20, cfg.vocab, 4)
    with gen_for(model, trace_layers=True) as gen:
        got = gen.step([(0, toks)], list(range(20)))
        handed = gen.layer_outputs().cpu().to(F64)
    want, oh = orc.forward(toks, return_layers=True)
    assert_close(got, want, torch.float32, what)
    x0 = orc.W["embed"][torch.tensor(toks)] * cfg.embedding_scale
    if what == "gate_shut":                        # nothing passes the gates: the layer hands on a0 * x + a1 * x
        a = orc.W["l0.dwa"]
        assert (handed[0] - (a[0] + a[1]) * x0).abs().max() < 1e-4
    if what == "gate_open":
        assert (handed[0] - oh[0]).abs().max() < 1e-4 and (oh[0] - (orc.W["l0.dwa"].sum()) * x0).abs().max() > 1e-2


@pytest.mark.parametrize("cfg", [ODD, TCATTN], ids=["odd", "tcattn"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_portions_and_single_tokens_equal_the_whole_prompt(dtype, cfg):
    model, orc = build(cfg, dtype)
    toks = tokens(75, cfg.vocab, 5)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        whole = gen.step([(0, toks)], list(range(75))).cpu()
        for sizes in ([2, 3, 31, 2, 26, 1, 1, 2, 7], [33, 31, 2, 2, 2, 2, 2, 1], [1] * 75):
            assert sum(sizes) == 75
            rows, at = [], 0
            for n in sizes:
                rows.append(gen.step([(1, toks[at:at + n])], list(range(n))).cpu())
                at += n
            gen.release(1)
            got = torch.cat(rows)
            assert_close(got, want, dtype, f"portions {sizes[:4]}")
            assert float(logit_error(got, whole.to(F64)).max()) < (1e-5 if dtype == torch.float32 else 2e-2)
    assert_close(whole, want, dtype, "whole")


def test_long_decoding_token_by_token():
    cfg = make_cfg([layer(2, 16, 8, 24, 0.25, 48)] * 2, vocab=90, width=48)
    model, orc = build(cfg, torch.float32)
    toks = tokens(140, cfg.vocab, 6)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        rows = [gen.step([(2, toks[:20])], [19]).cpu()]
        for t in range(20, 140):
            rows.append(gen.step([(2, [toks[t]])], [0]).cpu())
    assert_close(torch.cat(rows), want[19:], torch.float32)


def test_long_decoding_on_the_tensor_core_attention():
    """bfloat16, latents the tensor-core kernel takes: 100 single tokens cross three 32-key tile edges, the number of key splits
    changes on the way, and no copy into shared memory is ever given up on (device error flags stay 0)."""
    model, orc = build(TCATTN, torch.bfloat16)
    toks = tokens(131, TCATTN.vocab, 8)
    want = orc.forward(toks)
    with gen_for(model) as gen:
        rows = [gen.step([(1, toks[:31])], [30]).cpu()]
        for t in range(31, 131):
            rows.append(gen.step([(1, [toks[t]])], [0]).cpu())
        assert gen.error_flags() == 0
    assert_close(torch.cat(rows), want[30:], torch.bfloat16)


@pytest.mark.parametrize("cfg", [ODD, TCATTN], ids=["odd", "tcattn"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_batch_equals_each_request_alone(dtype, cfg):
    model, orc = build(cfg, dtype)
    reqs = [tokens(n, cfg.vocab, 10 + n) for n in (5, 67, 18, 1)]
    want = [orc.forward(r) for r in reqs]
    with gen_for(model, slots=4) as gen:
        # step 1: three prompts of unequal length (one of them only in part); step 2: the rest of it, one decoded token, a new prompt
        a = gen.step([(0, reqs[0]), (1, reqs[1][:40]), (2, reqs[2][:17])], list(range(5 + 40 + 17))).cpu()
        b = gen.step([(1, reqs[1][40:]), (2, reqs[2][17:]), (3, reqs[3])], list(range(27 + 1 + 1))).cpu()
    got = [a[:5], torch.cat([a[5:45], b[:27]]), torch.cat([a[45:62], b[27:28]]), b[28:29]]
    for g, w, r in zip(got, want, reqs):
        assert_close(g, w, dtype, f"request of {len(r)} tokens")


def test_slots_are_given_back_and_used_again():
    cfg = ODD
    model, orc = build(cfg, torch.float32)
    long, short = tokens(90, cfg.vocab, 20), tokens(9, cfg.vocab, 21)
    with gen_for(model, slots=1, capacity=100) as gen:
        gen.step([(0, long)], [])
        assert gen.slot_length(0) == 90
        with pytest.raises(Exception):
            gen.step([(0, tokens(11, cfg.vocab, 22))], [])           # 101 tokens do not fit
        assert gen.slot_length(0) == 90
        gen.release(0)
        got = gen.step([(0, short[:4])], list(range(4))).cpu()       # old latents lie behind the new request's keys: never seen
        got = torch.cat([got, gen.step([(0, short[4:])], list(range(5))).cpu()])
    assert_close(got, orc.forward(short), torch.float32)


def test_wide_latent_and_many_heads():
    """Ranks above 512 take the kernel's two-rows-per-warp form; 20 heads span two row tiles per token."""
    cfg = make_cfg([layer(20, 8, 8, 520, 0.2, 64)], vocab=80, width=64)
    model, orc = build(cfg, torch.float32)
    toks = tokens(12, cfg.vocab, 30)
    with gen_for(model) as gen:
        got = gen.step([(0, toks[:10])], list(range(10))).cpu()
        got = torch.cat([got, gen.step([(0, toks[10:11])], [0]).cpu(), gen.step([(0, toks[11:])], [0]).cpu()])
    assert_close(got, orc.forward(toks), torch.float32)


def test_token_outside_the_vocabulary_raises_the_error_flag():
    model, _ = build(ALIGNED, torch.bfloat16)
    with gen_for(model) as gen:
        gen.step([(0, [1, ALIGNED.vocab + 5])], [])
        assert gen.error_flags() == 1


# ---- generation through the scheduler and the command line ----------------------------------------------------------------------
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
                break                                                # after a tie the two trajectories differ: stop comparing


def write_model(folder, cfg, tensors):
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg.to_dict()))
    header, data = {}, b""
    for k, t in tensors.items():
        raw = t.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()      # reshape: a scalar has no axis to view as bytes
        header[k] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [len(data), len(data) + len(raw)]}
        data += raw
    hj = json.dumps(header).encode()
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + data)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_command_line_replays_steps_and_generates(tmp_path, dtype):
    cfg = ODD
    tensors = dict(iter_synth_decoder_tensors(cfg, seed=8))
    write_model(tmp_path / "m", cfg, tensors)
    orc = DecoderOracle(cfg, tensors)
    a, b = tokens(30, cfg.vocab, 50), tokens(6, cfg.vocab, 51)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:21], "want": [0, 20]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[21:], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": b, "want": [5]}], "end": ["b"]}]
    (tmp_path / "out").mkdir()
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype, "--out", str(tmp_path / "out"),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (tmp_path / "out" / "1.f32").exists()
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


def test_sampling_goes_through_the_lm_sampler():
    """temp > 0: the LM's sampler (softmax / top-k / Exp(1) race) on the bf16 rounding of the logits; with top_k = 1 it is the
    arg-max, with given noise the winner maximises p / noise among the top k."""
    cfg = ODD
    model, orc = build(cfg, torch.float32)
    toks = tokens(12, cfg.vocab, 60)
    want = orc.forward(toks)[-1]
    with gen_for(model, use_sampling=True, temp=1.0, top_k=1) as gen:
        gen.step([(0, toks)], [11])
        assert int(gen.sample()[0]) in torch.topk(want, 2).indices.tolist()
        gen.top_k = 6
        noise = torch.empty(1, 6).exponential_(1, generator=torch.Generator().manual_seed(0))
        tok = int(gen.sample(noise)[0])
        lg = gen.read_buffer("logits", torch.float32, (1, cfg.vocab))[0].cpu().bfloat16().float()
        vals, idx = torch.sort(lg, descending=True, stable=True)
        p = torch.softmax(vals[:6], -1)
        assert tok == int(idx[int(torch.argmax(p / noise[0]))])
