"""Text-only decoder LMs given as a list of layers, backed by the sm_100a library (``b200_dlm_*``).

``DecoderLM`` owns the weights (like ``LMModel``); ``DecoderLMGen`` owns what the cache slots hold (latents, or keys and values,
carried convolution inputs and recurrent state, by the model's mixers) and runs steps (like ``LMGen`` owns the streaming state): a step is a ragged batch, any number of new tokens per cache slot, so prompt portions and single-token
decoding are the same call.  Nothing here computes: every operation is a kernel of ``libmoshi_b200.so``.
"""
from __future__ import annotations

import ctypes as C
import typing as tp

import torch

from .. import _lib
from ..config import BLOCKS, MIXERS, MLP_KINDS, ROT_PAIRINGS, ROT_SCALINGS, SINKS, DecoderLMConfig, MixerConfig

_DTYPES = {torch.bfloat16: _lib.B200_BF16, torch.float32: _lib.B200_F32}


def _fill_mixer(dst, m: MixerConfig) -> None:
    dst.kind, dst.heads, dst.dim, dst.vdim, dst.kv_heads, dst.kv_rank = MIXERS[m.kind], m.heads, m.dim, m.vdim, m.kv_heads, m.kv_rank
    dst.scale, dst.window, dst.conv_taps, dst.rot_dims, dst.rot_base = m.scale, m.window, m.conv, m.rot_dims, m.rot_base
    sc = m.rot_scaling or {}
    dst.rot_factor, dst.rot_low, dst.rot_high = float(sc.get("factor", 0.0)), float(sc.get("low", 1.0)), float(sc.get("high", 1.0))
    dst.rot_original, dst.gate_cap, dst.tau = float(sc.get("original", 0.0)), m.gate_cap, m.tau
    dst.rot_pairing = ROT_PAIRINGS[m.rot_pairing]
    dst.rot_scaling = ROT_SCALINGS[m.rot_scaling_kind if m.rot_scaling else None] if m.rot_scaling_kind else (1 if m.rot_scaling else 0)
    dst.rot_fast, dst.rot_slow = float(sc.get("fast", 0.0)), float(sc.get("slow", 0.0))
    dst.softcap, dst.v_mix = m.softcap, int(m.v_mix)
    dst.bias, dst.sink, dst.head_gate = int(m.bias), SINKS[m.sink], int(m.head_gate)
    if m.decay:
        dst.decay = (C.c_float * len(m.decay))(*m.decay)      # ctypes keeps the array alive with the struct; create() copies it


class DecoderLM:
    """Weights of a layer-list decoder LM on one B200.  Construct via ``loaders.get_decoder_lm``."""

    def __init__(self, cfg: DecoderLMConfig, tensors: tp.Iterable[tuple[str, torch.Tensor]] | tp.Mapping[str, torch.Tensor],
                 device: torch.device | str = "cuda", dtype: torch.dtype = torch.bfloat16, use_tc: bool = True):
        if dtype not in _DTYPES:
            raise ValueError("the decoder LM computes in bfloat16 or float32")
        self.cfg = cfg
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("moshi_b200.DecoderLM runs on a CUDA device only (no CPU fallback)")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype
        self.vocab, self.width = cfg.vocab, cfg.width
        self._lib = _lib.lib()
        self._h = C.c_void_p()
        layers = (_lib.DLMLayerC * len(cfg.layers))()
        for i, L in enumerate(cfg.layers):
            layers[i].mixer, layers[i].mlp, layers[i].ff = MIXERS[L.type], MLP_KINDS[L.mlp_kind], L.ff
            layers[i].experts, layers[i].top = L.experts, L.top
            layers[i].expert_limit, layers[i].router_scale = L.expert_limit, L.router_scale
            layers[i].a_scale, layers[i].b_scale = L.a_scale, L.b_scale
            for dst, m in zip((layers[i].a, layers[i].b), L.mixers()):
                if m is not None:
                    _fill_mixer(dst, m)
        c = _lib.DLMConfigC()
        c.vocab, c.width, c.n_layers = cfg.vocab, cfg.width, len(cfg.layers)
        c.embedding_scale, c.residual_mult, c.norm_eps = cfg.embedding_scale, cfg.residual_mult, cfg.norm_eps
        c.block, c.canon_taps, c.logit_softcap = BLOCKS[cfg.block], cfg.canon_taps, cfg.logit_softcap
        c.streams, c.logit_scale, c.tied_head = cfg.streams, cfg.logit_scale, int(cfg.tied_head)
        c.compute_dtype = _DTYPES[dtype]
        c.layers = layers
        items = tensors.items() if isinstance(tensors, tp.Mapping) else tensors
        with torch.cuda.device(self.device):
            _lib.check(self._lib.b200_dlm_create(C.byref(c), C.byref(self._h)))
            _lib.check(self._lib.b200_dlm_set_option(self._h, b"use_tc", int(use_tc)))
            for name, t in items:
                want = torch.float32 if t.dtype in (torch.float32, torch.float64, torch.int32, torch.int64) else torch.bfloat16
                t2 = t.detach().to(device=self.device, dtype=want).contiguous()
                shape = (C.c_int64 * max(t2.dim(), 1))(*t2.shape)
                _lib.check(self._lib.b200_dlm_load_tensor(self._h, name.encode(), _lib.ptr(t2), _lib.dtype_code(want), t2.dim(), shape))
                del t2
            _lib.check(self._lib.b200_dlm_finalize(self._h))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h is not None and h.value:
            try:
                self._lib.b200_dlm_destroy(h)
            except Exception:
                pass
            self._h = C.c_void_p()

    def eval(self) -> "DecoderLM":
        return self

    def algorithmic_bytes(self, tokens: int, context: int) -> int:
        return int(self._lib.b200_dlm_algorithmic_bytes(self._h, int(tokens), int(context)))

    def algorithmic_flops(self, tokens: int, context: int) -> int:
        return int(self._lib.b200_dlm_algorithmic_flops(self._h, int(tokens), int(context)))


class DecoderLMGen:
    """The cache of a ``DecoderLM`` (``slots`` requests of up to ``capacity`` tokens) and its step function."""

    def __init__(self, model: DecoderLM, slots: int, capacity: int, max_step_tokens: int = 2048, max_want: int | None = None,
                 trace_layers: bool = False, use_sampling: bool = False, temp: float = 0.8, top_k: int = 250):
        self.model = model
        self.slots, self.capacity = int(slots), int(capacity)
        self.max_step_tokens = int(max_step_tokens)
        self.max_want = int(max_want if max_want is not None else max_step_tokens)
        self.use_sampling, self.temp, self.top_k = use_sampling, temp, top_k
        self._lib, self._h = model._lib, model._h
        self._open = False
        with torch.cuda.device(model.device):
            _lib.check(self._lib.b200_dlm_set_option(self._h, b"trace_layers", int(trace_layers)))
            _lib.check(self._lib.b200_dlm_cache_begin(self._h, self.slots, self.capacity, self.max_step_tokens, self.max_want,
                                                      _lib.current_stream(model.device)))
        self._open = True
        self._last_want = 0
        self._last_tokens = 0

    def close(self) -> None:
        if self._open:
            with torch.cuda.device(self.model.device):
                self._lib.b200_dlm_cache_end(self._h)
            self._open = False

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self) -> "DecoderLMGen":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def set_option(self, name: str, value: int) -> None:
        _lib.check(self._lib.b200_dlm_set_option(self._h, name.encode(), int(value)))

    def kernel_times(self, reset: bool = True) -> dict[str, float]:
        """Milliseconds per class of operation since the last reset (needs ``set_option("time_kernels", 1)``)."""
        ms = (C.c_double * 6)()
        _lib.check(self._lib.b200_dlm_read_timers(self._h, ms, int(reset)))
        return dict(zip(("linear", "attention", "fold", "elementwise", "recurrent", "experts"), (float(x) for x in ms)))

    def release(self, slot: int) -> None:
        """The slot's request is finished: what it holds is given back."""
        _lib.check(self._lib.b200_dlm_release(self._h, int(slot)))

    def slot_length(self, slot: int) -> int:
        return int(self._lib.b200_dlm_slot_length(self._h, int(slot)))

    @torch.no_grad()
    def step(self, entries: tp.Sequence[tuple[int, tp.Sequence[int]]], want: tp.Sequence[int] = ()) -> torch.Tensor | None:
        """``entries``: (slot, new tokens) per request of the step; ``want``: indices into the step's concatenated tokens.
        Returns the logits f32 [len(want), vocab] on the device (None if nothing is wanted)."""
        dev = self.model.device
        slots = [int(s) for s, _ in entries]
        counts = [len(t) for _, t in entries]
        toks = [int(x) for _, t in entries for x in t]
        n, nw = len(entries), len(want)
        a_slots, a_counts = (C.c_int32 * n)(*slots), (C.c_int32 * n)(*counts)
        a_toks = (C.c_int32 * max(len(toks), 1))(*toks)
        a_want = (C.c_int32 * max(nw, 1))(*[int(w) for w in want])
        out = torch.empty(nw, self.model.vocab, device=dev, dtype=torch.float32) if nw else None
        with torch.cuda.device(dev):
            _lib.check(self._lib.b200_dlm_set_stream(self._h, _lib.current_stream(dev)))
            _lib.check(self._lib.b200_dlm_step(self._h, n, a_slots, a_counts, a_toks, nw, a_want, _lib.ptr(out)))
        self._last_want, self._last_tokens = nw, len(toks)
        return out

    @torch.no_grad()
    def sample(self, noise: torch.Tensor | None = None) -> torch.Tensor:
        """One token per logit row of the last step (the LM's sampler: softmax(logits / temp) -> top-k -> argmax(p / Exp(1));
        greedy when ``use_sampling`` is off or ``temp`` is 0) -> i64 [rows]."""
        dev = self.model.device
        sampling = bool(self.use_sampling and self.temp > 0)
        k = min(int(self.top_k), self.model.vocab)
        if sampling and noise is None:
            noise = torch.empty(self._last_want, k, device=dev, dtype=torch.float32).exponential_(1)
        if noise is not None:
            noise = noise.to(device=dev, dtype=torch.float32).contiguous()
        out = torch.empty(self._last_want, device=dev, dtype=torch.int64)
        with torch.cuda.device(dev):
            _lib.check(self._lib.b200_dlm_sample(self._h, _lib.ptr(noise), int(sampling), float(self.temp), k, _lib.ptr(out)))
        return out

    def read_buffer(self, name: str, dtype: torch.dtype, shape: tuple[int, ...]) -> torch.Tensor:
        out = torch.empty(shape, device=self.model.device, dtype=dtype)
        n = C.c_int64()
        with torch.cuda.device(self.model.device):
            _lib.check(self._lib.b200_dlm_read_buffer(self._h, name.encode(), _lib.ptr(out), out.numel() * out.element_size(), C.byref(n)))
        assert n.value == out.numel() * out.element_size(), (name, n.value, shape)
        return out

    def layer_outputs(self) -> torch.Tensor:
        """What every layer handed on in the last step, f32 [layers, tokens, width] (needs ``trace_layers=True``)."""
        return self.read_buffer("layers", torch.float32, (len(self.model.cfg.layers), self._last_tokens, self.model.width))

    def error_flags(self) -> int:
        return int(self.read_buffer("error_flags", torch.int32, (1,)).item())
