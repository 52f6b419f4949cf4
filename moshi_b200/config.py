"""Hyper-parameter records for the two models on the hot path.

The field names and defaults restate the reference's configuration dictionaries so that the same
JSON / dict a reference user has keeps working:

* Mimi: ``moshi/moshi/models/loaders.py:38-88`` (``_seanet_kwargs``, ``_quantizer_kwargs``,
  ``_transformer_kwargs``, ``_mimi_config``).
* Moshi LM: ``configs/moshi_7b_202409.json`` and ``loaders.py:90-119`` (``_lm_kwargs``).

Only the options the 7B / Mimi hot path uses are honoured by the CUDA path; anything else raises
at construction time instead of silently computing something different.
"""
from __future__ import annotations

import dataclasses
import json
import typing as tp
from dataclasses import dataclass, field


@dataclass
class MimiConfig:
    sample_rate: int = 24000
    frame_rate: float = 12.5
    channels: int = 1
    # SEANet (loaders.py:38-58)
    dimension: int = 512
    n_filters: int = 64
    n_residual_layers: int = 1
    ratios: tp.List[int] = field(default_factory=lambda: [8, 6, 5, 4])  # decoder order
    kernel_size: int = 7
    residual_kernel_size: int = 3
    last_kernel_size: int = 3
    dilation_base: int = 2
    compress: int = 2
    # transformer bottlenecks (loaders.py:65-80)
    tr_d_model: int = 512
    tr_num_heads: int = 8
    tr_num_layers: int = 8
    tr_dim_feedforward: int = 2048
    tr_context: int = 250
    tr_max_period: float = 10000.0
    tr_layer_scale: float = 0.01
    # quantizer (loaders.py:59-64)
    q_dimension: int = 256
    q_bins: int = 2048
    q_n_q: int = 32          # codebooks stored in the checkpoint
    q_n_semantic: int = 1
    num_codebooks: int = 8   # codebooks active (loaders.py:323-326 default)

    @property
    def hop_length(self) -> int:
        h = 1
        for r in self.ratios:
            h *= r
        return h

    @property
    def encoder_frame_rate(self) -> float:
        return self.sample_rate / self.hop_length

    @property
    def frame_size(self) -> int:
        return int(self.sample_rate / self.frame_rate)

    @property
    def resample_stride(self) -> int:
        return int(self.encoder_frame_rate / self.frame_rate)

    @staticmethod
    def from_reference_dict(cfg: dict | None, num_codebooks: int = 8) -> "MimiConfig":
        """Accepts the nested dict layout of ``loaders._mimi_config``."""
        if cfg is None:
            return MimiConfig(num_codebooks=num_codebooks)
        sea, qt, tr = cfg["seanet"], cfg["quantizer"], cfg["transformer"]
        unsupported = []
        if sea.get("norm", "none") != "none":
            unsupported.append("seanet.norm")
        if sea.get("pad_mode", "constant") != "constant":
            unsupported.append("seanet.pad_mode")
        if not sea.get("true_skip", True):
            unsupported.append("seanet.true_skip")
        if tr.get("gating", "none") != "none" or tr.get("norm", "layer_norm") != "layer_norm":
            unsupported.append("transformer.gating/norm")
        if tr.get("positional_embedding", "rope") != "rope":
            unsupported.append("transformer.positional_embedding")
        if sea.get("activation", "ELU") != "ELU" or sea.get("activation_params", {"alpha": 1.0}).get("alpha", 1.0) != 1.0:
            unsupported.append("seanet.activation")
        if not sea.get("causal", True) or not tr.get("causal", True):
            unsupported.append("causal=False")
        if sea.get("disable_norm_outer_blocks", 0) != 0:
            unsupported.append("seanet.disable_norm_outer_blocks")
        if not tr.get("conv_layout", True):
            unsupported.append("transformer.conv_layout=False")
        if unsupported:
            raise ValueError(f"Mimi options outside the B200 hot path: {unsupported}")
        return MimiConfig(
            sample_rate=cfg["sample_rate"], frame_rate=cfg["frame_rate"], channels=cfg["channels"],
            dimension=sea["dimension"], n_filters=sea["n_filters"],
            n_residual_layers=sea["n_residual_layers"], ratios=list(sea["ratios"]),
            kernel_size=sea["kernel_size"], residual_kernel_size=sea["residual_kernel_size"],
            last_kernel_size=sea["last_kernel_size"], dilation_base=sea["dilation_base"],
            compress=sea["compress"], tr_d_model=tr["d_model"], tr_num_heads=tr["num_heads"],
            tr_num_layers=tr["num_layers"], tr_dim_feedforward=tr["dim_feedforward"],
            tr_context=tr["context"], tr_max_period=float(tr["max_period"]),
            tr_layer_scale=tr["layer_scale"], q_dimension=qt["dimension"], q_bins=qt["bins"],
            q_n_q=qt["n_q"], num_codebooks=num_codebooks)

    def to_reference_dict(self) -> dict:
        """The nested dict ``loaders.get_mimi(mimi_config=...)`` takes (used by the golden generator)."""
        seanet = {
            "channels": self.channels, "dimension": self.dimension, "causal": True,
            "n_filters": self.n_filters, "n_residual_layers": self.n_residual_layers,
            "activation": "ELU", "compress": self.compress, "dilation_base": self.dilation_base,
            "disable_norm_outer_blocks": 0, "kernel_size": self.kernel_size,
            "residual_kernel_size": self.residual_kernel_size,
            "last_kernel_size": self.last_kernel_size, "norm": "none", "pad_mode": "constant",
            "ratios": list(self.ratios), "true_skip": True,
        }
        quantizer = {"dimension": self.q_dimension, "n_q": self.q_n_q, "bins": self.q_bins,
                     "input_dimension": self.dimension, "output_dimension": self.dimension}
        transformer = {
            "d_model": self.tr_d_model, "num_heads": self.tr_num_heads,
            "num_layers": self.tr_num_layers, "causal": True, "layer_scale": self.tr_layer_scale,
            "context": self.tr_context, "conv_layout": True, "max_period": self.tr_max_period,
            "gating": "none", "norm": "layer_norm", "positional_embedding": "rope",
            "dim_feedforward": self.tr_dim_feedforward, "input_dimension": self.dimension,
            "output_dimensions": [self.dimension],
        }
        return {"sample_rate": self.sample_rate, "channels": self.channels,
                "frame_rate": self.frame_rate, "seanet": seanet, "quantizer": quantizer,
                "transformer": transformer}


@dataclass
class LMConfig:
    """``LMModel.__init__`` keyword arguments (``lm.py:76-113``) restricted to the 7B family."""
    dim: int = 4096
    text_card: int = 32000
    existing_text_padding_id: int = 3
    n_q: int = 16
    dep_q: int = 8
    card: int = 2048
    num_heads: int = 32
    num_layers: int = 32
    hidden_scale: float = 4.125
    causal: bool = True
    layer_scale: tp.Optional[float] = None
    context: int = 3000
    max_period: float = 10000.0
    gating: str = "silu"
    norm: str = "rms_norm_f32"
    positional_embedding: str = "rope"
    depformer_dim: int = 1024
    depformer_dim_feedforward: int = 4224
    depformer_num_heads: int = 16
    depformer_num_layers: int = 6
    depformer_layer_scale: tp.Optional[float] = None
    depformer_multi_linear: bool = True
    depformer_context: int = 8
    depformer_max_period: float = 10000.0
    depformer_gating: str = "silu"
    depformer_pos_emb: str = "none"
    depformer_weights_per_step: bool = True
    quantize: bool = False       # LMModel(quantize=True), lm.py:107,242-243: every nn.Linear becomes an int8 QLinear
    extra_heads_num_heads: int = 0   # lm.py:108-109, 224-226: nn.Linear(dim, extra_heads_dim) heads on the temporal output (STT)
    extra_heads_dim: int = 6
    # lm.py:110-118 via loaders.get_conditioner_provider / get_condition_fuser (loaders.py:449-487): the JSON's "conditioners"
    # and "fuser" sections (configs/moshi_dev_2b.json).  Only LUT conditioners fused by "sum" are on the step path.
    conditioners: tp.Optional[dict] = None
    fuser: tp.Optional[dict] = None
    cross_attention: bool = False
    delays: tp.List[int] = field(
        default_factory=lambda: [0, 0, 1, 1, 1, 1, 1, 1, 1, 0, 1, 1, 1, 1, 1, 1, 1])

    @property
    def num_codebooks(self) -> int:
        return self.n_q + 1

    @property
    def max_delay(self) -> int:
        return max(self.delays)

    @property
    def ffn_hidden(self) -> int:
        """Gated hidden width, ``gating.py:52-58``."""
        return _gated_hidden(self.dim, int(self.hidden_scale * self.dim))

    @property
    def depformer_ffn_hidden(self) -> int:
        return _gated_hidden(self.depformer_dim, self.depformer_dim_feedforward)

    @staticmethod
    def from_dict(d: dict) -> "LMConfig":
        d = dict(d)
        d.pop("depformer_causal", None)  # deprecated key, dropped by loaders.py:391-392
        known = {f.name for f in dataclasses.fields(LMConfig)}
        extra = sorted(set(d) - known)
        if extra:
            raise ValueError(f"LM options outside the B200 hot path: {extra}")
        cfg = LMConfig(**d)
        cfg.check_supported()
        return cfg

    @staticmethod
    def from_json(path: str) -> "LMConfig":
        with open(path) as f:
            return LMConfig.from_dict(json.load(f))

    def to_reference_kwargs(self) -> dict:
        """Keyword arguments of the reference's ``LMModel`` (the ``conditioners`` / ``fuser`` JSON sections are turned into
        modules by ``loaders.get_conditioner_provider`` / ``get_condition_fuser`` there, so they are not constructor arguments)."""
        d = dataclasses.asdict(self)
        d.pop("conditioners")
        d.pop("fuser")
        return d

    def check_supported(self) -> None:
        bad = []
        if self.norm != "rms_norm_f32":
            bad.append("norm")
        if self.gating != "silu" or self.depformer_gating != "silu":
            bad.append("gating")
        if self.positional_embedding != "rope" or self.depformer_pos_emb != "none":
            bad.append("positional_embedding")
        if self.layer_scale is not None or self.depformer_layer_scale is not None:
            bad.append("layer_scale")
        if not (self.depformer_multi_linear and self.depformer_weights_per_step):
            bad.append("depformer_multi_linear/weights_per_step")
        if len(self.delays) != self.n_q + 1:
            bad.append("delays")
        if not self.causal:
            bad.append("causal=False")
        if self.dep_q and self.depformer_context < self.dep_q:
            bad.append("depformer_context < dep_q (the depformer attends over all of a frame's codebooks)")
        if self.cross_attention or (self.fuser or {}).get("cross") or (self.fuser or {}).get("prepend"):
            bad.append("cross-attention / prepend conditioning (only fuser.sum is on the step path)")
        for name, c in (self.conditioners or {}).items():
            if c.get("type") != "lut":
                bad.append(f"conditioner {name!r} of type {c.get('type')!r} (only 'lut')")
        if not 0 <= self.dep_q <= 16 or not 1 <= self.n_q <= 32 or self.dep_q > self.n_q:
            bad.append("n_q / dep_q (n_q <= 32, 0 <= dep_q <= 16)")
        if self.dim % self.num_heads or (self.dep_q and self.depformer_dim % self.depformer_num_heads):
            bad.append("heads")
        if self.quantize and any(k % 16 for k in (self.dim, self.ffn_hidden, self.depformer_dim, self.depformer_ffn_hidden)):
            bad.append("quantize (int8 k-extents must be multiples of 16)")
        if bad:
            raise ValueError(f"LM options outside the B200 hot path: {bad}")


def _gated_hidden(dim: int, dim_feedforward: int) -> int:
    if dim_feedforward == 4 * dim:
        return (21 * dim) // 8
    return (2 * dim_feedforward) // 3


MOSHI_7B = LMConfig()


def tiny_lm_config(**over) -> LMConfig:
    """A scaled-down member of the 7B family that the CPU oracle steps in milliseconds."""
    base = dict(dim=256, text_card=500, n_q=16, dep_q=8, card=64, num_heads=2, num_layers=3,
                hidden_scale=4.125, context=12, depformer_dim=128, depformer_dim_feedforward=528,
                depformer_num_heads=2, depformer_num_layers=2)
    base.update(over)
    return LMConfig(**base)


# ---------------------------------------------------------------------------------------------------
# Decoder LMs given as a list of layers (text-only; no reference counterpart)
# ---------------------------------------------------------------------------------------------------
MIXERS = {"latent_attention": 1, "window_attention": 2, "gla": 3, "mlstm": 4, "parallel": 5,    # name -> B200_MIXER_*
          "sigmoid_attention": 6, "retention": 7, "delta": 8, "mingru": 9, "channel_delta": 10}
# feed-forward kind -> B200_MLP_*: "dense" / "moe" are the squared-ReLU layers (a null "mlp" = none), "gated_gelu" a gated dense
# layer with the tanh form of GELU, "moe_clamped_glu" routed experts with clamped gates behind a sigmoid router
MLP_KINDS = {None: 0, "dense": 1, "moe": 2, "gated_gelu": 3, "moe_clamped_glu": 4}
BLOCKS = {"gated_depth_average": 0, "sandwich": 1, "parallel_residual": 2, "pre_norm_streams": 3}  # block arrangement -> B200_BLOCK_*
NO_WINDOW = 1 << 30                                                                               # a window attention without a mask: every earlier key is seen
SINKS = {"learned": 0, "none": 1, "unit": 2}                                                      # softmax denominator's extra term -> B200_SINK_*
ROT_PAIRINGS = {"halves": 0, "adjacent": 1}                                                       # -> B200_ROT_HALVES / B200_ROT_ADJACENT
ROT_SCALINGS = {None: 0, "bands": 1, "ramp": 2}                                                   # -> B200_ROT_PLAIN / BANDS / RAMP


@dataclass
class MixerConfig:
    """One token mixer with its sizes and constants (the fields a kind does not use stay 0).

    ``window_attention``: ``kv_heads`` key/value heads, position p attends to keys j with 0 <= p - j < ``window``, a causal
    convolution of ``conv`` taps on the projected q / k / v, rotary positions on the first ``rot_dims`` dimensions of a head with
    base ``rot_base`` and (optionally) wavelength-dependent rescaling ``rot_scaling`` = {factor, low, high, original}.
    ``gla``: per-channel decay sigmoid(z)^(1 / tau), z through a bottleneck of ``decay_rank`` (a tensor's shape, not a config key).
    ``mlstm``: both gate pre-activations are capped by ``gate_cap * tanh(. / gate_cap)``.
    ``sigmoid_attention``: causal, weights sigmoid(softcap * tanh(q.k * scale / softcap) + bias) mixed over heads after the sigmoid;
    ``rot_pairing`` "adjacent" turns dimension 2i with 2i + 1; ``rot_scaling_kind`` "ramp" reads ``rot_scaling`` = {factor, original,
    fast, slow}; ``v_mix``: values blended with those of the first such layer.  ``retention``: one fixed ``decay`` per head.
    ``delta``: gated delta rule behind convolutions of ``conv`` taps, ``kv_heads`` query/key heads shared by ``heads`` value heads.
    ``channel_delta``: the same with one decay per head and key channel through a bottleneck of ``decay_rank``, and a sigmoid
    output gate through one of ``gate_rank`` (both are tensor shapes, not config keys).  ``mingru``: an element-wise gated
    recurrence of ``dim`` channels.  ``bias``: the q / k / v (or gate / candidate) projections add a bias.  ``sink``: what the
    softmax denominator holds beside the keys ("learned": exp of a weight per head, "none", "unit": one).  ``head_gate``: a
    sigmoid gate per head on the attention's result.  A ``latent_attention`` with ``rot_dims`` > 0 has that many rotated
    query / key dimensions per head beside its ``dim`` unrotated ones; the rotated key part is one row shared by the heads."""
    kind: str
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    window: int = 0
    conv: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_scaling: tp.Optional[dict] = None
    gate_cap: float = 0.0
    tau: float = 1.0
    decay_rank: int = 16
    rot_pairing: str = "halves"
    rot_scaling_kind: tp.Optional[str] = None      # None: "bands" when rot_scaling is given (the window attention's form)
    softcap: float = 0.0
    v_mix: bool = False
    decay: tp.Optional[tp.List[float]] = None
    bias: bool = False
    sink: str = "learned"
    head_gate: bool = False
    gate_rank: int = 16


def _window_attention_from_dict(m: dict) -> MixerConfig:
    rot = m.get("rot") or {}
    return MixerConfig(kind="window_attention", heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                       scale=float(m["scale"]), window=int(m["mask"]["size"]), conv=int(m.get("conv", 0)), rot_dims=int(rot.get("dims", 0)),
                       rot_base=float(rot.get("base", 10000.0)), rot_scaling=dict(rot["scaling"]) if rot.get("scaling") else None)


def _window_attention_to_dict(m: MixerConfig) -> dict:
    rot: dict = {"base": m.rot_base, "dims": m.rot_dims}
    if m.rot_scaling:
        rot["scaling"] = dict(m.rot_scaling)
    return {"conv": m.conv, "dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "mask": {"size": m.window}, "rot": rot, "scale": m.scale, "vdim": m.vdim}


@dataclass
class DecoderLayerConfig:
    """One entry of ``layers``: the token mixer with its sizes, and the feed-forward (``mlp_kind`` None = the layer has none).
    The flat fields describe a ``latent_attention`` mixer; the other kinds are carried as ``MixerConfig`` in ``a`` (the only
    mixer, or the left one of a ``parallel`` pair) and ``b`` (the right one)."""
    type: str
    heads: int = 0
    dim: int = 0
    vdim: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    mlp_kind: tp.Optional[str] = "dense"
    ff: int = 0
    a: tp.Optional[MixerConfig] = None
    b: tp.Optional[MixerConfig] = None
    experts: int = 0
    top: int = 0
    expert_limit: float = 0.0
    router_scale: float = 1.0
    a_scale: float = 1.0                # a parallel pair whose results are summed with constant factors
    b_scale: float = 1.0

    @staticmethod
    def from_dict(d: dict) -> "DecoderLayerConfig":
        kind = d["type"]
        if kind not in MIXERS:
            raise ValueError(f"unknown mixer type {kind!r} (known: {sorted(MIXERS)})")
        m = d["mixer"]
        mlp = d.get("mlp")
        if mlp is not None and mlp.get("kind") not in MLP_KINDS:
            raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        mlp_kind = None if mlp is None else mlp["kind"]
        if mlp_kind == "moe":
            ff, experts, top = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        else:
            ff, experts, top = (0 if mlp is None else int(mlp["ff"])), 0, 0
        if kind == "latent_attention":
            return DecoderLayerConfig(type=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]),
                                      scale=float(m["scale"]), mlp_kind=mlp_kind, ff=ff)
        if kind == "parallel":
            r = m["right"]
            a = _window_attention_from_dict(m["left"])
            b = MixerConfig(kind="gla", heads=int(r["heads"]), dim=int(r["dim"]), vdim=int(r["vdim"]), tau=float(r["tau"]),
                            decay_rank=int(r.get("decay_rank", 16)))
        elif kind == "mlstm":
            a, b = MixerConfig(kind="mlstm", heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), gate_cap=float(m["gate_cap"])), None
        else:
            raise ValueError(f"mixer {kind!r} stands only inside a parallel pair")
        return DecoderLayerConfig(type=kind, mlp_kind=mlp_kind, ff=ff, a=a, b=b, experts=experts, top=top)

    def to_dict(self) -> dict:
        if self.mlp_kind is None:
            mlp = None
        elif self.mlp_kind == "moe":
            mlp = {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        else:
            mlp = {"kind": self.mlp_kind, "ff": self.ff}
        if self.type == "parallel":
            mixer = {"left": _window_attention_to_dict(self.a),
                     "right": {"dim": self.b.dim, "heads": self.b.heads, "tau": self.b.tau, "vdim": self.b.vdim}}
        elif self.type == "mlstm":
            mixer = {"dim": self.a.dim, "gate_cap": self.a.gate_cap, "heads": self.a.heads, "vdim": self.a.vdim}
        else:
            mixer = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale}
        return {"type": self.type, "mixer": mixer, "mlp": mlp}

    def mixers(self) -> tuple:
        """(a, b) as ``MixerConfig`` whatever the kind (a latent attention's flat fields are wrapped)."""
        if self.type == "latent_attention" and self.a is None:
            return MixerConfig(kind=self.type, heads=self.heads, dim=self.dim, vdim=self.vdim, kv_rank=self.kv_rank, scale=self.scale), None
        return self.a, self.b


@dataclass
class DecoderLMConfig:
    """``config.json`` of a layer-list decoder LM.  ``architecture`` selects the block arrangement; "Likosun" is a parallel block
    (one layer norm feeds mixer and feed-forward), sigmoid-gated sublayer results, a residual multiplier, and a depth-weighted
    average of all earlier layer results in front of every layer."""
    architecture: str
    vocab: int
    width: int
    layers: tp.List[DecoderLayerConfig]
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    norm_eps: float = 1e-6
    block: str = "gated_depth_average"
    canon_taps: int = 0
    logit_softcap: float = 0.0
    streams: int = 0                    # pre_norm_streams: residual streams with learned read / write weights (0: one plain residual)
    logit_scale: float = 1.0
    tied_head: bool = False             # the logits come from the embedding table

    @staticmethod
    def from_dict(d: dict) -> "DecoderLMConfig":
        arch = d.get("architecture")
        if arch not in DECODER_ARCHITECTURES:
            raise ValueError(f"unknown architecture {arch!r} (known: {sorted(DECODER_ARCHITECTURES)})")
        if DECODER_ARCHITECTURES[arch] is not DecoderLMConfig:
            return DECODER_ARCHITECTURES[arch].from_dict(d)
        return DecoderLMConfig(architecture=arch, vocab=int(d["vocab"]), width=int(d["width"]),
                               layers=[DecoderLayerConfig.from_dict(x) for x in d["layers"]],
                               embedding_scale=float(d["embedding"]["scale"]), residual_mult=float(d["residual_mult"]),
                               norm_eps=float(d["norm"]["eps"]))

    @staticmethod
    def from_json(path: str) -> "DecoderLMConfig":
        with open(path) as f:
            return DecoderLMConfig.from_dict(json.load(f))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                "layers": [x.to_dict() for x in self.layers], "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}

    def tensor_shapes(self) -> dict:
        """Checkpoint names -> shapes (linear weights are [out, in])."""
        W = self.width
        out = {"embed": (self.vocab, W)}
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            out.update({p + "norm1": (W,), p + "norm1.b": (W,), p + "mix.q": (L.heads * L.dim, W), p + "mix.dkv": (L.kv_rank, W),
                        p + "mix.dkv.norm": (L.kv_rank,), p + "mix.uk": (L.heads * L.dim, L.kv_rank),
                        p + "mix.uv": (L.heads * L.vdim, L.kv_rank), p + "mix.sink": (L.heads,), p + "mix.o": (W, L.heads * L.vdim),
                        p + "rg1": (W, W), p + "rg1.b": (W,), p + "dwa": (i + 2,)})
            if L.mlp_kind is not None:
                out.update({p + "mlp.up": (L.ff, W), p + "mlp.down": (W, L.ff), p + "rg2": (W, W), p + "rg2.b": (W,)})
        out.update({"final.norm": (W,), "final.norm.b": (W,), "head": (self.vocab, W)})
        return out


@dataclass
class GovuvikConfig(DecoderLMConfig):
    """``config.json`` of the Govuvik design: RMS norms before and after every sublayer (mixer, then a routed mixture of
    experts), an RMS-normed embedding, a causal convolution (``canon.taps``) on what every mixer reads, capped logits.  Layers
    are ``mlstm`` (a gated matrix memory) or ``parallel`` (sliding-window attention beside gated linear attention)."""

    @staticmethod
    def from_dict(d: dict) -> "GovuvikConfig":
        layers = [DecoderLayerConfig.from_dict(x) for x in d["layers"]]
        for i, L in enumerate(layers):
            if L.type not in ("parallel", "mlstm") or L.mlp_kind not in (None, "moe"):
                raise ValueError(f"layer {i}: a Govuvik layer is 'parallel' or 'mlstm' with a 'moe' feed-forward or none")
        return GovuvikConfig(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]), layers=layers,
                             norm_eps=float(d["norm"]["eps"]), block="sandwich", canon_taps=int((d.get("canon") or {}).get("taps", 0)),
                             logit_softcap=float(d.get("logit_softcap", 0.0)))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "canon": {"taps": self.canon_taps}, "layers": [x.to_dict() for x in self.layers],
                "logit_softcap": self.logit_softcap, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def tensor_shapes(self) -> dict:
        W = self.width
        out = {"embed": (self.vocab, W), "embed.norm": (W,)}
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            out.update({p + "norm1": (W,), p + "norm1b": (W,)})
            if self.canon_taps > 0:
                out[p + "canon1"] = (W, self.canon_taps)
            if L.type == "parallel":
                a, b, l, r = L.a, L.b, p + "mix.left.", p + "mix.right."
                nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
                out.update({l + "q": (nq, W), l + "k": (nk, W), l + "v": (nv, W), l + "q.norm": (nq,), l + "k.norm": (nk,)})
                if a.conv >= 1:
                    out.update({l + "q.conv": (nq, a.conv), l + "k.conv": (nk, a.conv), l + "v.conv": (nv, a.conv)})
                out.update({l + "talk": (a.heads, a.heads), l + "temp": (a.heads,), l + "sink": (a.heads,), l + "o": (W, a.heads * a.vdim),
                            r + "q": (b.heads * b.dim, W), r + "k": (b.heads * b.dim, W), r + "v": (b.heads * b.vdim, W),
                            r + "g": (b.heads * b.vdim, W), r + "o": (W, b.heads * b.vdim), r + "norm": (b.vdim,),
                            r + "a1": (b.decay_rank, W), r + "a2": (b.heads * b.dim, b.decay_rank), r + "a2.b": (b.heads * b.dim,),
                            l + "out": (W,), r + "out": (W,)})
            else:
                a, m = L.a, p + "mix."
                out.update({m + "q": (a.heads * a.dim, W), m + "k": (a.heads * a.dim, W), m + "v": (a.heads * a.vdim, W),
                            m + "g": (a.heads * a.vdim, W), m + "o": (W, a.heads * a.vdim), m + "norm": (a.heads * a.vdim,),
                            m + "i": (a.heads, W), m + "i.b": (a.heads,), m + "f": (a.heads, W), m + "f.b": (a.heads,)})
            if L.mlp_kind == "moe":
                out.update({p + "norm2": (W,), p + "norm2b": (W,), p + "mlp.router": (L.experts, W)})
                for e in range(L.experts):
                    out.update({p + f"mlp.e{e}.up": (L.ff, W), p + f"mlp.e{e}.down": (W, L.ff)})
        out.update({"final.norm": (W,), "head": (self.vocab, W)})
        return out


def _rot_fields(m: dict, pairing: str) -> dict:
    rot = m.get("rot") or {}
    sc = rot.get("scaling")
    return dict(rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)), rot_scaling=dict(sc) if sc else None,
                rot_scaling_kind="ramp" if sc else None, rot_pairing=pairing)


def _rot_to_dict(m: MixerConfig) -> tp.Optional[dict]:
    if m.rot_dims <= 0:
        return None
    rot: dict = {"base": m.rot_base, "dims": m.rot_dims}
    if m.rot_scaling:
        rot["scaling"] = dict(m.rot_scaling)
    return rot


@dataclass
class NamalixConfig(DecoderLMConfig):
    """``config.json`` of the Namalix design: parallel blocks (one zero-centred RMS norm feeds mixer and feed-forward,
    ``x += mixer(h) + ff(h)``), a scaled embedding, layers of type ``attention`` (sigmoid weights mixed over heads, optional
    blending of values with the first such layer's, a gate per head), ``retention`` (fixed decay per head) or ``delta`` (gated
    delta rule behind short convolutions), each with a ``dense`` (gated tanh-GELU) or ``moe`` (sigmoid router with a choice
    correction, clamped gated experts) feed-forward or none."""

    TYPES = {"attention": "sigmoid_attention", "retention": "retention", "delta": "delta"}
    FF = {"dense": "gated_gelu", "moe": "moe_clamped_glu"}

    @staticmethod
    def _layer(i: int, d: dict) -> DecoderLayerConfig:
        t, m, mlp = d["type"], d["mixer"], d.get("mlp")
        if t not in NamalixConfig.TYPES:
            raise ValueError(f"layer {i}: a Namalix layer is one of {sorted(NamalixConfig.TYPES)}, not {t!r}")
        kind = NamalixConfig.TYPES[t]
        if t == "attention":
            a = MixerConfig(kind=kind, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                            scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0), v_mix=bool(m.get("v_mix", False)),
                            **_rot_fields(m, "adjacent"))
        elif t == "retention":
            a = MixerConfig(kind=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), decay=[float(x) for x in m["decay"]],
                            **_rot_fields(m, "halves"))
            if len(a.decay) != a.heads:
                raise ValueError(f"layer {i}: retention wants one decay per head")
        else:
            a = MixerConfig(kind=kind, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                            conv=int(m["conv"]))
        if mlp is None:
            return DecoderLayerConfig(type=kind, mlp_kind=None, a=a)
        if mlp["kind"] not in NamalixConfig.FF:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
        if mlp["kind"] == "dense":
            return DecoderLayerConfig(type=kind, mlp_kind="gated_gelu", ff=int(mlp["ff"]), a=a)
        r, e = mlp["router"], mlp["expert"]
        return DecoderLayerConfig(type=kind, mlp_kind="moe_clamped_glu", ff=int(e["ff"]), a=a, experts=int(r["experts"]), top=int(r["top"]),
                                  expert_limit=float(e["limit"]), router_scale=float(r.get("scale", 1.0)))

    @staticmethod
    def from_dict(d: dict) -> "NamalixConfig":
        return NamalixConfig(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]),
                             layers=[NamalixConfig._layer(i, x) for i, x in enumerate(d["layers"])],
                             embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), norm_eps=float(d["norm"]["eps"]),
                             block="parallel_residual")

    @staticmethod
    def _layer_to_dict(L: DecoderLayerConfig) -> dict:
        a = L.a
        if a.kind == "sigmoid_attention":
            mixer: dict = {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "scale": a.scale, "softcap": a.softcap, "v_mix": a.v_mix, "vdim": a.vdim}
            t = "attention"
        elif a.kind == "retention":
            mixer, t = {"decay": list(a.decay), "dim": a.dim, "heads": a.heads, "vdim": a.vdim}, "retention"
        else:
            mixer, t = {"conv": a.conv, "dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "vdim": a.vdim}, "delta"
        rot = _rot_to_dict(a)
        if rot is not None:
            mixer["rot"] = rot
        if L.mlp_kind is None:
            mlp = None
        elif L.mlp_kind == "gated_gelu":
            mlp = {"ff": L.ff, "kind": "dense"}
        else:
            mlp = {"expert": {"ff": L.ff, "limit": L.expert_limit}, "kind": "moe",
                   "router": {"experts": L.experts, "scale": L.router_scale, "top": L.top}}
        return {"mixer": mixer, "mlp": mlp, "type": t}

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                "layers": [self._layer_to_dict(x) for x in self.layers], "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def first_v_mix_layer(self) -> int:
        """Index of the first attention layer that blends values (its own values are the ones the later layers blend in); -1: none."""
        for i, L in enumerate(self.layers):
            if L.a.kind == "sigmoid_attention" and L.a.v_mix:
                return i
        return -1

    def tensor_shapes(self) -> dict:
        W = self.width
        out = {"embed": (self.vocab, W)}
        for i, L in enumerate(self.layers):
            p, m, a = f"l{i}.", f"l{i}.mix.", L.a
            out[p + "norm1"] = (W,)
            if a.kind == "sigmoid_attention":
                out.update({m + "q": (a.heads * a.dim, W), m + "k": (a.kv_heads * a.dim, W), m + "v": (a.kv_heads * a.vdim, W)})
                if a.v_mix:
                    out[m + "vmix"] = ()
                out.update({m + "talk": (a.heads, a.heads), m + "pb": (a.heads,), m + "g": (a.heads, W), m + "o": (W, a.heads * a.vdim)})
            elif a.kind == "retention":
                out.update({m + "q": (a.heads * a.dim, W), m + "k": (a.heads * a.dim, W), m + "v": (a.heads * a.vdim, W),
                            m + "g": (a.heads * a.vdim, W), m + "o": (W, a.heads * a.vdim)})
            else:
                nq, nv = a.kv_heads * a.dim, a.heads * a.vdim
                out.update({m + "q": (nq, W), m + "q.conv": (nq, a.conv), m + "k": (nq, W), m + "k.conv": (nq, a.conv), m + "v": (nv, W),
                            m + "v.conv": (nv, a.conv), m + "b": (a.heads, W), m + "A_log": (a.heads,), m + "norm": (a.vdim,),
                            m + "a": (a.heads, W), m + "dt_bias": (a.heads,), m + "g": (nv, W), m + "o": (W, nv)})
            if L.mlp_kind == "gated_gelu":
                out.update({p + "mlp.gate": (L.ff, W), p + "mlp.up": (L.ff, W), p + "mlp.down": (W, L.ff)})
            elif L.mlp_kind == "moe_clamped_glu":
                for e in range(L.experts):
                    out.update({p + f"mlp.e{e}.gate": (L.ff, W), p + f"mlp.e{e}.up": (L.ff, W), p + f"mlp.e{e}.down": (W, L.ff)})
                out.update({p + "mlp.router": (L.experts, W), p + "mlp.correction": (L.experts,)})
        out.update({"final.norm": (W,), "head": (self.vocab, W)})
        return out


@dataclass
class DibulixConfig(DecoderLMConfig):
    """``config.json`` of the Dibulix design: pre-norm sublayers (mixer, then a dense squared-ReLU feed-forward or none) on
    ``streams`` residual streams that every sublayer reads as a weighted sum and rewrites through a small mixing matrix; layers of
    type ``latent_attention`` (a cached latent plus one rotated key part shared by the heads, rotation by halves with the index
    ramp, a sliding window, a sigmoid gate per head), ``parallel`` (sliding-window attention with biased projections, rotation of
    adjacent pairs and one extra unit in the softmax denominator, beside a minGRU; summed with constant factors) and
    ``channel_delta`` (gated delta rule with a decay per key channel); logits from the embedding table times ``logit_scale``."""

    TYPES = ("latent_attention", "parallel", "channel_delta")

    @staticmethod
    def _layer(i: int, d: dict) -> DecoderLayerConfig:
        t, m, mlp = d["type"], d["mixer"], d.get("mlp")
        if t not in DibulixConfig.TYPES:
            raise ValueError(f"layer {i}: a Dibulix layer is one of {sorted(DibulixConfig.TYPES)}, not {t!r}")
        if mlp is not None and mlp.get("kind") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        kw: dict = dict(type=t, mlp_kind=None if mlp is None else "dense", ff=0 if mlp is None else int(mlp["ff"]))
        if t == "latent_attention":
            rot = dict(m.get("rot") or {})
            rd = int(m.get("rot_dim", 0))
            if rd and int(rot.get("dims", rd)) != rd:
                raise ValueError(f"layer {i}: the rotation covers the rotated part (rot.dims = rot_dim)")
            rot["dims"] = rd
            a = MixerConfig(kind=t, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                            window=int((m.get("mask") or {}).get("size", 0)), sink="none", head_gate=True, **_rot_fields({"rot": rot}, "halves"))
            return DecoderLayerConfig(a=a, **kw)
        if t == "parallel":
            l, r = m["left"], m["right"]
            a = MixerConfig(kind="window_attention", heads=int(l["heads"]), kv_heads=int(l["kv_heads"]), dim=int(l["dim"]), vdim=int(l["vdim"]),
                            scale=float(l["scale"]), window=int((l.get("mask") or {}).get("size", 0)) or NO_WINDOW, bias=True, sink="unit",
                            **_rot_fields(l, "adjacent"))
            b = MixerConfig(kind="mingru", heads=1, dim=int(r["width"]), vdim=int(r["width"]), bias=True)
            return DecoderLayerConfig(a=a, b=b, a_scale=float(m.get("left_scale", 1.0)), b_scale=float(m.get("right_scale", 1.0)), **kw)
        a = MixerConfig(kind=t, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), conv=int(m["conv"]),
                        decay_rank=int(m.get("decay_rank", 16)), gate_rank=int(m.get("gate_rank", 16)))
        return DecoderLayerConfig(a=a, **kw)

    @staticmethod
    def from_dict(d: dict) -> "DibulixConfig":
        return DibulixConfig(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]),
                             layers=[DibulixConfig._layer(i, x) for i, x in enumerate(d["layers"])], norm_eps=float(d["norm"]["eps"]),
                             block="pre_norm_streams", streams=int(d.get("streams", 0)), logit_scale=float(d.get("logit_scale", 1.0)), tied_head=True)

    @staticmethod
    def _layer_to_dict(L: DecoderLayerConfig) -> dict:
        a = L.a
        if L.type == "latent_attention":
            mixer: dict = {"dim": a.dim, "heads": a.heads, "kv_rank": a.kv_rank, "rot_dim": a.rot_dims, "scale": a.scale, "vdim": a.vdim}
            rot = _rot_to_dict(a)
            if rot is not None:
                mixer["rot"] = rot
            if a.window:
                mixer["mask"] = {"size": a.window}
        elif L.type == "parallel":
            left: dict = {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "scale": a.scale, "vdim": a.vdim}
            rot = _rot_to_dict(a)
            if rot is not None:
                left["rot"] = rot
            if a.window and a.window < NO_WINDOW:
                left["mask"] = {"size": a.window}
            mixer = {"left": left, "left_scale": L.a_scale, "right": {"width": L.b.dim}, "right_scale": L.b_scale}
        else:
            mixer = {"conv": a.conv, "dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "vdim": a.vdim}
        return {"mixer": mixer, "mlp": None if L.mlp_kind is None else {"ff": L.ff, "kind": "dense"}, "type": L.type}

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "layers": [self._layer_to_dict(x) for x in self.layers], "logit_scale": self.logit_scale,
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.streams:
            d["streams"] = self.streams
        return d

    def tensor_shapes(self) -> dict:
        W, s = self.width, self.streams
        out = {"embed": (self.vocab, W)}
        for i, L in enumerate(self.layers):
            p, m, a = f"l{i}.", f"l{i}.mix.", L.a
            out[p + "norm1"] = (W,)
            if L.mlp_kind is not None:
                out[p + "norm2"] = (W,)
            if L.type == "latent_attention":
                out.update({m + "q": (a.heads * (a.dim + a.rot_dims), W), m + "dkv": (a.kv_rank + a.rot_dims, W), m + "dkv.norm": (a.kv_rank,),
                            m + "uk": (a.heads * a.dim, a.kv_rank), m + "uv": (a.heads * a.vdim, a.kv_rank), m + "g": (a.heads, W),
                            m + "o": (W, a.heads * a.vdim)})
            elif L.type == "parallel":
                l, r, n = m + "left.", m + "right.", L.b.dim
                for nm, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
                    out.update({l + nm: (rows, W), l + nm + ".b": (rows,)})
                out.update({l + "o": (W, a.heads * a.vdim), r + "z": (n, W), r + "z.b": (n,), r + "x": (n, W), r + "x.b": (n,), r + "g": (n, W),
                            r + "o": (W, n)})
            else:
                nq, nv, nd = a.kv_heads * a.dim, a.heads * a.vdim, a.heads * a.dim
                out.update({m + "q": (nq, W), m + "q.conv": (nq, a.conv), m + "k": (nq, W), m + "k.conv": (nq, a.conv), m + "v": (nv, W),
                            m + "v.conv": (nv, a.conv), m + "b": (a.heads, W), m + "A_log": (a.heads,), m + "norm": (a.vdim,),
                            m + "a1": (a.decay_rank, W), m + "a2": (nd, a.decay_rank), m + "dt_bias": (nd,), m + "g1": (a.gate_rank, W),
                            m + "g2": (nv, a.gate_rank), m + "o": (W, nv)})
            if L.mlp_kind is not None:
                out.update({p + "mlp.up": (L.ff, W), p + "mlp.down": (W, L.ff)})
            for q in (1, 2) if L.mlp_kind is not None else (1,):
                if s:
                    out.update({p + f"hc{q}.in": (s,), p + f"hc{q}.out": (s,), p + f"hc{q}.mix": (s, s)})
        out["final.norm"] = (W,)
        return out


# architecture name in config.json -> configuration class (the model registry of the text-only decoder LMs)
DECODER_ARCHITECTURES: dict = {"Likosun": DecoderLMConfig, "Govuvik": GovuvikConfig, "Namalix": NamalixConfig, "Dibulix": DibulixConfig}
