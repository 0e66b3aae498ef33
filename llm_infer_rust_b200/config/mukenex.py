"""Typed configuration of Mukenex, read from its own config.json keys.

    architecture    "Mukenex"
    vocab, width    sizes of the embedding table and of the residual
    norm.eps        eps of every RMS norm of the model (inside the root)
    streams         copies of the residual that the layers read and write through learned coefficients
                    (absent: one copy and the ordinary residual sum)
    loop            {start, stop, times}: layers start .. stop-1 run ``times`` times in a row with the same weights,
                    every pass with a cache and state of its own (absent: every layer once)
    logit_softcap   c: logits <- c tanh(logits / c) (absent: none)
    layers[i]       type ("latent_attention" | "attention" | "lightning"), mixer (sizes and constants, below),
                    mlp: null, {"kind": "dense", "ff": F} or {"kind": "moe", "expert": {"ff": F},
                    "router": {"experts": E, "top": K}}

    latent_attention  heads, dim (unrotated query/key size), rot_dim (rotated size), vdim, kv_rank, scale,
                      rot {base, dims}, mask {size} (a sliding window)
    attention         heads, kv_heads, dim, vdim, scale, mask {size} (blocks of that many positions)
    lightning         heads, dim, vdim, decay (one number per head)

Nothing here is a default for a size: a key that the design needs and the file lacks is an error.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .kefetar import MAX_POSITIONS, _int, _number
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

MAX_STREAMS = 8


@dataclass(frozen=True)
class MukenexFF:
    kind: str                  # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class MukenexLayer:
    kind: str                  # "latent_attention" | "attention" | "lightning"
    heads: int
    dim: int
    vdim: int
    ff: Optional[MukenexFF]
    scale: float = 1.0
    mask: int = 0              # latent_attention: the window; attention: the block of positions
    kv_heads: int = 0          # attention
    rot_dim: int = 0           # latent_attention
    kv_rank: int = 0
    rot_base: float = 0.0
    rot_dims: int = 0
    decay: Tuple[float, ...] = ()      # lightning


@dataclass(frozen=True)
class MukenexConfig:
    vocab: int
    width: int
    eps: float
    streams: Optional[int]             # None: the ordinary residual sum
    softcap: Optional[float]
    layers: Tuple[MukenexLayer, ...]
    run: Tuple[int, ...]               # the order in which layers run

    architecture = "Mukenex"
    model_type = None

    @staticmethod
    def _feed_forward(mlp: Any, where: str) -> Optional[MukenexFF]:
        if mlp is None:
            return None
        if not isinstance(mlp, dict):
            raise ConfigError(f"invalid {where}mlp: an object or null is required")
        kind = mlp.get("kind")
        if kind == "dense":
            return MukenexFF("dense", _int(mlp, "ff", where + "mlp."))
        if kind == "moe":
            expert, router = mlp.get("expert"), mlp.get("router")
            if not isinstance(expert, dict) or not isinstance(router, dict):
                raise ConfigError(f"{where}mlp needs expert and router objects")
            experts, top = _int(router, "experts", where + "mlp.router."), _int(router, "top", where + "mlp.router.")
            if top > experts:
                raise ConfigError(f"{where}mlp.router.top must be at most experts")
            return MukenexFF("moe", _int(expert, "ff", where + "mlp.expert."), experts, top)
        raise ConfigError(f"unsupported {where}mlp.kind: {kind!r} (dense and moe are known)")

    @staticmethod
    def _mask(m: dict, where: str) -> int:
        mask = m.get("mask")
        if not isinstance(mask, dict):
            raise ConfigError(f"missing {where}mask (an object with size)")
        return _int(mask, "size", where + "mask.")

    @staticmethod
    def parse(raw: Any) -> "MukenexConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config must be an object")
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("missing norm (an object with eps)")
        eps = _number(norm, "eps", "norm.")
        streams = None
        if raw.get("streams") is not None:
            streams = _int(raw, "streams", "")
            if streams > MAX_STREAMS:
                raise ConfigError(f"streams: {streams} is refused (at most {MAX_STREAMS})")
        softcap = _number(raw, "logit_softcap", "") if raw.get("logit_softcap") is not None else None
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{where}mixer must be an object")
            m, kind = entry["mixer"], entry.get("type")
            w = where + "mixer."
            ff = MukenexConfig._feed_forward(entry.get("mlp"), where)
            heads, dim, vdim = _int(m, "heads", w), _int(m, "dim", w), _int(m, "vdim", w)
            if kind == "latent_attention":
                rot_dim, kv_rank = _int(m, "rot_dim", w), _int(m, "kv_rank", w)
                rot = m.get("rot")
                if not isinstance(rot, dict):
                    raise ConfigError(f"missing {w}rot (an object with base and dims)")
                dims = _int(rot, "dims", w + "rot.", 2)
                if dims % 2 or dims > rot_dim:
                    raise ConfigError(f"invalid {w}rot.dims: {dims} (even and at most rot_dim = {rot_dim})")
                if kv_rank % 2 or rot_dim % 2 or kv_rank + rot_dim > 512:
                    raise ConfigError(f"{w}kv_rank and rot_dim must be even and together at most 512")
                layers.append(MukenexLayer("latent_attention", heads, dim, vdim, ff, scale=_number(m, "scale", w),
                                           mask=MukenexConfig._mask(m, w), rot_dim=rot_dim, kv_rank=kv_rank,
                                           rot_base=_number(rot, "base", w + "rot."), rot_dims=dims))
            elif kind == "attention":
                kv_heads = _int(m, "kv_heads", w)
                if heads % kv_heads:
                    raise ConfigError(f"{w}heads must be a multiple of kv_heads")
                if dim % 2 or vdim % 2 or dim > 512 or vdim > 512:
                    raise ConfigError(f"{w}dim and vdim must be even and at most 512")
                layers.append(MukenexLayer("attention", heads, dim, vdim, ff, scale=_number(m, "scale", w),
                                           mask=MukenexConfig._mask(m, w), kv_heads=kv_heads))
            elif kind == "lightning":
                decay = m.get("decay")
                if not isinstance(decay, list) or len(decay) != heads or any(
                        isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
                    raise ConfigError(f"{w}decay must list one number per head")
                if dim > 512:
                    raise ConfigError(f"{w}dim must be at most 512")
                layers.append(MukenexLayer("lightning", heads, dim, vdim, ff, decay=tuple(float(g) for g in decay)))
            else:
                raise ConfigError(f"unsupported {where}type: {kind!r} "
                                  f"(latent_attention, attention and lightning are known)")
        n = len(layers)
        run = list(range(n))
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("invalid loop: an object is required")
            start, stop = _int(loop, "start", "loop.", 0), _int(loop, "stop", "loop.", 0)
            times = _int(loop, "times", "loop.", 1)
            if not 0 <= start <= stop <= n:
                raise ConfigError(f"loop: 0 <= start <= stop <= {n} is required")
            run = list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))
        return MukenexConfig(vocab, width, eps, streams, softcap, tuple(layers), tuple(run))

    # ------------------------------------------------------------------ parts
    def model_spec(self) -> ModelSpec:
        s = self.streams or 1
        norm = PartSpec("stream_rms_norm", {"width": self.width, "eps": self.eps, "offset": 1.0, "streams": s})
        mix = PartSpec("stream_mix", {"streams": s, "fixed": self.streams is None})
        encodings: Dict[str, PartSpec] = {}
        names: Dict[tuple, str] = {}

        def encoding(base: float, dims: int) -> str:
            key = (base, dims)
            if key not in names:
                names[key] = f"rot{len(names)}"
                encodings[names[key]] = PartSpec("rotary_frequencies", {"rotary_dim": dims, "theta": base,
                                                                        "pairing": "interleaved"})
            return names[key]

        layers = []
        for l in self.layers:
            if l.kind == "latent_attention":
                mixer = PartSpec("latent_attention", {
                    "hidden_size": self.width, "num_heads": l.heads, "head_dim": l.dim, "rot_dim": l.rot_dim,
                    "v_head_dim": l.vdim, "kv_rank": l.kv_rank, "eps": self.eps, "softmax_scale": l.scale,
                    "window": l.mask, "sink": True, "gate": True, "rot_dims": l.rot_dims,
                    "position_encoding": encoding(l.rot_base, l.rot_dims)})
            elif l.kind == "attention":
                mixer = PartSpec("grouped_attention", {
                    "hidden_size": self.width, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "head_dim": l.dim,
                    "v_head_dim": l.vdim, "bias": True, "qk_norm_eps": self.eps, "softmax_scale": l.scale,
                    "chunk": l.mask})
            else:
                mixer = PartSpec("decay_retention", {
                    "hidden_size": self.width, "num_heads": l.heads, "head_dim": l.dim, "v_head_dim": l.vdim,
                    "decay": l.decay, "eps": self.eps, "k_scale": 1.0, "qkv_activation": "silu",
                    "output": "joint_norm_sigmoid"})
            parts = {"input_norm": norm, "mixer": mixer, "mixer_mix": mix}
            if l.ff is not None:
                parts["post_mixer_norm"] = norm
                parts["ff_mix"] = mix
                if l.ff.kind == "dense":
                    parts["feed_forward"] = PartSpec("dense_act", {"hidden_size": self.width,
                                                                   "intermediate_size": l.ff.ff,
                                                                   "activation": "gelu_erf"})
                else:
                    parts["feed_forward"] = PartSpec("table_experts", {
                        "hidden_size": self.width, "intermediate_size": l.ff.ff, "experts": l.ff.experts,
                        "top": l.ff.top, "vocab_size": self.vocab})
            layers.append(LayerSpec(PartSpec("multi_stream_pre_norm"), parts))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "out_dtype": "float32"}),
            layers=tuple(layers), run_list=tuple(RunEntry(i) for i in self.run),
            final_norm=norm,
            lm_head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False,
                                             "softcap": self.softcap}),
            position_encodings=encodings)
        spec.validate()
        return spec
