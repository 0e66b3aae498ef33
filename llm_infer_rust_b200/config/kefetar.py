"""Typed configuration of Kefetar, read from its own config.json keys.

    architecture   "Kefetar"
    vocab, width   sizes of the embedding table and of the residual stream
    norm.eps       eps of every RMS norm of the model (inside the root)
    canon.taps     taps of the causal convolution through which every sublayer reads its normed input
                   (absent: no such convolution; 1: a gain per channel)
    layers[i]      type ("attention" | "retention"), mixer (sizes and constants, below), mlp (null, or
                   {"kind": "dense", "ff": F})

    attention mixer: heads, kv_heads, dim (query / key size), vdim (value size), scale, and optionally conv
                   (taps of the convolution on q, k, v), rot {base, dims, scaling {factor}}, softcap, v_mix
    retention mixer: heads, dim, vdim, decay (one number per head), optionally rot {base, dims, scaling {factor}}

Nothing here is a default for a size: a key that the design needs and the file lacks is an error.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

# The design names no longest sequence; rotation angles are formed from the position itself.  Positions stay
# exact as floats up to 2^24; the engine's own --max-seq-len bounds a request.
MAX_POSITIONS = 1 << 20


def _int(raw: dict, key: str, where: str, minimum: int = 1) -> int:
    if key not in raw:
        raise ConfigError(f"missing {where}{key}")
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int) or value < minimum:
        raise ConfigError(f"invalid {where}{key}: {value!r} (an integer >= {minimum} is required)")
    return value


def _number(raw: dict, key: str, where: str, positive: bool = True) -> float:
    if key not in raw:
        raise ConfigError(f"missing {where}{key}")
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)) \
            or (positive and float(value) <= 0.0):
        raise ConfigError(f"invalid {where}{key}: {value!r} (a{' positive' if positive else ''} number is required)")
    return float(value)


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    factor: float          # linear scaling: every frequency is divided by it (1: none)


@dataclass(frozen=True)
class KefetarLayer:
    kind: str                              # "attention" | "retention"
    heads: int
    dim: int
    vdim: int
    rot: Optional[Rotation]
    ff: Optional[int]                      # None: no feed-forward sublayer
    # attention
    kv_heads: int = 0
    conv: int = 0                          # taps of the q/k/v convolution, 0: none
    scale: float = 1.0
    softcap: Optional[float] = None
    v_mix: bool = False
    # retention
    decay: Tuple[float, ...] = ()


@dataclass(frozen=True)
class KefetarConfig:
    vocab: int
    width: int
    eps: float
    canon_taps: int                        # 0: sublayers read the normed input itself
    layers: Tuple[KefetarLayer, ...]

    architecture = "Kefetar"
    model_type = None

    @staticmethod
    def _rotation(m: dict, where: str, dim: int) -> Optional[Rotation]:
        rot = m.get("rot")
        if rot is None:
            return None
        if not isinstance(rot, dict):
            raise ConfigError(f"invalid {where}rot: an object is required")
        dims = _int(rot, "dims", where + "rot.", 2)
        if dims % 2 or dims > dim:
            raise ConfigError(f"invalid {where}rot.dims: {dims} (even and at most the head's {dim})")
        scaling = rot.get("scaling")
        factor = 1.0
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"invalid {where}rot.scaling: an object is required")
            factor = _number(scaling, "factor", where + "rot.scaling.")
        return Rotation(_number(rot, "base", where + "rot."), dims, factor)

    @staticmethod
    def parse(raw: Any) -> "KefetarConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config must be an object")
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("missing norm (an object with eps)")
        eps = _number(norm, "eps", "norm.")
        canon = raw.get("canon")
        canon_taps = 0
        if canon is not None:
            if not isinstance(canon, dict):
                raise ConfigError("invalid canon: an object is required")
            canon_taps = _int(canon, "taps", "canon.")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{where}mixer must be an object")
            m = entry["mixer"]
            kind = entry.get("type")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"unsupported {where}mlp.kind: {mlp.get('kind') if isinstance(mlp, dict) else mlp!r}")
                ff = _int(mlp, "ff", where + "mlp.")
            heads, dim, vdim = (_int(m, "heads", where + "mixer."), _int(m, "dim", where + "mixer."),
                                _int(m, "vdim", where + "mixer."))
            rot = KefetarConfig._rotation(m, where + "mixer.", dim)
            if kind == "attention":
                kv_heads = _int(m, "kv_heads", where + "mixer.")
                if heads % kv_heads:
                    raise ConfigError(f"{where}mixer.heads must be a multiple of kv_heads")
                if dim % 2 or vdim % 2 or dim > 512 or vdim > 512:
                    raise ConfigError(f"{where}mixer: dim and vdim must be even and at most 512")
                layers.append(KefetarLayer(
                    "attention", heads, dim, vdim, rot, ff, kv_heads=kv_heads,
                    conv=_int(m, "conv", where + "mixer.") if m.get("conv") is not None else 0,
                    scale=_number(m, "scale", where + "mixer."),
                    softcap=_number(m, "softcap", where + "mixer.") if m.get("softcap") is not None else None,
                    v_mix=bool(m.get("v_mix", False))))
            elif kind == "retention":
                decay = m.get("decay")
                if not isinstance(decay, list) or len(decay) != heads or any(
                        isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
                    raise ConfigError(f"{where}mixer.decay must list one number per head")
                if dim > 512:
                    raise ConfigError(f"{where}mixer.dim must be at most 512")
                layers.append(KefetarLayer("retention", heads, dim, vdim, rot, ff, decay=tuple(float(g) for g in decay)))
            else:
                raise ConfigError(f"unsupported {where}type: {kind!r} (attention and retention are known)")
        mixing = [l for l in layers if l.v_mix]
        if any(l.kv_heads * l.vdim != mixing[0].kv_heads * mixing[0].vdim for l in mixing):
            raise ConfigError("layers that mix their values (v_mix) must agree in kv_heads * vdim")
        if canon_taps > 8 or any(l.conv > 8 for l in layers):
            raise ConfigError("a convolution of more than 8 taps is refused")
        return KefetarConfig(vocab, width, eps, canon_taps, tuple(layers))

    # ------------------------------------------------------------------ parts
    def model_spec(self) -> ModelSpec:
        norm = PartSpec("scalar_rms_norm", {"eps": self.eps})
        encodings: Dict[str, PartSpec] = {}
        names: Dict[Rotation, str] = {}

        def encoding(rot: Optional[Rotation]) -> Optional[str]:
            if rot is None:
                return None
            if rot not in names:
                names[rot] = f"rot{len(names)}"
                encodings[names[rot]] = PartSpec("rotary_frequencies", {
                    "rotary_dim": rot.dims, "theta": rot.base, "scaling_factor": rot.factor})
            return names[rot]

        canon = PartSpec("causal_taps", {"channels": self.width, "taps": max(self.canon_taps, 1), "identity": True})
        layers = []
        seen_v_mix = False
        for l in self.layers:
            if l.kind == "attention":
                role = None
                if l.v_mix:
                    role, seen_v_mix = ("mix" if seen_v_mix else "source"), True
                mixer = PartSpec("gated_conv_attention", {
                    "hidden_size": self.width, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "head_dim": l.dim,
                    "v_head_dim": l.vdim, "conv_taps": l.conv, "softmax_scale": l.scale, "softcap": l.softcap,
                    "window": None, "gate": True, "v_mix": role, "v_mix_group": "first",
                    "position_encoding": encoding(l.rot)})
            else:
                mixer = PartSpec("decay_retention", {
                    "hidden_size": self.width, "num_heads": l.heads, "head_dim": l.dim, "v_head_dim": l.vdim,
                    "decay": l.decay, "eps": self.eps, "k_scale": l.dim ** -0.5,
                    "position_encoding": encoding(l.rot)})
            parts = {"input_norm": norm, "mixer": mixer}
            if self.canon_taps >= 1:
                parts["mixer_conv"] = canon
            if l.ff is not None:
                parts["post_mixer_norm"] = norm
                parts["feed_forward"] = PartSpec("poly_norm", {"hidden_size": self.width, "intermediate_size": l.ff,
                                                               "eps": self.eps})
                if self.canon_taps >= 1:
                    parts["ff_conv"] = canon
            layers.append(LayerSpec(PartSpec("pre_norm_input_conv"), parts))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "out_dtype": "float32"}),
            layers=tuple(layers), run_list=tuple(RunEntry(i) for i in range(len(layers))),
            final_norm=norm,
            lm_head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False}),
            position_encodings=encodings)
        spec.validate()
        return spec
