"""Small Mukenex configurations, random weights for them and helpers that run them through the engine.

The configurations differ from one another in every size and option: the order and the kinds of the layers, head
counts and groups, key, value, latent and rotated widths (also a rotation narrower than the rotated part), windows
and blocks, one to four residual streams or the ordinary residual, loops over a leading, a middle or no range of
layers, dense, routed (one to all experts a token) and absent feed-forwards, a logit cap or none.  Weights are
drawn with torch's generator and are representable in bfloat16, so that the float32 engine, the bfloat16 engine
and the plain implementation read the same numbers.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_mukenex as P
from kefetar_kit import bf16_values, check, make_engine, run_alone, tokens  # noqa: F401  (shared helpers)


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, window, base=10000.0, dims=None, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": dims or rot_dim}, "mask": {"size": window}}}


def attention(heads, kv_heads, dim, vdim, scale, block, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                      "mask": {"size": block}}}


def lightning(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(vocab, width, eps, layers, streams=None, loop=None, softcap=None):
    raw = {"architecture": "Mukenex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        raw["streams"] = streams
    if loop is not None:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    if softcap is not None:
        raw["logit_softcap"] = softcap
    return raw


CONFIGS = {
    # two streams, a loop over the two middle layers, two experts a token, a rotation narrower than the rotated part,
    # values narrower and wider than keys, a layer without feed-forward, odd widths
    "M1": config(101, 44, 1e-5, [
        attention(4, 2, 16, 8, 0.3, 7, mlp=moe(24, 5, 2)),
        lightning(2, 8, 16, [0.9, 0.99], mlp=dense(40)),
        latent(3, 8, 8, 12, 16, 0.25, 9, base=100.0, dims=4),
        lightning(1, 24, 8, [0.97], mlp=moe(20, 4, 1)),
    ], streams=2, loop=(1, 3, 2), softcap=12.0),
    # the ordinary residual, no loop, no cap; one KV head for six query heads; a latent narrower than a head's keys
    "M2": config(131, 40, 3e-6, [
        latent(5, 12, 4, 6, 10, 0.4, 25, base=77.0, mlp=dense(56)),
        attention(6, 1, 10, 10, 0.2, 16, mlp=dense(32)),
        lightning(3, 10, 6, [0.5, 0.95, 0.999]),
    ]),
    # four streams, a loop over the first layer alone, head sizes of the tensor-core kernels, every expert for every token
    "M3": config(211, 64, 1e-6, [
        attention(4, 2, 32, 32, 0.18, 33, mlp=moe(48, 3, 3)),
        latent(2, 16, 16, 32, 32, 0.2, 40, mlp=moe(32, 6, 2)),
        lightning(2, 32, 32, [0.96, 0.99], mlp=dense(96)),
    ], streams=4, loop=(0, 1, 3), softcap=30.0),
    # one stream that still has coefficients, a loop that runs once, heads wider than 128, forty query heads on one latent
    "M4": config(73, 56, 1e-5, [
        lightning(1, 192, 72, [0.99], mlp=dense(48)),
        latent(40, 4, 2, 4, 6, 0.5, 12, base=50.0),
        attention(2, 1, 160, 136, 0.08, 20, mlp=moe(16, 2, 1)),
    ], streams=1, loop=(1, 2, 1)),
}

# One mixer alone, with scores so sharp that a single key (or the sink) decides a position's result, and decays
# so slow that the first tokens still count hundreds of tokens later.
ONLY_LATENT = config(89, 34, 1e-5, [latent(4, 6, 6, 10, 12, 2.5, 41, base=1000.0)], streams=3)
ONLY_BLOCKS = config(89, 36, 1e-5, [attention(4, 2, 12, 14, 3.0, 48)])
ONLY_LIGHTNING = config(89, 36, 1e-5, [lightning(2, 16, 24, [0.999, 0.9995])], streams=2)


def random_weights(raw: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors by name, float32 with bfloat16-representable values (the expert table int32)."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return bf16_values(mean + std * torch.randn(tuple(shape), generator=g))

    w, width, s = {}, raw["width"], raw.get("streams")
    w["embed"] = normal(raw["vocab"], width)
    w["head"] = normal(raw["vocab"], width, std=2.0 * width ** -0.5)
    w["final.norm"] = normal(width, std=0.2)

    def stream_mix(prefix):
        if s:
            w[prefix + ".in"] = normal(s, std=0.2, mean=1.0 / s)
            w[prefix + ".out"] = normal(s, std=0.3, mean=1.0)
            w[prefix + ".mix"] = bf16_values(torch.eye(s) + 0.2 * torch.randn((s, s), generator=g))

    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = normal(width, std=0.2)
        stream_mix(p + "hc1")
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        wide = 2.0 * width ** -0.5
        if layer["type"] == "latent_attention":
            r, c = m["rot_dim"], m["kv_rank"]
            w[p + "mix.q"] = normal(H * (d + r), width, std=wide)
            w[p + "mix.dkv"] = normal(c + r, width, std=wide)
            w[p + "mix.dkv.norm"] = normal(c, std=0.2, mean=1.0)
            w[p + "mix.uk"] = normal(H * d, c, std=c ** -0.5)
            w[p + "mix.uv"] = normal(H * dv, c, std=c ** -0.5)
            w[p + "mix.sink"] = normal(H, std=1.5)
            w[p + "mix.g"] = normal(H * dv, width, std=wide)
            w[p + "mix.o"] = normal(width, H * dv, std=(H * dv) ** -0.5)
        elif layer["type"] == "attention":
            G = m["kv_heads"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[p + "mix." + name] = normal(rows, width, std=wide if name != "v" else width ** -0.5)
                w[p + "mix." + name + ".b"] = normal(rows, std=0.5)
            w[p + "mix.q.norm"] = normal(d, std=0.3, mean=1.0)
            w[p + "mix.k.norm"] = normal(d, std=0.3, mean=1.0)
            w[p + "mix.o"] = normal(width, H * dv, std=(H * dv) ** -0.5)
        else:
            for name, rows in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                w[p + "mix." + name] = normal(rows, width, std=width ** -0.5)
            w[p + "mix.norm"] = normal(H * dv, std=0.2, mean=1.0)
            w[p + "mix.o"] = normal(width, H * dv, std=(H * dv) ** -0.5)
        mlp = layer.get("mlp")
        if mlp:
            w[p + "norm2"] = normal(width, std=0.2)
            stream_mix(p + "hc2")
            if mlp["kind"] == "dense":
                w[p + "mlp.up"] = normal(mlp["ff"], width, std=width ** -0.5)
                w[p + "mlp.down"] = normal(width, mlp["ff"], std=mlp["ff"] ** -0.5)
            else:
                ff, E, top = mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["top"]
                for e in range(E):
                    w[f"{p}mlp.e{e}.gate"] = normal(ff, width, std=width ** -0.5)
                    w[f"{p}mlp.e{e}.up"] = normal(ff, width, std=width ** -0.5)
                    w[f"{p}mlp.e{e}.down"] = normal(width, ff, std=ff ** -0.5)
                rows = [torch.randperm(E, generator=g)[:top] for _ in range(raw["vocab"])]
                w[p + "mlp.table"] = torch.stack(rows).to(torch.int32)
    return w


def write_model(folder: str, raw: dict, weights: Dict[str, torch.Tensor], dtype: str = "bfloat16") -> str:
    import json
    import os
    from llm_infer_rust_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(raw, fh)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(n, t.to(store) if t.is_floating_point() else t) for n, t in weights.items()])
    return folder


def oracle(raw: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int]) -> np.ndarray:
    """The plain implementation's logits in float64, [T, vocab]."""
    return P.forward(raw, weights, list(ids), dtype=torch.float64).numpy()


TOL = {"float32": 2e-5, "bfloat16": 4e-2}
# The one-mixer attention models have scores of tens: q and k rounded to bfloat16 (2^-9 each) move such a score by a
# tenth, and so a key's weight by a tenth.  Their bfloat16 bound is that share of the logits' scale; their float32
# bound is the common one, and that is the run which shows a wrong key.
SHARP_BF16_TOL = 0.15


def tolerance(name: str, dtype: str) -> float:
    return SHARP_BF16_TOL if (name in ("latent", "blocks") and dtype == "bfloat16") else TOL[dtype]
