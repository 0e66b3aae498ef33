"""Small Kefetar configurations, random weights for them and helpers that run them through the engine.

The configurations differ from one another in every size and option: the order of the layers, head counts and
groups, key and value widths, the rotated share of a head, taps of both kinds of convolution, soft-cap or none,
value mixing or none, layers with and without a feed-forward.  Weights are drawn with torch's generator and are
representable in bfloat16, so that the float32 engine, the bfloat16 engine and the plain implementation read
the same numbers.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_kefetar as P


def attention(heads, kv_heads, dim, vdim, scale, conv=None, rot=None, softcap=None, v_mix=False, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = rot
    if softcap:
        m["softcap"] = softcap
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def retention(heads, dim, vdim, decay, rot=None, ff=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = rot
    return {"type": "retention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, eps, layers, canon_taps=None):
    raw = {"architecture": "Kefetar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if canon_taps:
        raw["canon"] = {"taps": canon_taps}
    return raw


CONFIGS = {
    # retention first; partial rotation with scaling; values narrower than keys; three attention layers that mix values
    "K1": config(97, 48, 1e-5, [
        retention(2, 8, 16, [0.9, 0.995], rot={"base": 1000.0, "dims": 4}, ff=40),
        attention(4, 2, 16, 8, 0.31, conv=3, rot={"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0}},
                  softcap=20.0, v_mix=True, ff=56),
        attention(4, 2, 16, 8, 0.27, conv=2, rot={"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0}},
                  softcap=20.0, v_mix=True),
        retention(3, 16, 8, [0.97, 0.5, 0.999], ff=24),
        attention(2, 2, 12, 8, 0.4, rot={"base": 500.0, "dims": 12}, v_mix=True, ff=32),
    ], canon_taps=4),
    # no input convolution at all, one query head per key head, values wider than keys, no soft-cap, no rotation
    "K2": config(131, 40, 3e-6, [
        attention(3, 3, 8, 24, 0.5, conv=4, ff=64),
        retention(1, 24, 40, [0.98], rot={"base": 77.0, "dims": 24, "scaling": {"factor": 2.0}}),
        attention(6, 1, 10, 10, 0.2, softcap=5.0, rot={"base": 3000.0, "dims": 2}),
    ]),
    # a head size of the tensor-core kernels and values as wide as keys, one layer with a soft-cap and one without
    "K3": config(211, 64, 1e-6, [
        attention(4, 2, 32, 32, 0.18, conv=2, rot={"base": 10000.0, "dims": 32}, softcap=6.0, v_mix=True, ff=96),
        retention(2, 32, 32, [0.96, 0.99], rot={"base": 10000.0, "dims": 16}),
        attention(4, 2, 32, 32, 0.18, rot={"base": 10000.0, "dims": 32}, v_mix=True, ff=96),
    ], canon_taps=2),
}

# convolutions of ONE tap (a gain per channel, no state), a layer order that ends on retention without feed-forward
CONFIGS["K4"] = config(61, 24, 1e-5, [
    attention(2, 1, 8, 8, 0.35, conv=1, rot={"base": 10.0, "dims": 8}, ff=16),
    retention(2, 8, 8, [0.9, 0.8]),
], canon_taps=1)

# heads wider than 128: the all-sizes attention kernel with keys of 160 and values of 136, retention by the scan alone
CONFIGS["K5"] = config(73, 56, 1e-5, [
    attention(2, 1, 160, 136, 0.08, conv=2, rot={"base": 1000.0, "dims": 96}, softcap=10.0, ff=48),
    retention(1, 192, 72, [0.99], rot={"base": 1000.0, "dims": 64}),
], canon_taps=2)

# One mixer alone, the attention one with scores so sharp that a single key decides a position's result; widths
# that are no whole 16-byte pieces (the kernels' one-channel-a-thread forms).
ONLY_ATTENTION = config(89, 34, 1e-5, [
    attention(4, 2, 16, 12, 3.0, conv=3, rot={"base": 100.0, "dims": 8, "scaling": {"factor": 2.0}}, softcap=30.0)],
    canon_taps=3)
ONLY_RETENTION = config(89, 36, 1e-5, [
    retention(2, 16, 24, [0.999, 0.9995], rot={"base": 100.0, "dims": 16})], canon_taps=3)


def bf16_values(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def random_weights(raw: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors by name, float32 with bfloat16-representable values."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return bf16_values(mean + std * torch.randn(tuple(shape), generator=g))

    w, width = {}, raw["width"]
    taps = (raw.get("canon") or {}).get("taps", 0)
    w["embed"] = normal(raw["vocab"], width)
    w["head"] = normal(raw["vocab"], width, std=width ** -0.5)
    w["final.norm"] = normal(std=0.1, mean=1.0)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        kv = m.get("kv_heads", m["heads"])
        rows = {"q": m["heads"] * m["dim"], "k": kv * m["dim"], "v": kv * m["vdim"], "g": m["heads"] * m["vdim"]}
        w[p + "norm1"] = normal(std=0.2, mean=1.0)
        if taps >= 1:
            w[p + "canon1"] = normal(width, taps, std=0.4)
        for name, n in rows.items():
            w[p + "mix." + name] = normal(n, width, std=width ** -0.5 * (2.0 if name in "qk" else 1.0))
        w[p + "mix.o"] = normal(width, rows["g"], std=rows["g"] ** -0.5)
        if layer["type"] == "attention":
            if m.get("conv", 0) >= 1:
                for name in "qkv":
                    w[p + f"mix.{name}.conv"] = normal(rows[name], m["conv"], std=0.6)
            if m.get("v_mix"):
                w[p + "mix.vmix"] = bf16_values(torch.tensor(0.25 + 0.5 * torch.rand((), generator=g).item()))
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            w[p + "norm2"] = normal(std=0.2, mean=1.0)
            if taps >= 1:
                w[p + "canon2"] = normal(width, taps, std=0.4)
            w[p + "mlp.up"] = normal(ff, width, std=width ** -0.5)
            w[p + "mlp.down"] = normal(width, ff, std=ff ** -0.5)
            w[p + "mlp.act"] = normal(4, std=0.7)
    return w


def write_model(folder: str, raw: dict, weights: Dict[str, torch.Tensor], dtype: str = "bfloat16") -> str:
    from llm_infer_rust_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(raw, fh)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    write_safetensors(os.path.join(folder, "model.safetensors"), [(n, t.to(store)) for n, t in weights.items()])
    return folder


def make_engine(folder: str, dtype: str, page_size: int = 16, pool_tokens: int = 1024, max_requests: int = 4, **kw):
    from llm_infer_rust_b200.engine import Engine
    kw.setdefault("cuda_graph_bs", 0)
    kw.setdefault("max_prefill_tokens_per_batch", 0)
    kw.setdefault("chunked_prefill_size", 0)
    kw.setdefault("log_level", "error")
    return Engine(folder, dtype=dtype, max_running_req=max_requests, page_size=page_size,
                  max_total_tokens=pool_tokens, max_seq_len=4096, **kw)


def tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def oracle(raw: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int]) -> np.ndarray:
    """The plain implementation's logits in float64, [T, vocab]."""
    return P.forward(raw, weights, list(ids), dtype=torch.float64).numpy()


def run_alone(engine, rid: int, ids: Sequence[int], portions: Sequence[int]) -> np.ndarray:
    """One request in the given portions, every position wanted; logits [T, vocab]."""
    from llm_infer_rust_b200.engine import StepEntry
    assert sum(portions) == len(ids)
    engine.open_request(rid)
    out, at = [], 0
    for n in portions:
        out.append(engine.step([StepEntry(rid, ids[at:at + n], list(range(n)))]).cpu().numpy().copy())
        at += n
    engine.close_request(rid)
    engine.check_kernel_errors()
    return np.concatenate(out)


TOL = {"float32": 2e-5, "bfloat16": 4e-2}
# The one-mixer attention model has scores up to its cap of 30: q and k rounded to bfloat16 (2^-9 each) move such a
# score by up to 30 * 2^-8 = 0.12, and so a key's weight by 12 %.  Its bfloat16 bound is that share of the logits' scale;
# its float32 bound is the common one, and that is the run which shows a wrong key.
SHARP_BF16_TOL = 0.12


def tolerance(name: str, dtype: str) -> float:
    return SHARP_BF16_TOL if (name == "attention" and dtype == "bfloat16") else TOL[dtype]


def check(got: np.ndarray, want: np.ndarray, dtype: str, what: str, tol: float = None) -> None:
    """Every position's logits within ``tol`` of the logits' scale (largest absolute difference)."""
    tol = TOL[dtype] if tol is None else tol
    scale = max(1.0, float(np.abs(want).max()))
    err = np.abs(got.astype(np.float64) - want).max(axis=1)
    bad = np.nonzero(err > tol * scale)[0]
    assert bad.size == 0, (f"{what}: {bad.size} of {len(err)} positions are off, the first at {int(bad[0])} by "
                           f"{err[bad[0]]:.3e}, the worst at {int(err.argmax())} by {err.max():.3e} "
                           f"(allowed {tol * scale:.3e})")
