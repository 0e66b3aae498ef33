"""A plain, slow Kefetar: whole sequences on the CPU, one function per mechanism.

Written from the design's equations and nothing else; it shares no code with the
package.  Everything is float32 (or float64 with ``dtype=torch.float64``) torch on the
CPU, token by token where a recurrence is involved.  ``weights`` maps checkpoint
tensor names to tensors; ``config`` is the dict of a config.json.

    x_0 = embed[token]
    per layer:  x <- x + mixer(canon1(norm1(x)));  x <- x + ff(canon2(norm2(x)))   (the second only with an mlp)
    logits = head . norm_final(x)
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


def scalar_rms_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * g with ONE gain g for all coordinates."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_taps(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start.  u [T, C], w [C, taps]."""
    T = u.shape[0]
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j                 # tap j reads the input `back` steps earlier
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def canon(h: torch.Tensor, w: Optional[torch.Tensor]) -> torch.Tensor:
    """What a sublayer reads: h + conv(h) (h itself in a model without this convolution)."""
    return h if w is None else h + causal_taps(h, w)


def rotate_half_split(x: torch.Tensor, base: float, dims: int, factor: float = 1.0) -> torch.Tensor:
    """x [T, heads, d]; the first ``dims`` coordinates of every head are rotated, coordinate i paired with
    i + dims/2, by the angle p * base^(-2i/dims) / factor at position p (= row index)."""
    T = x.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims) / factor
    a = torch.arange(T, dtype=torch.float64)[:, None] * f[None, :]
    cos, sin = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def retention_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                         S0: Optional[torch.Tensor] = None, return_state: bool = False):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token.  q, k [T, H, d]; v [T, H, dv]."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype) if S0 is None else S0.clone()
    o = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return (o, S) if return_state else o


def retention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head, no softmax and no denominator."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W["q"].T).view(T, H, d)
    k = (h @ W["k"].T).view(T, H, d)
    v = (h @ W["v"].T).view(T, H, dv)
    rot = m.get("rot")
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_half_split(q, rot["base"], rot["dims"], factor)
        k = rotate_half_split(k, rot["base"], rot["dims"], factor)
    k = k * d ** -0.5
    o = retention_recurrence(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = unit_rms(o, eps).reshape(T, H * dv)
    gate = h @ W["g"].T
    return (o * (gate * torch.sigmoid(gate))) @ W["o"].T


def capped_causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                            cap: Optional[float]) -> torch.Tensor:
    """softmax over j <= i of cap * tanh(scale q_i . k_j / cap) (no cap: the scaled score itself), times v.
    q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~mask, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, kv]
    return out


def attention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict, v_first: Optional[torch.Tensor],
                    is_first_vmix: bool):
    """Grouped-query softmax attention with short convolutions on q, k, v, soft-capped scores, value mixing
    and a sigmoid output gate.  Returns (output, this layer's unmixed-or-mixed v as [T, G*dv])."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ W["q"].T, h @ W["k"].T, h @ W["v"].T
    if m.get("conv"):
        q, k, v = causal_taps(q, W["q.conv"]), causal_taps(k, W["k.conv"]), causal_taps(v, W["v.conv"])
    q, k = q.view(T, H, d), k.view(T, G, d)
    rot = m.get("rot")
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_half_split(q, rot["base"], rot["dims"], factor)
        k = rotate_half_split(k, rot["base"], rot["dims"], factor)
    if m.get("v_mix") and not is_first_vmix:
        lam = W["vmix"]
        v = (1.0 - lam) * v + lam * v_first
    v_out = v
    out = capped_causal_attention(q, k, v.view(T, G, dv), m["scale"], m.get("softcap"))
    gate = torch.sigmoid(h @ W["g"].T)
    return (out.reshape(T, H * dv) * gate) @ W["o"].T, v_out


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """a N(z) + b N(z^2) + c N(z^3) + e, N = division by the root mean square over a token's vector."""
    a, b, c, e = coef[0], coef[1], coef[2], coef[3]
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    return poly_norm(h @ W["up"].T, W["act"], eps) @ W["down"].T


def sub(weights: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(dtype) for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float32,
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    eps = float(config["norm"]["eps"])
    x = weights["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        taps = {n: weights[p + n].to(dtype) if config.get("canon") else None for n in ("canon1", "canon2")
                if config.get("canon") is None or p + n in weights}
        h = canon(scalar_rms_norm(x, weights[p + "norm1"].to(dtype), eps), taps["canon1"])
        W = sub(weights, p + "mix.", dtype)
        if layer["type"] == "retention":
            y = retention_mixer(h, W, m, eps)
        elif layer["type"] == "attention":
            first = bool(m.get("v_mix")) and v_first is None
            y, v = attention_mixer(h, W, m, v_first, first)
            if first:
                v_first = v
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            h = canon(scalar_rms_norm(x, weights[p + "norm2"].to(dtype), eps), taps["canon2"])
            x = x + dense_ff(h, sub(weights, p + "mlp.", dtype), eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = scalar_rms_norm(x, weights["final.norm"].to(dtype), eps)
    return x @ weights["head"].to(dtype).T
