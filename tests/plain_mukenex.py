"""A plain, slow Mukenex: whole sequences on the CPU, one function per mechanism.

Written from the design's equations and nothing else; it shares no code with the package.  Everything is
torch on the CPU in ``dtype`` (float64 by default), token by token where a recurrence is involved.
``weights`` maps checkpoint tensor names to tensors, ``config`` is the dict of a config.json.

    e = embed[token];  X = (e, ..., e)  (``streams`` copies; one copy and the ordinary residual sum without the key)
    run list: layers [0, a), then layers [a, b) ``times`` times, then layers [b, L)   (``loop`` = {start a, stop b, times})
    per sublayer q of a layer (mixer, then feed-forward if the layer has one):
        u = sum_s in_q[s] X_s;   y = sublayer(N(u));   X_t <- sum_s mix_q[s, t] X_s + out_q[t] y
    x = sum_s X_s;  z = head . N_final(x);  logits = cap * tanh(z / cap)
    N(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------ small pieces
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, one_plus: bool) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * g over the last axis, g = 1 + w or w."""
    g = 1.0 + w if one_plus else w
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def rotate_pairs(x: torch.Tensor, base: float, dims: int, first_position: int = 0) -> torch.Tensor:
    """x [T, heads, d]: of every head's first ``dims`` coordinates, coordinate 2i is paired with 2i + 1 and the pair
    (u, v) of the token at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i / dims)."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    a = (first_position + torch.arange(T, dtype=torch.float64))[:, None] * f[None, :]
    cos, sin = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def window_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] True where query i reads key j: 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] True where query i reads key j: j <= i and both lie in the same block of ``size`` positions
    counted from position 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def masked_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: torch.Tensor,
                             sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, d], k [T, H, d], v [T, H, dv] (keys and values already spread over the query heads).
    p_ij = exp(s_ij) / (sum_visible exp(s_ij) [+ exp(sink_h)]), s = scale q.k; the sink has no value."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.to(s.dtype)[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(s.dtype)[:, None, None] - m)
    return torch.einsum("hij,jhd->ihd", e / den, v)


# ------------------------------------------------------------------------------------------------ mixers
def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Attention whose keys and values are expanded from a narrow latent.  Per head the query is [dim plain | rot_dim
    rotated]; the down projection gives [kv_rank latent (normed, plain weight) | rot_dim rotated key part that all
    heads share]; keys' plain part and values come from the latent by two up projections."""
    T = h.shape[0]
    H, d, r, dv, c_dim = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).reshape(T, H, d + r)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :c_dim], w[p + "dkv.norm"], eps, one_plus=False)
    k_rot = down[:, c_dim:].reshape(T, 1, r)
    rot = m["rot"]
    q_rot = rotate_pairs(q[..., d:], rot["base"], rot["dims"])
    k_rot = rotate_pairs(k_rot, rot["base"], rot["dims"]).expand(T, H, r)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    o = masked_softmax_attention(torch.cat([q[..., :d], q_rot], -1), torch.cat([k_plain, k_rot], -1), v, m["scale"],
                                 window_mask(T, m["mask"]["size"]), sink=w[p + "sink"])
    o = o.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def grouped_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention with biased projections, a per-head norm of q and k (one weight for all heads, plain),
    no rotation, and keys visible only inside the query's block of positions."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps, one_plus=False)
    k = rms_norm(k, w[p + "k.norm"], eps, one_plus=False)
    rep = H // G
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    o = masked_softmax_attention(q, k, v, m["scale"], chunk_mask(T, m["mask"]["size"]))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """Per head S_t = g S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t.  q, k [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype)
    g = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    out = []
    for t in range(T):
        S = g * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hde,hd->he", S, q[t]))
    return torch.stack(out)


def lightning(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, d)
    k = silu(h @ w[p + "k"].T).reshape(T, H, d)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    o = decay_recurrence(q, k, v, m["decay"]).reshape(T, H * dv)
    o = rms_norm(o, w[p + "norm"], eps, one_plus=False) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def table_experts(h: torch.Tensor, ids: List[int], w: Dict[str, torch.Tensor], p: str, top: int) -> torch.Tensor:
    """Every token's experts are the row of its token id in an integer table; each counts 1 / top."""
    out = torch.zeros_like(h)
    table = w[p + "table"]
    for t, token in enumerate(ids):
        for e in table[token].tolist():
            e = int(e)
            x = h[t]
            a = silu(w[f"{p}e{e}.gate"].to(h.dtype) @ x) * (w[f"{p}e{e}.up"].to(h.dtype) @ x)
            out[t] += (w[f"{p}e{e}.down"].to(h.dtype) @ a) / top
    return out


# ------------------------------------------------------------------------------------------------ the model
def run_list(config: dict) -> List[int]:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(config: dict, weights: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives the stream (the sum over the
    copies) after every layer run."""
    w = {n: (t if not t.is_floating_point() else t.to(dtype)) for n, t in weights.items()}
    eps = config["norm"]["eps"]
    s = config.get("streams")
    e = w["embed"][torch.tensor(ids)]
    X = [e.clone() for _ in range(s or 1)]

    def sublayer(X, prefix, norm_name, fn):
        if s:
            cin, cout, cmix = w[prefix + ".in"], w[prefix + ".out"], w[prefix + ".mix"]
            u = sum(cin[a] * X[a] for a in range(s))
            y = fn(rms_norm(u, w[norm_name], eps, one_plus=True))
            return [sum(cmix[a, t] * X[a] for a in range(s)) + cout[t] * y for t in range(s)]
        return [X[0] + fn(rms_norm(X[0], w[norm_name], eps, one_plus=True))]

    mixers = {"latent_attention": latent_attention, "attention": grouped_attention, "lightning": lightning}
    for i in run_list(config):
        layer = config["layers"][i]
        p = f"l{i}."
        X = sublayer(X, p + "hc1", p + "norm1",
                     lambda h: mixers[layer["type"]](h, w, p + "mix.", layer["mixer"], eps))
        mlp = layer.get("mlp")
        if mlp:
            if mlp["kind"] == "dense":
                X = sublayer(X, p + "hc2", p + "norm2", lambda h: dense_ff(h, w, p + "mlp."))
            else:
                X = sublayer(X, p + "hc2", p + "norm2",
                             lambda h: table_experts(h, ids, w, p + "mlp.", mlp["router"]["top"]))
        if layers_out is not None:
            layers_out.append(sum(X))
    z = rms_norm(sum(X), w["final.norm"], eps, one_plus=True) @ w["head"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
