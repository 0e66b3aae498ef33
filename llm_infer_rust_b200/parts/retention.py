"""Retention: linear attention with a fixed decay per head."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamDecl, Part, StateSpec
from .registry import register_part


class DecayRetention(Part):
    """q, k, v, g = x W^T (one packed matrix: q rows, k rows, v rows, gate rows); q and k rotated (the model's
    position encoding of that name, or none), k times ``k_scale``; per head

        S_t = decay_h S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t

    with S [head_dim, v_head_dim] in float32 in the request's state slot (zeros at a sequence's start); every
    head's o divided by its root mean square (``eps``, no weight), times silu(g), then the output projection.
    No softmax, no denominator, no bias.  ``decay``: one number per head.

    Two options.  ``qkv_activation`` (silu, ...): q, k and v pass through it right after the projection.
    ``output`` "joint_norm_sigmoid": instead of the per-head unit norm and silu gate, all heads' o together are
    RMS-normed with a weight (``norm`` [heads * v_head_dim]) and multiplied by sigmoid(g)."""
    category = "mixer"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec["v_head_dim"])
        self.eps = float(spec["eps"])
        self.k_scale = float(spec.get("k_scale", self.d ** -0.5))
        self.qkv_activation = spec.get("qkv_activation")
        self.output = str(spec.get("output", "head_unit_silu"))
        if self.qkv_activation is not None and self.qkv_activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.qkv_activation!r} is refused: {sorted(ops.ACTIVATIONS)}")
        if self.output not in ("head_unit_silu", "joint_norm_sigmoid"):
            raise ValueError(f"output {self.output!r} is refused: head_unit_silu or joint_norm_sigmoid")
        decay = [float(g) for g in spec["decay"]]
        if len(decay) != self.nh:
            raise ValueError("one decay per head is needed")
        if self.d > 512:
            raise ValueError(f"head_dim {self.d} is refused: the retention kernel keeps up to 512 rows of a state")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=env.device)
        name = spec.get("position_encoding")
        self.rope = env.position_encodings[name] if name else None
        if self.rope is not None and self.rope.rot_dim > self.d:
            raise ValueError("the rotation is wider than a head")

    def param_decls(self):
        decls = {"qkvg_proj": ParamDecl((self.nh * (2 * self.d + 2 * self.dv), self.hidden)),
                 "o_proj": ParamDecl((self.hidden, self.nh * self.dv))}
        if self.output == "joint_norm_sigmoid":
            decls["norm"] = ParamDecl((self.nh * self.dv,), "vector")
        return decls

    def bind(self, name, tensor):
        super().bind(name, tensor)
        if name == "norm":
            self.params[name] = tensor.to(torch.float32).contiguous()

    def cache_spec(self):
        return None

    def state_spec(self):
        return StateSpec((self.nh, self.d, self.dv), torch.float32)

    def forward(self, x, ctx, cache):
        p = self.params
        packed = ops.linear(x, p["qkvg_proj"])
        rope = self.rope
        gate_column = self.nh * (2 * self.d + self.dv)
        if self.qkv_activation is not None:
            ops.activate(packed, self.qkv_activation, columns=gate_column, in_place=True)
        o = ops.retention(packed, cache.state, self.decay, rope.inv_freq if rope else None,
                          rope.rot_dim if rope else 0, self.k_scale, ctx, self.nh, self.d, self.dv)
        if self.output == "joint_norm_sigmoid":
            gated = ops.row_norm_gate(o, p["norm"], packed, gate_column, self.eps)
        else:
            gated = ops.head_unit_norm_gate(o, packed, gate_column, self.nh, self.dv, self.eps)
        return ops.linear(gated, p["o_proj"])


register_part("mixer", "decay_retention", DecayRetention)
