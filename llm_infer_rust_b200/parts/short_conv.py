"""Short causal convolutions over time whose last inputs are per-request state."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamDecl, Part, StateSpec
from .registry import register_part


class CausalTaps(Part):
    """y_t = (u_t if ``identity``) + sum_j w[:, j] * u_(t - taps + 1 + j) on every channel, zeros before the
    sequence's start, no bias; u_t = x_t * scale_t when a per-token scale is given (a norm handed on unrun).

    The last ``taps - 1`` inputs u of a sequence are its state ([taps - 1, channels] float32 in the request's
    slot), so a step may bring any portion of a sequence."""
    category = "token_conv"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.channels = int(spec["channels"])
        self.taps = int(spec["taps"])
        self.identity = bool(spec.get("identity", False))
        if not 1 <= self.taps <= 8:
            raise ValueError(f"{self.taps} taps are refused: the convolution kernels take 1 to 8")

    def param_decls(self):
        return {"weight": ParamDecl((self.channels, self.taps))}

    def bind(self, name, tensor):
        super().bind(name, tensor)
        self.params[name] = tensor.to(torch.float32).contiguous()       # (a small tensor; the kernels read floats)

    def state_spec(self):
        return StateSpec((self.taps - 1, self.channels), torch.float32) if self.taps > 1 else None

    def forward_after_norm(self, x, add, gain, eps, ctx, state, out_dtype):
        """x += add, a one-gain RMS norm of x and this convolution over it in one kernel, where the step allows it
        (every row one token); None otherwise."""
        return ops.add_norm_taps_single(x, add, gain, eps, self.params["weight"], state, ctx, out_dtype, self.identity)

    def forward(self, x, scale, ctx, state, out_dtype):
        return ops.causal_taps(x, self.params["weight"], state, ctx, out_dtype, scale=scale, identity=self.identity)


register_part("token_conv", "causal_taps", CausalTaps)
