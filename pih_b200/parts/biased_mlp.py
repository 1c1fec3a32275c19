"""Two-matrix feed-forward with biases: ``W_down act(W_up x + b_up) + b_down``.

The activation is xIELU with two learned numbers ``(p, q)``: for z > 0 ``softplus(p) z^2 + z / 2``, for z <= 0
``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``.  The up product is rounded to the compute dtype; bias and
activation are one kernel in 32-bit.  The output bias is left to the caller (``output_bias``): a block that norms
the feed-forward's output adds it in the kernel that norms, and ``forward_with_bias`` adds it here.
"""
from __future__ import annotations

import math

import torch

from .registry import Runtime, TensorInfo, register_ffn
from ._bind import bind_matrix


def _softplus(z: float) -> float:
    return z if z > 30.0 else math.log1p(math.exp(z))


@register_ffn("biased_mlp")
class BiasedMLP:
    pad_safe = True                        # row-wise: rows of padding are computed and never read

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        return {n["up"]: TensorInfo((spec.intermediate, spec.hidden)), n["up_bias"]: TensorInfo((spec.intermediate,)),
                n["down"]: TensorInfo((spec.hidden, spec.intermediate)), n["down_bias"]: TensorInfo((spec.hidden,)),
                n["act"]: TensorInfo((2,), "unit_normal")}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.activation != "xielu":
            raise ValueError(f"the biased feed-forward supports activation 'xielu', got {spec.activation!r}")
        self.spec, self.rt = spec, rt
        n = spec.names
        self.w_up = bind_matrix(weights[n["up"]], rt)
        self.w_down = bind_matrix(weights[n["down"]], rt)
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.up_bias = weights[n["up_bias"]].to(**f32).contiguous()
        self.output_bias = weights[n["down_bias"]].to(**f32).contiguous()
        p, q = (float(v) for v in weights[n["act"]].to(torch.float64))
        self.alpha_positive, self.alpha_negative = _softplus(p), 0.5 + _softplus(q)

    def forward(self, x):
        """Without the output bias (see ``output_bias``)."""
        ops = self.rt.ops
        z = ops.linear(x, self.w_up)
        a = ops.bias_xielu(z, self.up_bias, self.alpha_positive, self.alpha_negative)
        return ops.linear(a, self.w_down)
