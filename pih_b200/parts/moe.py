"""Mixture-of-experts feed-forward: ``experts`` gated feed-forward layers of which every row uses ``top``.

Router logits ``z = W_r x`` are 32-bit; the ``top`` largest choose the experts (ties: the smaller index) and the
softmax over the CHOSEN logits alone gives their weights.  Expert e is ``W_down_e (silu(W_gate_e x) * (W_up_e x))``
without biases; the output is the weighted sum of the chosen experts' outputs, summed in 32-bit in the order of
the choice.

The experts' weights are stacked ``[experts, ...]``; rows are grouped by expert on the device and the grouped
products find their rows there, so nothing returns to the host and a step's launches do not depend on the routing.
"""
from __future__ import annotations

import torch

from .registry import Runtime, TensorInfo, register_ffn
from ._bind import bind_matrix


@register_ffn("moe")
class MixtureOfExperts:
    pad_safe = True            # row-wise: rows of padding are routed and computed like any other and never read

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        out = {n["router"]: TensorInfo((spec.experts, spec.hidden))}
        for e in range(spec.experts):
            p = n["expert"].format(e)
            out[p + n["gate"]] = TensorInfo((spec.intermediate, spec.hidden))
            out[p + n["up"]] = TensorInfo((spec.intermediate, spec.hidden))
            out[p + n["down"]] = TensorInfo((spec.hidden, spec.intermediate))
        return out

    def __init__(self, spec, weights, rt: Runtime):
        if spec.activation != "silu":
            raise ValueError(f"the experts support activation 'silu', got {spec.activation!r}")
        if not 1 <= spec.top <= spec.experts:
            raise ValueError(f"top ({spec.top}) must be between 1 and experts ({spec.experts})")
        self.spec, self.rt = spec, rt
        n = spec.names

        def stack(role):
            return bind_matrix(torch.stack([weights[n["expert"].format(e) + n[role]] for e in range(spec.experts)]), rt)

        self.w_router = bind_matrix(weights[n["router"]], rt)
        # an expert's gate rows and behind them its up rows: one matrix [experts, 2 ff, hidden], so that one grouped
        # product reads the rows once
        self.w_gate_up = bind_matrix(torch.cat([torch.stack([weights[n["expert"].format(e) + n[r]]
                                                             for e in range(spec.experts)]) for r in ("gate", "up")], dim=1), rt)
        self.w_down = stack("down")

    def forward(self, x):
        ops = self.rt.ops
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)      # [T, experts], 32-bit
        return ops.moe_experts(x, logits, self.w_gate_up, self.w_down, self.spec.top)
