"""Retention as a mixer: linear attention with a fixed decay a head, its matrix state in the request's state slot.

For every head, with ``S [key_dim, value_dim]`` starting at zero, token by token::

    S <- decay * S + k v^T
    o  = S^T q                       (the read-out sees this token's write)

without softmax or denominator.  q and k are rotated by the position (rotate-half over the first ``rotary_dim``
columns of a head), k is then multiplied by ``key_scale``.  The read-out of a head is divided by its root mean square
over ``value_dim`` (no weight), multiplied by ``silu`` of a gate projection, and projected.

One product computes q, k, v and the gate from the block's input; a kernel rotates and scales q and k into 32-bit;
the recurrence runs from the state slot, request by request; ``gated_rmsnorm`` (with a weight of ones) and the output
product follow.  Rotation, state, decay and the read-out's norm are 32-bit whatever the compute dtype.  The decay is
applied as ``S + (decay - 1) S`` with ``decay - 1`` formed in double: a decay next to one keeps its distance from one.
"""
from __future__ import annotations

import torch

from .registry import Runtime, StateNeed, TensorInfo, part_class, register_mixer
from ._bind import bind_matrix


@register_mixer("retention")
class Retention:
    pad_safe = True            # the kernels go by requests: rows of no request are never read or written

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        return {n["q"]: TensorInfo((spec.qk_size, spec.hidden)), n["k"]: TensorInfo((spec.qk_size, spec.hidden)),
                n["v"]: TensorInfo((spec.v_size, spec.hidden)), n["gate"]: TensorInfo((spec.v_size, spec.hidden)),
                n["o"]: TensorInfo((spec.hidden, spec.v_size))}

    def __init__(self, spec, weights, rt: Runtime):
        if len(spec.decays) != spec.heads:
            raise ValueError(f"retention needs one decay a head, got {len(spec.decays)} for {spec.heads} heads")
        self.spec, self.rt = spec, rt
        n = spec.names
        self.w_in = bind_matrix(torch.cat([weights[n[r]] for r in ("q", "k", "v", "gate")], dim=0), rt)
        self.w_o = bind_matrix(weights[n["o"]], rt)
        self.decay_minus_one = torch.tensor([d - 1.0 for d in spec.decays], dtype=torch.float64).to(
            device=rt.device, dtype=torch.float32).contiguous()
        self.ones = torch.ones(spec.value_dim, dtype=torch.float32, device=rt.device)
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, rt)
            if not hasattr(self.position, "frequencies"):
                raise TypeError("retention rotates by frequencies (a position part that computes its angles)")

    def cache_need(self):
        s = self.spec
        return StateNeed((s.heads * s.key_dim * s.value_dim,), torch.float32)

    def forward(self, x, step, cache):
        s, ops = self.spec, self.rt.ops
        QK, VS = s.qk_size, s.v_size
        proj = ops.linear(x, self.w_in)                                     # [T, 2 QK + 2 VS]: q | k | v | gate
        freq = self.position.frequencies() if self.position is not None else None
        o = ops.retention(proj[:, :2 * QK], proj[:, 2 * QK:2 * QK + VS], frequencies=freq,
                          decay_minus_one=self.decay_minus_one, key_scale=s.key_scale, state=cache.state, step=step,
                          heads=s.heads, key_dim=s.key_dim, value_dim=s.value_dim)
        y = ops.gated_rmsnorm(o, proj[:, 2 * QK + VS:], self.ones, s.norm_eps)
        return ops.linear(y, self.w_o)
