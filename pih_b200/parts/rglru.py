"""Recurrent block with a real-gated linear recurrent unit (RG-LRU), as a mixer.

Two branches of ``width`` channels read the block's input: ``y = gelu_tanh(W_y h + b_y)`` and
``u = conv(W_x h + b_x)`` (a short causal convolution per channel with a bias, no activation).  The channels of ``u``
are cut into ``blocks`` equal parts; within part b two square matrices give the gates
``r = sigmoid(R_b u_b + r_b)`` and ``i = sigmoid(I_b u_b + i_b)``.  Then, per channel, with ``S`` starting at zero::

    a = exp(-decay_scale * r * softplus(lam))        S <- a * S + sqrt(1 - a^2) * (i * u)

and the output is ``W_o (S * y)``.  (The recurrence is the one of De et al., "Griffin: Mixing Gated Linear
Recurrences with Local Attention for Efficient Language Models".)  The gates, the decay and the state are 32-bit
whatever the compute dtype.  The state slot holds ``S [width]`` and behind it the convolution's last ``taps - 1``
inputs ``[taps - 1, width]``.
"""
from __future__ import annotations

import torch

from .registry import Runtime, StateNeed, TensorInfo, register_mixer
from ._bind import bind_matrix


@register_mixer("rglru")
class RGLRU:
    pad_safe = True            # the kernels go by requests: rows of no request are never read or written

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        W, B = spec.width, spec.blocks
        bw = W // B
        return {n["y"]: TensorInfo((W, spec.hidden)), n["y_bias"]: TensorInfo((W,)),
                n["x"]: TensorInfo((W, spec.hidden)), n["x_bias"]: TensorInfo((W,)),
                n["conv"]: TensorInfo((W, spec.conv_taps), "conv"), n["conv_bias"]: TensorInfo((W,)),
                n["r"]: TensorInfo((B, bw, bw)), n["r_bias"]: TensorInfo((B, bw), "unit_normal"),
                n["i"]: TensorInfo((B, bw, bw)), n["i_bias"]: TensorInfo((B, bw), "unit_normal"),
                n["lam"]: TensorInfo((W,), "unit_normal"), n["o"]: TensorInfo((spec.hidden, W))}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.width % spec.blocks:
            raise ValueError(f"width ({spec.width}) must be a multiple of blocks ({spec.blocks})")
        self.spec, self.rt = spec, rt
        n = spec.names
        self.w_in = bind_matrix(torch.cat([weights[n["y"]], weights[n["x"]]], dim=0), rt)          # [y | x]
        self.w_conv = bind_matrix(weights[n["conv"]], rt)
        self.w_gates = bind_matrix(torch.cat([weights[n["r"]], weights[n["i"]]], dim=1), rt)       # [B, 2 bw, bw]
        self.w_o = bind_matrix(weights[n["o"]], rt)
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.y_bias = weights[n["y_bias"]].to(**f32).contiguous()
        self.x_bias = weights[n["x_bias"]].to(**f32).contiguous()
        self.conv_bias = weights[n["conv_bias"]].to(**f32).contiguous()
        self.r_bias = weights[n["r_bias"]].to(**f32).reshape(-1).contiguous()
        self.i_bias = weights[n["i_bias"]].to(**f32).reshape(-1).contiguous()
        self.lam = weights[n["lam"]].to(**f32).contiguous()

    def cache_need(self):
        return StateNeed((self.spec.conv_taps * self.spec.width,), torch.float32)

    def forward(self, x, step, cache):
        s, ops = self.spec, self.rt.ops
        W, B = s.width, s.blocks
        proj = ops.linear(x, self.w_in)                                     # [T, 2 W]: y branch, x branch
        u = ops.causal_conv(proj[:, W:], self.w_conv, step=step, state=cache.state, state_offset=W,
                            in_bias=self.x_bias, out_bias=self.conv_bias)
        gates = ops.linear_batched(u.view(u.shape[0], B, W // B), self.w_gates, out_dtype=torch.float32)
        out = ops.rglru_scan(u, gates, proj[:, :W], y_bias=self.y_bias, r_bias=self.r_bias, i_bias=self.i_bias,
                             lam=self.lam, decay_scale=s.decay_scale, state=cache.state, step=step, blocks=B)
        return ops.linear(out, self.w_o)
