"""Gated delta rule as a mixer: a matrix state per head, carried in the request's state slot.

For every head, with ``S [key_dim, value_dim]`` starting at zero, token by token::

    S <- g * S                       g = exp(-exp(A) * softplus(a + bias))     decay, one number a head
    u  = beta * (v - S^T k)          beta = sigmoid(b)                         how strongly the new value is written
    S <- S + k u^T
    o  = S^T q                       (the read-out sees this token's write)

q and k have ``kv_heads`` heads, each shared by ``heads / kv_heads`` value heads; q, k and v pass a short causal
convolution and SiLU; q and k are made unit vectors (q also times ``key_dim ** -0.5``).  The read-out of a head is
RMS-normed over ``value_dim``, weighted, and multiplied by ``silu`` of a gate projection; then the output projection.

One product computes q, k, v, the gate and the two per-head logits from the block's input; the convolution, the
unit norms, decay and write strength, the recurrence and the gated norm are kernels of ``csrc/sequence.cu``.  State,
decays, write strengths and unit norms are 32-bit whatever the compute dtype.  The state slot holds
``S [heads, key_dim, value_dim]`` and behind it the convolution's last ``taps - 1`` inputs ``[taps - 1, channels]``.
"""
from __future__ import annotations

import torch

from .registry import Runtime, StateNeed, TensorInfo, register_mixer
from ._bind import bind_matrix


@register_mixer("gated_delta")
class GatedDelta:
    pad_safe = True            # the kernels go by requests: rows of no request are never read or written

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        conv = spec.conv_taps
        return {n["q"]: TensorInfo((spec.qk_size, spec.hidden)), n["k"]: TensorInfo((spec.qk_size, spec.hidden)),
                n["v"]: TensorInfo((spec.v_size, spec.hidden)),
                n["q_conv"]: TensorInfo((spec.qk_size, conv), "conv"), n["k_conv"]: TensorInfo((spec.qk_size, conv), "conv"),
                n["v_conv"]: TensorInfo((spec.v_size, conv), "conv"),
                n["beta"]: TensorInfo((spec.heads, spec.hidden)), n["decay"]: TensorInfo((spec.heads, spec.hidden)),
                n["decay_log"]: TensorInfo((spec.heads,), "unit_normal"), n["decay_bias"]: TensorInfo((spec.heads,), "unit_normal"),
                n["out_norm"]: TensorInfo((spec.value_dim,), "one_plus_normal"),
                n["gate"]: TensorInfo((spec.v_size, spec.hidden)), n["o"]: TensorInfo((spec.hidden, spec.v_size))}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads ({spec.heads}) must be a multiple of kv_heads ({spec.kv_heads})")
        self.spec, self.rt = spec, rt
        n = spec.names
        # one product for everything that reads the block's input: [q | k | v | gate | beta | decay]
        self.w_in = bind_matrix(torch.cat([weights[n[r]] for r in ("q", "k", "v", "gate", "beta", "decay")], dim=0), rt)
        self.w_conv = bind_matrix(torch.cat([weights[n[r]] for r in ("q_conv", "k_conv", "v_conv")], dim=0), rt)
        self.w_o = bind_matrix(weights[n["o"]], rt)
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.decay_log = weights[n["decay_log"]].to(**f32).contiguous()
        self.decay_bias = weights[n["decay_bias"]].to(**f32).contiguous()
        self.out_norm = weights[n["out_norm"]].to(**f32).contiguous()
        self.channels = 2 * spec.qk_size + spec.v_size
        self.matrix_numbers = spec.heads * spec.key_dim * spec.value_dim

    def cache_need(self):
        return StateNeed((self.matrix_numbers + (self.spec.conv_taps - 1) * self.channels,), torch.float32)

    def forward(self, x, step, cache):
        s, ops = self.spec, self.rt.ops
        C, VS, H = self.channels, s.v_size, s.heads
        proj = ops.linear(x, self.w_in)                                     # [T, C + VS + 2 H]
        qkv = ops.causal_conv(proj[:, :C], self.w_conv, step=step, state=cache.state, state_offset=self.matrix_numbers,
                              activation="silu")
        o = ops.gated_delta_rule(qkv, proj[:, C + VS:], decay_log=self.decay_log, decay_bias=self.decay_bias,
                                 state=cache.state, step=step, heads=H, kv_heads=s.kv_heads, key_dim=s.key_dim,
                                 value_dim=s.value_dim, unit_eps=s.unit_eps, q_scale=s.key_dim ** -0.5)
        y = ops.gated_rmsnorm(o, proj[:, C:C + VS], self.out_norm, s.norm_eps)
        return ops.linear(y, self.w_o)
