"""Differential attention over a paged cache, as a mixer.

Every query head has two maps.  With ``q [heads, 2, key_dim]``, ``k [kv_heads, 2, key_dim]`` (laid out head by head
as [map 1 | map 2]) and ``v [kv_heads, value_dim]``::

    a_j = softmax(scale * q_j . k_j over the keys up to the row's position) v          j = 1, 2: the same values
    o   = a_1 - lambda * a_2            lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init, one number a layer
    o   = o / sqrt(mean(o^2) + eps) * out_scale                                        per head, over value_dim

q and k pass a per-map RMS norm (one weight vector of ``key_dim`` for all heads and maps) and then the rotation.
Query head ``h`` reads key/value head ``h // (heads // kv_heads)``.

The cache holds ONE vector per token, ``[k: kv_heads x 2 x key_dim | v: kv_heads x value_dim]``, after norm and
rotation (``PagedVectorNeed``: key and value sizes need not be equal).  A mixer built with ``own_kv`` False has no
key/value tensors: its schedule entry reads another entry's cache, with queries, ``lambda`` and output projection of
its own.  Scores, softmax, the combination and the head's norm are 32-bit whatever the compute dtype.
"""
from __future__ import annotations

import math

import torch

from .registry import PagedVectorNeed, Runtime, TensorInfo, part_class, register_mixer
from ._bind import bind_matrix


@register_mixer("diff_attention")
class DiffAttention:
    pad_safe = True            # rows of no request carry the padding slot: nothing is written for them, and what is
                               # computed for them is never read

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        out = {n["q"]: TensorInfo((spec.q_size, spec.hidden)), n["o"]: TensorInfo((spec.hidden, spec.heads * spec.value_dim))}
        for r in ("lq1", "lk1", "lq2", "lk2"):
            out[n[r]] = TensorInfo((spec.key_dim,))
        if spec.qk_norm_eps is not None:
            out[n["q_norm"]] = TensorInfo((spec.key_dim,), "one_plus_normal")
        if spec.own_kv:
            out[n["k"]] = TensorInfo((spec.k_size, spec.hidden))
            out[n["v"]] = TensorInfo((spec.v_size, spec.hidden))
            if spec.qk_norm_eps is not None:
                out[n["k_norm"]] = TensorInfo((spec.key_dim,), "one_plus_normal")
        return out

    def __init__(self, spec, weights, rt: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads ({spec.heads}) must be a multiple of kv_heads ({spec.kv_heads})")
        self.spec, self.rt = spec, rt
        n = spec.names
        rows = [weights[n["q"]]] + ([weights[n["k"]], weights[n["v"]]] if spec.own_kv else [])
        self.w_in = bind_matrix(torch.cat(rows, dim=0), rt)
        self.w_o = bind_matrix(weights[n["o"]], rt)
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.q_norm = self.k_norm = None
        if spec.qk_norm_eps is not None:
            self.q_norm = weights[n["q_norm"]].to(**f32).contiguous()
            if spec.own_kv:
                self.k_norm = weights[n["k_norm"]].to(**f32).contiguous()
        # lambda in 32-bit, as the kernels' other scalars
        lq1, lk1, lq2, lk2 = (weights[n[r]].to(torch.float32) for r in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + torch.tensor(spec.lambda_init))
        if not math.isfinite(self.lam):
            raise ValueError("differential attention: lambda is not finite")
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, rt)
            if not hasattr(self.position, "frequencies"):
                raise TypeError("differential attention rotates by frequencies (a position part that computes its angles)")

    def cache_need(self):
        s = self.spec
        return PagedVectorNeed(s.k_size + s.v_size, s.window) if s.own_kv else None

    def forward(self, x, step, cache):
        s, ops = self.spec, self.rt.ops
        if cache.writable != s.own_kv:
            raise ValueError("differential attention: the schedule entry's cache does not fit the mixer "
                             "(a mixer without keys and values reads another entry's cache, and only such a mixer)")
        qkv = ops.linear(x, self.w_in)                      # [T, q_size (+ k_size + v_size)]
        freq = self.position.frequencies() if self.position is not None else None
        geometry = dict(heads=s.heads, kv_heads=s.kv_heads, key_dim=s.key_dim, value_dim=s.value_dim)
        ops.diff_qk_prepare(qkv, q_norm=self.q_norm, k_norm=self.k_norm, eps=s.qk_norm_eps or 0.0, frequencies=freq,
                            positions=step.positions, slot_mapping=cache.slot_mapping, cache=cache.kv,
                            write_kv=cache.writable, **geometry)
        attn = ops.diff_attention(qkv, cache=cache.kv, block_table=cache.block_table, step=step, scale=s.scale,
                                  lam=self.lam, out_scale=s.out_scale, norm_eps=s.norm_eps, window=s.window or 0,
                                  **geometry)
        return ops.linear(attn, self.w_o)
