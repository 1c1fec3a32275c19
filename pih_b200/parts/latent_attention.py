"""Causal attention over a cached latent, without positions, as a mixer.

Per token one vector ``c = rmsnorm(W_down h) * w`` of ``latent_rank`` numbers is cached; head h's key is
``K_h c`` and its value ``V_h c``.  Scores are ``(q_h . k) * scale`` over all earlier tokens and the token
itself.  With ``sink`` the softmax denominator also holds ``exp(sink_h)``: a learned logit per head without a key
or a value.  With ``gated`` head h's output is multiplied by ``sigmoid(G h)_h``.  Then the output projection.

Keys and values are never formed: both are linear in c, so ``K_h`` is folded into the query
(``q'_h = K_h^T q_h``, a batched product) and ``V_h`` is applied to the weighted sum of latents (another batched
product); the attention kernel sees queries of ``latent_rank`` numbers and ONE cached vector per token that serves
every head as key and as value.  Scores, weights and sums are 32-bit.
"""
from __future__ import annotations

import torch

from .registry import PagedVectorNeed, Runtime, TensorInfo, register_mixer
from ._bind import bind_matrix


@register_mixer("latent_attention")
class LatentAttention:
    pad_safe = True            # rows without a request are skipped; a padding row's cache slot is left alone

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        H, D, V, R = spec.heads, spec.key_dim, spec.value_dim, spec.latent_rank
        out = {n["q"]: TensorInfo((H * D, spec.hidden)), n["down"]: TensorInfo((R, spec.hidden)),
               n["down_norm"]: TensorInfo((R,), "one_plus_normal"), n["up_k"]: TensorInfo((H * D, R)),
               n["up_v"]: TensorInfo((H * V, R)), n["o"]: TensorInfo((spec.hidden, H * V))}
        if spec.sink:
            out[n["sink"]] = TensorInfo((H,), "unit_normal")
        if spec.gated:
            out[n["gate"]] = TensorInfo((H, spec.hidden))
        return out

    def __init__(self, spec, weights, rt: Runtime):
        self.spec, self.rt = spec, rt
        n = spec.names
        H, D, V, R = spec.heads, spec.key_dim, spec.value_dim, spec.latent_rank
        stacked = [weights[n["q"]], weights[n["down"]]] + ([weights[n["gate"]]] if spec.gated else [])
        self.w_in = bind_matrix(torch.cat(stacked, dim=0), rt)                                 # [q | latent | gate]
        # q'_h = q_h . K_h with K_h [D, R]: as a product with rows of outputs, the weight is K_h^T [R, D]
        self.w_fold_k = bind_matrix(weights[n["up_k"]].reshape(H, D, R).transpose(1, 2), rt)   # [H, R, D]
        self.w_up_v = bind_matrix(weights[n["up_v"]].reshape(H, V, R), rt)                     # [H, V, R]
        self.w_o = bind_matrix(weights[n["o"]], rt)
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.down_norm = weights[n["down_norm"]].to(**f32).contiguous()
        self.sink = weights[n["sink"]].to(**f32).contiguous() if spec.sink else None

    def cache_need(self):
        return PagedVectorNeed(self.spec.latent_rank)

    def forward(self, x, step, cache):
        s, ops = self.spec, self.rt.ops
        H, D, V, R = s.heads, s.key_dim, s.value_dim, s.latent_rank
        T = x.shape[0]
        proj = ops.linear(x, self.w_in)                                     # [T, H D + R (+ H)]
        ops.latent_write(proj[:, H * D:H * D + R], self.down_norm, s.norm_eps, cache.kv, cache.slot_mapping)
        q_lat = ops.linear_batched(proj[:, :H * D].view(T, H, D), self.w_fold_k)                # [T, H, R]
        gate = proj[:, H * D + R:] if s.gated else None
        o_lat = ops.latent_attention(q_lat, gate=gate, sink=self.sink, cache=cache.kv, block_table=cache.block_table,
                                     step=step, scale=s.scale, window=cache.window or 0)
        heads_out = ops.linear_batched(o_lat, self.w_up_v)                                      # [T, H, V]
        return ops.linear(heads_out.view(T, H * V), self.w_o)
