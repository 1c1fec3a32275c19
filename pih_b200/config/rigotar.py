"""Typed configuration of the Rigotar design, read from its config.json keys.

A Rigotar model is a list of pre-norm layers, each with one of three mixers — a gated delta rule
(``"delta"``), a recurrent block with a real-gated linear recurrent unit (``"rglru"``) or attention over
a cached latent (``"latent_attention"``) — and a mixture-of-experts feed-forward or none.  config.json
holds::

    {"architecture": "Rigotar", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": ..., "mixer": {...sizes...}, "mlp": {...} | null, "weights_of": j (optional)}, ...]}

A layer with ``weights_of: j`` runs layer j's tensors with a cache or state of its own: it becomes a
second schedule entry of the same block.  Norm weights are single numbers; the residual stream is summed
in 32-bit.  Tensor names: ``embed``, ``head``, ``final.norm``, and ``l<i>.`` + ``norm1`` / ``norm2`` /
``mix.*`` / ``mlp.*`` (see the name tables of the part specs).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Tuple

from .registry import register_architecture
from .specs import (BlockSpec, GatedDeltaSpec, LatentAttentionSpec, ModelSpec, MoESpec, RGLRUSpec,
                    ScalarNormSpec, ScheduleEntry)

# Positions are not encoded, so the design has no longest context of its own; this bounds the engine's default.
DEFAULT_MAX_CONTEXT = 1 << 20


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ValueError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _number(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ValueError(f"config.json: {where}.{key} must be a positive number, got {v!r}")
    return float(v)


@register_architecture("Rigotar")
@dataclass(frozen=True)
class RigotarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[dict, ...]          # as in config.json, checked

    @classmethod
    def from_dict(cls, raw: dict) -> "RigotarConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ValueError("config.json: 'norm' must be an object with 'eps'")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  norm_eps=_number(norm, "eps", "norm"), layers=tuple(copy.deepcopy(layers)))
        cfg.model_spec()                      # every layer's keys and sizes are checked by building its spec
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}

    # -- layers -----------------------------------------------------------------
    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer ``i`` runs (itself unless it names another by ``weights_of``)."""
        seen = set()
        while True:
            layer = self.layers[i]
            if not isinstance(layer, dict):
                raise ValueError(f"config.json: layers[{i}] must be an object")
            j = layer.get("weights_of")
            if j is None:
                return i
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(self.layers) or j in seen or j == i:
                raise ValueError(f"config.json: layers[{i}].weights_of must name another layer, got {j!r}")
            seen.add(i)
            i = j

    def _mixer_spec(self, i: int):
        layer = self.layers[i]
        where = f"layers[{i}].mixer"
        kind, m = layer.get("type"), layer.get("mixer")
        if not isinstance(m, dict):
            raise ValueError(f"config.json: {where} must be an object")
        if kind == "delta":
            spec = GatedDeltaSpec(hidden=self.width, heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where),
                                  key_dim=_int(m, "dim", where), value_dim=_int(m, "vdim", where),
                                  conv_taps=_int(m, "conv", where), norm_eps=self.norm_eps)
            if spec.heads % spec.kv_heads:
                raise ValueError(f"config.json: {where}.heads must be a multiple of kv_heads")
            return spec
        if kind == "rglru":
            spec = RGLRUSpec(hidden=self.width, width=_int(m, "width", where), blocks=_int(m, "blocks", where),
                             conv_taps=_int(m, "conv", where))
            if spec.width % spec.blocks:
                raise ValueError(f"config.json: {where}.width must be a multiple of blocks")
            return spec
        if kind == "latent_attention":
            return LatentAttentionSpec(hidden=self.width, heads=_int(m, "heads", where), key_dim=_int(m, "dim", where),
                                       value_dim=_int(m, "vdim", where), latent_rank=_int(m, "kv_rank", where),
                                       scale=_number(m, "scale", where), norm_eps=self.norm_eps)
        raise ValueError(f"config.json: layers[{i}].type must be 'delta', 'rglru' or 'latent_attention', got {kind!r}")

    def _ffn_spec(self, i: int):
        f = self.layers[i].get("mlp")
        if f is None:
            return None
        where = f"layers[{i}].mlp"
        if not isinstance(f, dict) or f.get("kind") != "moe":
            raise ValueError(f"config.json: {where} must be null or an object of kind 'moe'")
        router, expert = f.get("router"), f.get("expert")
        if not isinstance(router, dict) or not isinstance(expert, dict):
            raise ValueError(f"config.json: {where} needs 'router' and 'expert' objects")
        spec = MoESpec(hidden=self.width, experts=_int(router, "experts", where + ".router"),
                       top=_int(router, "top", where + ".router"), intermediate=_int(expert, "ff", where + ".expert"))
        if spec.top > spec.experts:
            raise ValueError(f"config.json: {where}.router.top exceeds the number of experts")
        return spec

    # -- the model as parts --------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        norm = ScalarNormSpec(width=self.width, eps=self.norm_eps)
        blocks, block_of_layer, schedule = [], {}, []
        for i in range(len(self.layers)):
            src = self.weights_layer(i)
            if src == i:
                ffn = self._ffn_spec(i)
                block_of_layer[i] = len(blocks)
                blocks.append(BlockSpec(prefix=f"l{i}.", mixer=self._mixer_spec(i), ffn=ffn, norm_in=norm,
                                        norm_post=norm if ffn is not None else None,
                                        names={"norm_in": "norm1", "norm_post": "norm2"}))
        for i in range(len(self.layers)):
            schedule.append(ScheduleEntry(block_of_layer[self.weights_layer(i)]))
        spec = ModelSpec(vocab=self.vocab, hidden=self.width, blocks=tuple(blocks), schedule=tuple(schedule),
                         final_norm=norm, tie_embeddings=False, embed_name="embed", final_norm_prefix="final.norm",
                         head_name="head", max_positions=DEFAULT_MAX_CONTEXT, stream_dtype="float32")
        spec.validate()
        return spec
