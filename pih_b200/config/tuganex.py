"""Typed configuration of the Tuganex design, read from its config.json keys.

A Tuganex model is a list of layers whose norms sit on the sub-layers' OUTPUTS — ``x += norm1(mixer(x))``, then
``x += norm2(ff(x))`` — with one of two mixers: **retention** (``"retention"``: linear attention with a fixed decay
a head and a matrix state per sequence) or **differential attention** (``"attention"``: two softmax maps a head over
the same values, combined as ``a1 - lambda a2``), and a feed-forward that is dense (two biased matrices around the
xIELU activation) or a mixture of experts (softmax scores over all outputs, choice by score plus correction within
the best groups, identity experts, a shared expert behind a sigmoid gate) or absent.  config.json holds::

    {"architecture": "Tuganex", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "retention" | "attention", "mixer": {...}, "mlp": {...} | null}, ...]}

An attention layer with ``"kv_from": j`` has no key/value tensors and reads layer j's cache.  The residual stream is
summed in 32-bit.  Tensor names: ``embed``, ``head``, ``final.norm``, and ``l<i>.`` + ``norm1`` / ``norm2`` /
``mix.*`` / ``mlp.*`` (see the name tables of the part specs).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Tuple

from .registry import register_architecture
from .specs import (BiasedMLPSpec, BlockSpec, ComputedRopeSpec, DiffAttentionSpec, ModelSpec, NormSpec, RetentionSpec,
                    ScheduleEntry, ScoredMoESpec, SwiGLUSpec)

# The rotation's angles are computed from the position, so the design has no longest context of its own; this bounds
# the engine's default.
DEFAULT_MAX_CONTEXT = 1 << 20


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ValueError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _number(d: dict, key: str, where: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or (positive and v <= 0):
        raise ValueError(f"config.json: {where}.{key} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


def _object(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ValueError(f"config.json: {where}.{key} must be an object")
    return v


@register_architecture("Tuganex")
@dataclass(frozen=True)
class TuganexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[dict, ...]          # as in config.json, checked

    @classmethod
    def from_dict(cls, raw: dict) -> "TuganexConfig":
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
    def _rope(self, m: dict, where: str, head_dim: int):
        rot = m.get("rot")
        if rot is None:
            return None
        if not isinstance(rot, dict):
            raise ValueError(f"config.json: {where}.rot must be an object")
        dims = _int(rot, "dims", where + ".rot", minimum=2)
        if dims % 2 or dims > head_dim:
            raise ValueError(f"config.json: {where}.rot.dims must be even and at most dim ({head_dim}), got {dims}")
        return ComputedRopeSpec(head_dim=head_dim, rotary_dim=dims, theta=_number(rot, "base", where + ".rot"))

    def _kv_source(self, i: int):
        """The layer whose cache attention layer ``i`` reads (None: its own)."""
        m = self.layers[i]["mixer"]
        j = m.get("kv_from")
        if j is None:
            return None
        where = f"layers[{i}].mixer.kv_from"
        if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
            raise ValueError(f"config.json: {where} must name an earlier layer, got {j!r}")
        other = self.layers[j]
        if not isinstance(other, dict) or other.get("type") != "attention" or not isinstance(other.get("mixer"), dict) \
                or other["mixer"].get("kv_from") is not None:
            raise ValueError(f"config.json: {where} must name an attention layer with keys and values of its own")
        for key in ("kv_heads", "dim", "vdim", "rot"):
            if other["mixer"].get(key) != m.get(key):
                raise ValueError(f"config.json: {where}: layer {j}'s {key} differs from this layer's")
        return j

    def _mixer_spec(self, i: int):
        layer = self.layers[i]
        if not isinstance(layer, dict):
            raise ValueError(f"config.json: layers[{i}] must be an object")
        where = f"layers[{i}].mixer"
        kind, m = layer.get("type"), layer.get("mixer")
        if not isinstance(m, dict):
            raise ValueError(f"config.json: {where} must be an object")
        if kind == "retention":
            heads, dim = _int(m, "heads", where), _int(m, "dim", where)
            decays = m.get("decay")
            if not isinstance(decays, list) or len(decays) != heads or not all(
                    isinstance(d, (int, float)) and not isinstance(d, bool) and 0.0 < d <= 1.0 for d in decays):
                raise ValueError(f"config.json: {where}.decay must list one number in (0, 1] a head")
            return RetentionSpec(hidden=self.width, heads=heads, key_dim=dim, value_dim=_int(m, "vdim", where),
                                 decays=tuple(float(d) for d in decays), key_scale=dim ** -0.5, norm_eps=self.norm_eps,
                                 position=self._rope(m, where, dim))
        if kind == "attention":
            heads, kv_heads, dim = _int(m, "heads", where), _int(m, "kv_heads", where), _int(m, "dim", where)
            if heads % kv_heads:
                raise ValueError(f"config.json: {where}.heads must be a multiple of kv_heads")
            diff = _number(m, "diff", where, positive=False)
            return DiffAttentionSpec(hidden=self.width, heads=heads, kv_heads=kv_heads, key_dim=dim,
                                     value_dim=_int(m, "vdim", where), scale=_number(m, "scale", where),
                                     lambda_init=diff, out_scale=1.0 - diff, norm_eps=self.norm_eps,
                                     qk_norm_eps=self.norm_eps, position=self._rope(m, where, dim),
                                     own_kv=self._kv_source(i) is None)
        raise ValueError(f"config.json: layers[{i}].type must be 'retention' or 'attention', got {kind!r}")

    def _ffn_spec(self, i: int):
        f = self.layers[i].get("mlp")
        if f is None:
            return None
        where = f"layers[{i}].mlp"
        if not isinstance(f, dict):
            raise ValueError(f"config.json: {where} must be null or an object")
        if f.get("kind") == "dense":
            return BiasedMLPSpec(hidden=self.width, intermediate=_int(f, "ff", where))
        if f.get("kind") != "moe":
            raise ValueError(f"config.json: {where}.kind must be 'dense' or 'moe', got {f.get('kind')!r}")
        router, expert = _object(f, "router", where), _object(f, "expert", where)
        rw = where + ".router"
        experts, identity = _int(router, "experts", rw), _int(router, "identity", rw, 0) if "identity" in router else 0
        groups, keep = 1, 1
        if router.get("groups") is not None:
            g = _object(router, "groups", rw)
            groups, keep = _int(g, "count", rw + ".groups"), _int(g, "keep", rw + ".groups")
        shared = None
        if f.get("shared") is not None:
            shared = SwiGLUSpec(hidden=self.width, intermediate=_int(_object(f, "shared", where), "ff", where + ".shared"),
                                names={"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"})
        spec = ScoredMoESpec(hidden=self.width, experts=experts, identity=identity, top=_int(router, "top", rw),
                             intermediate=_int(expert, "ff", where + ".expert"), groups=groups, groups_keep=keep,
                             shared=shared)
        if spec.outputs % groups or keep > groups:
            raise ValueError(f"config.json: {rw}.groups must cut the {spec.outputs} router outputs into equal groups "
                             "and keep no more groups than there are")
        if spec.top > keep * (spec.outputs // groups):
            raise ValueError(f"config.json: {rw}.top exceeds the outputs of the groups that are kept")
        return spec

    # -- the model as parts --------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        norm = NormSpec(width=self.width, eps=self.norm_eps, weight_name="")
        blocks, schedule = [], []
        for i in range(len(self.layers)):
            mixer = self._mixer_spec(i)
            ffn = self._ffn_spec(i)
            blocks.append(BlockSpec(prefix=f"l{i}.", mixer=mixer, ffn=ffn, norm_in=norm,
                                    norm_post=norm if ffn is not None else None, arrangement="outnorm",
                                    names={"norm_in": "norm1", "norm_post": "norm2"}))
            source = self._kv_source(i) if self.layers[i].get("type") == "attention" else None
            schedule.append(ScheduleEntry(i, reads_cache_of=source))
        spec = ModelSpec(vocab=self.vocab, hidden=self.width, blocks=tuple(blocks), schedule=tuple(schedule),
                         final_norm=norm, tie_embeddings=False, embed_name="embed", final_norm_prefix="final.norm",
                         head_name="head", max_positions=DEFAULT_MAX_CONTEXT, stream_dtype="float32")
        spec.validate()
        return spec
