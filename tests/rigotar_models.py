"""Small Rigotar configurations with random weights for the tests, and their plain float64 logits.

Two configurations that differ from each other in every size: ``R1`` has every mixer twice (the second time through
``weights_of``), a layer without a feed-forward, one q/k head per value head, and experts of which one, two or all are
used; ``R2`` has one attention head, a convolution of ONE tap (no history), one diagonal block, grouped q/k heads and a
value size that is no power of two.
"""
import json
import os

import torch

import plain_rigotar


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


R1 = {"architecture": "Rigotar", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "layers": [
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 24, "conv": 3}, "mlp": _moe(5, 2, 40)},
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "vdim": 8, "kv_rank": 40, "scale": 0.3}, "mlp": _moe(3, 1, 56)},
    {"type": "rglru", "mixer": {"width": 64, "blocks": 4, "conv": 2}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "vdim": 8, "kv_rank": 40, "scale": 0.3}, "mlp": _moe(3, 1, 56),
     "weights_of": 1},
    {"type": "rglru", "mixer": {"width": 64, "blocks": 4, "conv": 2}, "mlp": None, "weights_of": 2},
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 24, "conv": 3}, "mlp": _moe(5, 2, 40), "weights_of": 0},
    {"type": "rglru", "mixer": {"width": 32, "blocks": 2, "conv": 4}, "mlp": _moe(4, 4, 24)},
]}
R2 = {"architecture": "Rigotar", "vocab": 257, "width": 64, "norm": {"eps": 1e-6}, "layers": [
    {"type": "latent_attention", "mixer": {"heads": 1, "dim": 8, "vdim": 8, "kv_rank": 16, "scale": 0.5}, "mlp": _moe(6, 3, 32)},
    {"type": "rglru", "mixer": {"width": 48, "blocks": 1, "conv": 5}, "mlp": _moe(2, 1, 72)},
    {"type": "delta", "mixer": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 40, "conv": 1}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 5, "dim": 24, "vdim": 12, "kv_rank": 72, "scale": 0.2}, "mlp": _moe(6, 3, 32)},
]}
CONFIGS = {"R1": R1, "R2": R2}
SIGMA = {"R1": 0.12, "R2": 0.15}


def single_layer(kind, mlp=None):
    """A model of ONE layer of the given mixer (a mechanism alone), sizes unlike R1's and R2's."""
    mixer = {"delta": {"heads": 2, "kv_heads": 1, "dim": 12, "vdim": 20, "conv": 4},
             "rglru": {"width": 40, "blocks": 5, "conv": 3},
             "latent_attention": {"heads": 2, "dim": 12, "vdim": 20, "kv_rank": 24, "scale": 0.4}}[kind]
    return {"architecture": "Rigotar", "vocab": 120, "width": 48, "norm": {"eps": 1e-5},
            "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}


def write_model(folder, raw, seed, sigma):
    from pih_b200.config import config_from_dict
    from pih_b200.weights import write_random_model
    return write_random_model(str(folder), config_from_dict(raw), seed=seed, sigma=sigma)


def load_plain(model_dir):
    from pih_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with SafetensorsFile(os.path.join(model_dir, "model.safetensors")) as sf:
        w = {n: sf.read_tensor(n).to(torch.float64) for n in sf.names()}
    return cfg, w


_LOGITS = {}


def plain_logits(model_dir, requests):
    """{rid: float64 logits [len, vocab]} of the plain implementation, cached per (folder, request)."""
    cfg, w = None, None
    out = {}
    for rid, toks in requests.items():
        key = (model_dir, tuple(toks))
        if key not in _LOGITS:
            if cfg is None:
                cfg, w = load_plain(model_dir)
            _LOGITS[key] = plain_rigotar.forward(cfg, w, toks)
        out[rid] = _LOGITS[key]
    return out
