"""Small Tuganex configurations with random weights for the tests, and their plain float64 logits.

Two configurations that differ from each other in every size.  ``T1``: two key/value heads for four query heads, a
value size that is neither the key size nor twice it, a rotation over part of the keys, three groups of router
outputs of which two are kept, two identity experts, a shared expert, a layer without a feed-forward, and a layer that
reads another's keys and values.  ``T2``: one query head per key/value head, a rotation over the whole head, retention
that rotates only part of its keys and has a decay of exactly one, a router without groups, identity experts or
shared expert that chooses one expert, and two layers that read the same layer's cache.
"""
import copy
import json
import os

import torch

import plain_tuganex


def _rot(dims, base=10000.0):
    return {"dims": dims, "base": base}


def _att(heads, kv_heads, dim, vdim, rot, scale, diff, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale, "diff": diff}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, identity, top, ff, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


T1 = {"architecture": "Tuganex", "vocab": 311, "width": 96, "norm": {"eps": 1e-5}, "layers": [
    {"type": "retention", "mixer": {"heads": 3, "dim": 16, "vdim": 24, "rot": _rot(16), "decay": [0.9, 0.97, 0.995]},
     "mlp": {"kind": "dense", "ff": 136}},
    {"type": "attention", "mixer": _att(4, 2, 16, 24, _rot(8), 0.3, 0.4), "mlp": _moe(7, 2, 2, 40, groups=(3, 2), shared=56)},
    {"type": "retention", "mixer": {"heads": 2, "dim": 24, "vdim": 16, "rot": _rot(12, 500.0), "decay": [0.99, 0.8]}, "mlp": None},
    {"type": "attention", "mixer": _att(4, 2, 16, 24, _rot(8), 0.3, 0.4, kv_from=1), "mlp": {"kind": "dense", "ff": 72}},
    {"type": "attention", "mixer": _att(2, 1, 24, 40, _rot(24, 1e6), 0.2, 0.7), "mlp": _moe(7, 2, 2, 40, groups=(3, 2), shared=56)},
]}
T2 = {"architecture": "Tuganex", "vocab": 257, "width": 64, "norm": {"eps": 1e-6}, "layers": [
    {"type": "attention", "mixer": _att(3, 3, 8, 12, _rot(8), 0.5, 0.2), "mlp": _moe(5, 0, 1, 48)},
    {"type": "attention", "mixer": _att(3, 3, 8, 12, _rot(8), 0.5, 0.2, kv_from=0), "mlp": None},
    {"type": "retention", "mixer": {"heads": 5, "dim": 8, "vdim": 40, "rot": _rot(4), "decay": [1.0, 0.5, 0.9, 0.999, 0.75]},
     "mlp": _moe(6, 3, 3, 24, groups=(3, 1))},
    {"type": "attention", "mixer": _att(3, 3, 8, 12, _rot(8), 0.5, 0.2, kv_from=0), "mlp": {"kind": "dense", "ff": 100}},
]}
CONFIGS = {"T1": T1, "T2": T2}
SIGMA = {"T1": 0.12, "T2": 0.15}


def all_chosen(raw):
    """The configuration with every router output chosen (all groups kept): in bfloat16 the rounding of a router's input
    flips choices between outputs whose scores are close, and a flip changes that position outright, so a model with
    random weights cannot be held to a rounding bound.  With every output chosen the weights still come from the
    router; the choice itself is tested with decided scores."""
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if layer.get("mlp") and layer["mlp"]["kind"] == "moe":
            r = layer["mlp"]["router"]
            r["top"] = r["experts"] + r.get("identity", 0)
            if "groups" in r:
                r["groups"]["keep"] = r["groups"]["count"]
    return raw


def single_layer(kind, mlp=None, **changes):
    """A model of ONE layer of the given mixer (a mechanism alone), sizes unlike T1's and T2's."""
    mixer = {"retention": {"heads": 2, "dim": 12, "vdim": 20, "rot": _rot(6), "decay": [0.93, 0.999]},
             "attention": _att(6, 2, 12, 20, _rot(4), 0.4, 0.3)}[kind]
    mixer.update(changes)
    return {"architecture": "Tuganex", "vocab": 120, "width": 48, "norm": {"eps": 1e-5},
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
            _LOGITS[key] = plain_tuganex.model_layers(cfg, w, toks)[1]
        out[rid] = _LOGITS[key]
    return out


def random_config(seed):
    """A configuration drawn at random: sizes (also odd ones and ones that no fast kernel takes), the order of layers,
    which layers read whose keys and values, every constant."""
    import random
    rnd = random.Random(seed)
    width = rnd.choice([40, 56, 64, 72, 96, 136])
    layers, attention_shapes = [], {}
    for i in range(rnd.randint(3, 7)):
        if rnd.random() < 0.4:
            heads = rnd.choice([1, 2, 3, 4])
            dim = rnd.choice([4, 8, 12, 16, 20, 32, 64])
            mixer = {"heads": heads, "dim": dim, "vdim": rnd.choice([8, 12, 20, 32, 40, 64, 96]),
                     "rot": _rot(rnd.choice([d for d in (2, 4, 8, 12, 16, 32, 64) if d <= dim]), rnd.choice([10.0, 1e4, 1e6])),
                     "decay": [rnd.choice([1.0, 1.0 - 2.0 ** -rnd.randint(1, 10), rnd.uniform(0.3, 0.999)]) for _ in range(heads)]}
            layer = {"type": "retention", "mixer": mixer}
        else:
            sources = [j for j, shape in attention_shapes.items()]
            if sources and rnd.random() < 0.4:
                j = rnd.choice(sources)
                mixer = dict(attention_shapes[j], kv_from=j, heads=attention_shapes[j]["kv_heads"] * rnd.choice([1, 2, 3]),
                             scale=rnd.uniform(0.1, 0.6), diff=rnd.choice([0.0, 0.2, 0.5, 0.8, -0.3]))
            else:
                kv_heads = rnd.choice([1, 2, 3])
                dim = rnd.choice([4, 8, 12, 16, 24, 32, 40, 64])
                mixer = _att(kv_heads * rnd.choice([1, 2, 4]), kv_heads, dim, rnd.choice([8, 12, 16, 24, 40, 64, 72, 128, 136]),
                             _rot(rnd.choice([d for d in (2, 4, 8, 12, 16, 24, 32, 40, 64) if d <= dim]), rnd.choice([10.0, 1e4, 1e6])),
                             rnd.uniform(0.1, 0.6), rnd.choice([0.0, 0.2, 0.5, 0.8, -0.3]))
                attention_shapes[i] = {k: mixer[k] for k in ("kv_heads", "dim", "vdim", "rot")}
            layer = {"type": "attention", "mixer": mixer}
        kind = rnd.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            layer["mlp"] = {"kind": "dense", "ff": rnd.choice([24, 50, 64, 130])}
        elif kind == "moe":
            groups = rnd.choice([None, (2, 1), (3, 2), (4, 4), (4, 1)])
            count = groups[0] if groups else 1
            outputs = count * rnd.randint(1, 4)
            identity = rnd.randint(0, outputs - 1)
            kept = (outputs // count) * (groups[1] if groups else 1)
            layer["mlp"] = _moe(outputs - identity, identity, rnd.randint(1, kept), rnd.choice([8, 24, 36, 64]), groups=groups,
                                shared=rnd.choice([None, 16, 40]))
        else:
            layer["mlp"] = None
        layers.append(layer)
    return {"architecture": "Tuganex", "vocab": rnd.choice([97, 256, 300]), "width": width,
            "norm": {"eps": rnd.choice([1e-5, 1e-6])}, "layers": layers}
