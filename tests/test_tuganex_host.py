"""Host-side logic of the Tuganex design without a GPU: configuration, tensor names, the cache a layer shares with
another, and the real parts, cache manager and step function over stand-in kernels (tests/fake_ops.py) against the
plain float64 restatement."""
import copy

import pytest
import torch

import plain_tuganex as plain
import traces
import tuganex_models as tm
from fake_ops import FakeOps


def test_configuration_to_parts():
    from pih_b200.config import config_from_dict
    cfg = config_from_dict(copy.deepcopy(tm.T1))
    spec = cfg.model_spec()
    assert cfg.architecture == "Tuganex" and spec.stream_dtype == "float32" and not spec.tie_embeddings
    assert [b.arrangement for b in spec.blocks] == ["outnorm"] * 5
    assert [b.mixer.kind for b in spec.blocks] == ["retention", "diff_attention", "retention", "diff_attention", "diff_attention"]
    assert [e.reads_cache_of for e in spec.schedule] == [None, None, None, 1, None]
    assert spec.blocks[3].mixer.own_kv is False and spec.blocks[1].mixer.own_kv is True
    assert spec.blocks[2].ffn is None and spec.blocks[2].norm_post is None
    moe = spec.blocks[1].ffn
    assert (moe.experts, moe.identity, moe.top, moe.groups, moe.groups_keep, moe.shared.intermediate) == (7, 2, 2, 3, 2, 56)
    att = spec.blocks[4].mixer
    assert (att.lambda_init, att.scale, att.position.rotary_dim, att.position.theta) == (0.7, 0.2, 24, 1e6)
    assert abs(att.out_scale - 0.3) < 1e-12 and spec.blocks[0].mixer.key_scale == 0.25
    assert config_from_dict(cfg.to_dict()) == cfg


def test_tensor_names():
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    names = expected_tensors(config_from_dict(copy.deepcopy(tm.T1)).model_spec())
    assert names["embed"].shape == (311, 96) and names["final.norm"].shape == (96,) and names["l2.norm1"].shape == (96,)
    assert names["l0.mix.q"].shape == (48, 96) and names["l0.mix.v"].shape == (72, 96) and names["l0.mix.g"].shape == (72, 96)
    assert names["l1.mix.q"].shape == (128, 96) and names["l1.mix.k"].shape == (64, 96) and names["l1.mix.v"].shape == (48, 96)
    assert names["l1.mix.q.norm"].shape == (16,) and names["l1.mix.lk2"].shape == (16,) and names["l1.mix.o"].shape == (96, 96)
    assert "l3.mix.k" not in names and "l3.mix.v" not in names and "l3.mix.k.norm" not in names and "l3.mix.q.norm" in names
    assert names["l1.mlp.router"].shape == (9, 96) and names["l1.mlp.correction"].shape == (9,)
    assert "l1.mlp.e6.down" in names and "l1.mlp.e7.down" not in names and names["l1.mlp.shared.sg"].shape == (1, 96)
    assert names["l0.mlp.up.b"].shape == (136,) and names["l0.mlp.act"].shape == (2,) and "l2.norm2" not in names


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(dim=8), "kv_from"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=2), "groups"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors(change, message):
    from pih_b200.config import config_from_dict
    raw = copy.deepcopy(tm.T1)
    change(raw)
    with pytest.raises(ValueError, match=message):
        config_from_dict(raw)


def test_the_plain_implementation_cut_in_two():
    """The oracle itself: a sequence fed in two parts through its state gives what it gives whole."""
    cfg = copy.deepcopy(tm.T2)
    g = torch.Generator().manual_seed(0)
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    w = {n: torch.randn(i.shape, generator=g, dtype=torch.float64) * 0.2
         for n, i in expected_tensors(config_from_dict(cfg).model_spec()).items()}
    toks = traces.make_requests(257, [21], seed=1)["r0"]
    _, whole, _ = plain.model_layers(cfg, w, toks)
    _, a, st = plain.model_layers(cfg, w, toks[:13])
    _, b, _ = plain.model_layers(cfg, w, toks[13:], st)
    assert float((torch.cat([a, b]) - whole).abs().max()) < 1e-9


def test_plain_routing_by_hand():
    """Six outputs in three groups of which one is kept: the group of the largest corrected score wins although
    another group holds the largest score; weights are the scores themselves."""
    f = {"router": {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 1}}}
    w = {"m.router": torch.eye(6, dtype=torch.float64),
         "m.correction": torch.tensor([0.0, 0.0, 0.9, 0.0, -1.0, -2.0], dtype=torch.float64)}
    h = torch.tensor([[3.0, 0.0, 1.0, 0.5, 0.0, 0.0]], dtype=torch.float64)
    chosen, weights = plain.route(h, f, w, "m.")
    s = torch.softmax(h[0], dim=0)
    assert chosen.tolist() == [[2, 3]] and torch.allclose(weights[0], s[[2, 3]])
    # all corrected scores negative: the masked groups still lose (they count as minus infinity, not as zero)
    w["m.correction"] = torch.full((6,), -5.0, dtype=torch.float64)
    assert plain.route(h, f, w, "m.")[0].tolist() == [[0, 1]]


@pytest.mark.parametrize("name", ["T1", "T2"])
@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
def test_cut_invariance_with_stand_in_kernels(tmp_path, name, family):
    """Block tables, slot mappings, state slots, the cache that one layer reads of another, and their reuse: the real
    parts and step function with torch stand-ins for the kernels agree with the plain implementation however the
    requests are cut."""
    from pih_b200.engine.factory import create_runner
    d = tm.write_model(tmp_path / name, tm.CONFIGS[name], seed=1, sigma=tm.SIGMA[name])
    requests = traces.make_requests(tm.CONFIGS[name]["vocab"], [19, 6, 23, 1, 12], seed=3)
    kw = dict(max_live=2, decode_tail=3, max_portion=7) if family == "mixed" else {}
    steps = getattr(traces, family)(requests, **kw)
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=4), max_requests=2,
                                            ops=FakeOps())
    # layers that read another's cache keep none: one group tensor entry per layer with keys of its own
    assert sum(len(g.entries) for g in cache.groups) == sum(
        1 for layer in tm.CONFIGS[name]["layers"] if layer["type"] == "attention" and "kv_from" not in layer["mixer"])
    got = traces.replay(runner, steps)
    for rid, ref in tm.plain_logits(d, requests).items():
        assert float((got[rid].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max()), (family, rid)
    cache.check()
    assert cache.slots.num_free == 2 and all(f == cache.num_pages for f in cache.num_free_pages())


def test_a_failed_step_leaves_the_states_as_they_were(tmp_path):
    """A step that raises after the retention layers have advanced their states is rolled back."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    d = tm.write_model(tmp_path / "m", tm.CONFIGS["T2"], seed=2, sigma=0.15)
    toks = traces.make_requests(257, [14], seed=1)["r0"]
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4, max_cache_tokens=32, max_requests=1,
                                            ops=FakeOps())
    runner.step([StepEntry("a", toks[:9], [])])
    head = model.head
    model.head = None                                   # the head product fails, after every layer has run
    with pytest.raises(Exception):
        runner.step([StepEntry("a", toks[9:], [4])])
    model.head = head
    again = runner.step([StepEntry("a", toks[9:], [4])])
    ref = tm.plain_logits(d, {"a": toks})["a"][-1]
    assert float((again[0].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max())
