"""Host-side logic of the Rigotar design without a GPU: configuration, tensor names, the paged cache of one vector
per token, and the real parts, cache manager and step function over stand-in kernels (tests/fake_ops.py) against
the plain float64 restatement."""
import copy

import pytest
import torch

import rigotar_models as rm
import traces
from fake_ops import FakeOps


def test_configuration_to_parts():
    from pih_b200.config import config_from_dict
    cfg = config_from_dict(copy.deepcopy(rm.R1))
    spec = cfg.model_spec()
    assert cfg.architecture == "Rigotar" and spec.stream_dtype == "float32" and not spec.tie_embeddings
    # four distinct layers, seven runs; a layer that names another runs that one's block with a cache of its own
    assert len(spec.blocks) == 4 and [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 0, 3]
    assert all(e.reads_cache_of is None for e in spec.schedule)
    assert [b.mixer.kind for b in spec.blocks] == ["gated_delta", "latent_attention", "rglru", "rglru"]
    assert spec.blocks[2].ffn is None and spec.blocks[2].norm_post is None
    assert (spec.blocks[0].ffn.experts, spec.blocks[0].ffn.top, spec.blocks[3].ffn.top) == (5, 2, 4)
    assert spec.blocks[1].mixer.scale == 0.3 and spec.blocks[1].mixer.latent_rank == 40
    assert config_from_dict(cfg.to_dict()) == cfg


def test_tensor_names():
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    names = expected_tensors(config_from_dict(copy.deepcopy(rm.R1)).model_spec())
    assert names["embed"].shape == (300, 96) and names["head"].shape == (300, 96) and names["final.norm"].shape == ()
    assert names["l0.norm1"].shape == () and names["l0.mix.q.conv"].shape == (64, 3) and names["l0.mix.A_log"].shape == (4,)
    assert names["l1.mix.uk"].shape == (48, 40) and names["l1.mix.sink"].shape == (3,) and names["l1.mix.g"].shape == (3, 96)
    assert names["l2.mix.ra"].shape == (4, 16, 16) and "l2.norm2" not in names and "l2.mlp.router" not in names
    assert names["l6.mlp.e3.down"].shape == (96, 24) and "l6.mlp.e4.down" not in names
    assert not any(n.startswith(("l3.", "l4.", "l5.")) for n in names)          # they run another layer's tensors


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][3].update(weights_of=3), "weights_of"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][2]["mixer"].update(blocks=5), "blocks"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors(change, message):
    from pih_b200.config import config_from_dict
    raw = copy.deepcopy(rm.R1)
    change(raw)
    with pytest.raises(ValueError, match=message):
        config_from_dict(raw)


def test_a_cache_of_one_vector_per_token():
    from pih_b200.cache import CacheManager
    from pih_b200.parts import PagedKVNeed, PagedVectorNeed, StateNeed
    needs = [PagedVectorNeed(40), StateNeed((7,), torch.float32), PagedVectorNeed(40), PagedKVNeed(2, 8), PagedVectorNeed(24)]
    m = CacheManager(needs, [None] * 5, page_size=4, num_pages=6, max_requests=2, device=torch.device("cpu"),
                     dtype=torch.float32)
    assert [tuple(g.kv.shape) for g in m.groups] == [(2, 6, 4, 40), (1, 6, 2, 2, 4, 8), (1, 6, 4, 24)]
    assert m.bytes_per_token() == 4 * (2 * 40 + 2 * 2 * 8 + 24)
    m.add_request("a")
    m.append("a", 9)
    m.commit("a")
    assert m.num_free_pages() == [3, 3, 3]
    view = m.view(2, [torch.zeros(1, 3, dtype=torch.int32)] * 3, [torch.zeros(9, dtype=torch.int32)] * 3)
    assert tuple(view.kv.shape) == (6, 4, 40) and view.writable and view.window is None
    m.release("a")
    m.check()


@pytest.mark.parametrize("name", ["R1", "R2"])
@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
def test_cut_invariance_with_stand_in_kernels(tmp_path, name, family):
    """Block tables, slot mappings, state slots and their reuse: the real parts and step function with torch
    stand-ins for the kernels agree with the plain implementation however the requests are cut."""
    from pih_b200.engine.factory import create_runner
    d = rm.write_model(tmp_path / name, rm.CONFIGS[name], seed=1, sigma=rm.SIGMA[name])
    requests = traces.make_requests(rm.CONFIGS[name]["vocab"], [19, 6, 23, 1, 12], seed=3)
    kw = dict(max_live=2, decode_tail=3, max_portion=7) if family == "mixed" else {}
    steps = getattr(traces, family)(requests, **kw)
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=4), max_requests=2,
                                            ops=FakeOps())
    got = traces.replay(runner, steps)
    for rid, ref in rm.plain_logits(d, requests).items():
        assert float((got[rid].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max()), (family, rid)
    cache.check()
    assert cache.slots.num_free == 2 and all(f == cache.num_pages for f in cache.num_free_pages())


def test_a_failed_step_leaves_the_states_as_they_were(tmp_path):
    """A step that raises after mixers have advanced their states is rolled back: the next try gives the same logits."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    d = rm.write_model(tmp_path / "m", rm.CONFIGS["R2"], seed=2, sigma=0.15)
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
    ref = rm.plain_logits(d, {"a": toks})["a"][-1]
    assert float((again[0].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max())
