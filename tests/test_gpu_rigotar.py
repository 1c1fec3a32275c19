"""The Rigotar design on the GPU against the plain float64 restatement (tests/plain_rigotar.py): each mechanism
alone, every way of cutting requests into steps, batches against requests alone, pages and state slots that are
used again, keys that must be found far back / at page borders / among the first tokens, long decoding, and greedy
generation through the engine's own entry point."""
import copy
import math
from types import SimpleNamespace

import pytest
import torch

import plain_rigotar as plain
import rigotar_models as rm
import traces

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {n: rm.write_model(tmp_path_factory.mktemp(f"rigotar_{n}"), raw, seed=5 + i, sigma=rm.SIGMA[n])
           for i, (n, raw) in enumerate(rm.CONFIGS.items())}
    for i, (n, raw) in enumerate(rm.CONFIGS.items()):
        out[n + "-all"] = rm.write_model(tmp_path_factory.mktemp(f"rigotar_{n}_all"), _all_experts(raw), seed=5 + i,
                                         sigma=rm.SIGMA[n])
    return out


def _check(got, truth, dtype, what):
    """Per position: the error of the logits (mean taken off, root mean square over the vocabulary) relative to the
    logits' spread.  32-bit: every position of every request.  bfloat16 (models whose routers choose every expert,
    see ``_all_experts``), over the positions of all requests together: the median within rounding, and at most one
    position in ten beyond three times that."""
    errs = []
    for rid, ref in truth.items():
        g = got[rid].double()
        assert g.shape == ref.shape, (what, rid)
        d = g - ref
        d = d - d.mean(dim=1, keepdim=True)
        err = d.pow(2).mean(dim=1).sqrt() / ref.std()
        errs.append(err)
        if dtype == "float32":
            worst = int(err.argmax())
            assert float(err.max()) < 5e-5, f"{what} {rid}: error {float(err.max()):.3e} of the logits' spread at position {worst}"
    if dtype != "float32":
        err = torch.cat(errs)
        over = int((err > 0.09).sum())
        assert float(err.median()) < 0.03 and over <= len(err) // 10, \
            f"{what}: median {float(err.median()):.3e}, {over} of {len(err)} positions beyond 0.09, worst {float(err.max()):.3e}"


def _all_experts(raw):
    """The configuration with every expert chosen.  In bfloat16 the rounding of a router's input flips choices between
    experts whose logits are close; a flip changes that position outright and, through the recurrent states, the
    positions after it, so a model with random weights cannot be held to a rounding bound.  With every expert chosen
    the weights still come from the router; the choice itself is tested in bfloat16 by
    ``test_routed_experts_with_decided_logits``."""
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if layer.get("mlp"):
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


LENGTHS = {"R1": [70, 45, 131, 33, 64, 50, 1, 2], "R2": [65, 33, 97, 128, 80, 3, 35, 66]}
FAMILIES = ["whole", "tail_decode", "portions", "mixed"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["R1", "R2"])
@pytest.mark.parametrize("family", FAMILIES)
def test_cuttings_against_the_plain_implementation(dirs, name, dtype, family):
    """Whole prompts; most of a prompt and then token by token; portions down to two tokens; up to three live
    requests mixed, with a pool so small and so few state slots that pages and slots are used again."""
    from pih_b200.engine.factory import create_runner
    requests = traces.make_requests(rm.CONFIGS[name]["vocab"], LENGTHS[name], seed=21)
    kw = dict(max_live=3) if family == "mixed" else {}
    steps = getattr(traces, family)(requests, **kw)
    folder = dirs[name] if dtype == "float32" else dirs[name + "-all"]
    _, model, cache, runner = create_runner(folder, dtype, page_size=16 if name == "R1" else 8,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=16), max_requests=3)
    got = traces.replay(runner, steps)
    model.rt.ops.check_errors()
    _check(got, rm.plain_logits(folder, requests), dtype, f"{name} {family} {dtype}")
    cache.check()
    assert all(f == cache.num_pages for f in cache.num_free_pages()) and cache.slots.num_free == 3
    if family == "mixed":
        assert all(g.pool.pages_handed_out > g.pool.num_pages for g in cache.groups)


@pytest.mark.parametrize("kind", ["delta", "rglru", "latent_attention"])
def test_a_mixer_alone(tmp_path, kind):
    """One layer of one mixer and no feed-forward, whole and token by token."""
    from pih_b200.engine.factory import create_runner
    d = rm.write_model(tmp_path / kind, rm.single_layer(kind), seed=3, sigma=0.2)
    requests = traces.make_requests(120, [40, 7], seed=2)
    truth = rm.plain_logits(d, requests)
    for family in ("whole", "tail_decode"):
        _, model, cache, runner = create_runner(d, "float32", page_size=8, max_cache_tokens=64, max_requests=2)
        _check(traces.replay(runner, getattr(traces, family)(requests)), truth, "float32", f"{kind} {family}")
        model.rt.ops.check_errors()


def test_the_experts_alone(tmp_path):
    """The routed feed-forward behind a mixer, against the same model without it: the difference is the experts'."""
    from pih_b200.engine.factory import create_runner
    raw = rm.single_layer("rglru", mlp={"kind": "moe", "router": {"experts": 7, "top": 3}, "expert": {"ff": 36}})
    d = rm.write_model(tmp_path / "moe", raw, seed=4, sigma=0.2)
    requests = traces.make_requests(120, [50, 9], seed=5)
    _, model, cache, runner = create_runner(d, "float32", page_size=8, max_cache_tokens=64, max_requests=2)
    _check(traces.replay(runner, traces.whole(requests)), rm.plain_logits(d, requests), "float32", "experts")
    # the router does route: over these rows more than `top` experts are chosen
    cfg, w = rm.load_plain(d)
    x = w["embed"][torch.tensor(requests["r0"])]
    h = plain.scalar_norm(x + plain.rglru_mixer(plain.scalar_norm(x, w["l0.norm1"], 1e-5), w, "l0.mix.", raw["layers"][0]["mixer"]),
                          w["l0.norm2"], 1e-5)
    assert len(set(torch.topk(h @ w["l0.mlp.router"].T, 3).indices.flatten().tolist())) > 3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_with_decided_logits(dtype):
    """The routed feed-forward as an op, with router logits given: distinct integers, so that no rounding decides a
    choice; every row's output against the plain weighted sum of its chosen experts."""
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    g = torch.Generator().manual_seed(6)
    rows, hidden, ff, experts, top = 300, 40, 72, 9, 3
    x = (torch.randn(rows, hidden, generator=g) * 0.8).to(dtype)
    wg, wu = [(torch.randn(experts, ff, hidden, generator=g) * 0.2).to(dtype) for _ in range(2)]
    wd = (torch.randn(experts, hidden, ff, generator=g) * 0.2).to(dtype)
    logits = torch.stack([torch.randperm(experts, generator=g).float() * 0.7 - 2.0 for _ in range(rows)])
    wgu = torch.cat([wg, wu], dim=1).to(DEV).contiguous()
    got = ops.moe_experts(x.to(DEV), logits.to(DEV), wgu, wd.to(DEV).contiguous(), top).double().cpu()
    ops.check_errors()
    # few rows take the kernel that streams the chosen experts' rows; many rows in bfloat16 the library's grouped product
    few = ops.moe_experts(x[:5].to(DEV), logits[:5].to(DEV), wgu, wd.to(DEV).contiguous(), top).double().cpu()
    ops.check_errors()
    w = {"router": None}
    val, idx = torch.topk(logits.double(), top, dim=-1)
    wt = torch.softmax(val, dim=-1)
    ref = torch.zeros(rows, hidden, dtype=F64)
    for t in range(rows):
        for j in range(top):
            e = int(idx[t, j])
            a = plain.silu(x[t].double() @ wg[e].double().T) * (x[t].double() @ wu[e].double().T)
            ref[t] += wt[t, j] * (a @ wd[e].double().T)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - ref).abs().max()) < tol * float(ref.abs().max())
    assert float((few - ref[:5]).abs().max()) < tol * float(ref.abs().max())
    assert len(set(idx.flatten().tolist())) == experts                    # every expert has rows, unequally many


def test_batches_against_each_request_alone(dirs):
    """Unequal requests side by side in one step — a long portion, a short one, single tokens — give each request
    the bits it gets alone (32-bit: every reduction has an order fixed by the row)."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    name = "R1"
    requests = traces.make_requests(rm.CONFIGS[name]["vocab"], [61, 18, 40, 9], seed=8)
    alone = {}
    for rid, toks in requests.items():
        _, _, _, runner = create_runner(dirs[name], "float32", page_size=16, max_cache_tokens=128, max_requests=1)
        alone[rid] = traces.replay(runner, traces.whole({rid: toks}))[rid]
    _, model, cache, runner = create_runner(dirs[name], "float32", page_size=16, max_cache_tokens=256, max_requests=4)
    cuts = {"r0": [33, 27, 1], "r1": [1, 16, 1], "r2": [2, 37, 1], "r3": [7, 1, 1]}
    got = {rid: [] for rid in requests}
    at = {rid: 0 for rid in requests}
    for i in range(3):
        entries = []
        for rid, toks in requests.items():
            n = cuts[rid][i]
            entries.append(StepEntry(rid, toks[at[rid]:at[rid] + n], list(range(n))))
            at[rid] += n
        logits = runner.step(entries)
        j = 0
        for e in entries:
            got[e.rid].append(logits[j:j + len(e.tokens)].clone())
            j += len(e.tokens)
    model.rt.ops.check_errors()
    for rid in requests:
        assert float((torch.cat(got[rid]).cpu() - alone[rid]).abs().max()) < 1e-6, rid


def _step(positions, request_of_row, cu_q, slots):
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(positions=t(positions), request_of_row=t(request_of_row), cu_q=t(cu_q), state_slots=t(slots),
                           num_requests=len(slots))


def _plain_latent_rows(q, latents, sink, gate, scale, window=0):
    """q [heads, rank] at the LAST position of ``latents`` [n, rank] (float64): the weighted sum of latents a head."""
    n = latents.shape[0]
    lat = latents[max(0, n - window):] if window else latents
    s = (q @ lat.T) * scale
    top = torch.maximum(s.max(dim=1).values, sink) if sink is not None else s.max(dim=1).values
    e = torch.exp(s - top[:, None])
    denom = e.sum(1) + (torch.exp(sink - top) if sink is not None else 0.0)
    out = (e / denom[:, None]) @ lat
    return out * torch.sigmoid(gate)[:, None] if gate is not None else out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank", [40, 64, 384])        # in bf16: the kernel that cuts the keys; the tensor-core kernel (384: in two stretches of columns)
@pytest.mark.parametrize("needle", [0, 1, 15, 16, 17, 250, 299])
def test_latent_attention_finds_one_key_among_hundreds(needle, rank, dtype):
    """300 cached latents of which ONE matches the query (its score stands out by construction): the first tokens, both
    sides of a page border, far back, and the row itself.  Random inputs would average such a key away."""
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    g = torch.Generator().manual_seed(needle)
    heads, n, page = 3, 300, 16
    lat = torch.randn(n, rank, generator=g, dtype=F64) * 0.3
    lat[needle] = torch.randn(rank, generator=g, dtype=F64)
    q = torch.randn(heads, rank, generator=g, dtype=F64) * 0.2 + 4.0 * lat[needle][None, :]
    lat, q = lat.to(dtype).double(), q.to(dtype).double()            # what the kernel reads
    sink = torch.tensor([0.5, -1.0, 2.0], dtype=F64)
    gate = torch.tensor([0.3, -0.7, 1.5], dtype=F64).to(dtype).double()
    pages = list(range(n // page + 1))[::-1]                           # pages in an order of their own
    cache = torch.zeros(len(pages) + 2, page, rank, dtype=dtype, device=DEV)
    for j in range(n):
        cache[pages[j // page], j % page] = lat[j].to(dtype)
    table = torch.tensor([pages], dtype=torch.int32, device=DEV)
    step = _step([n - 1], [0], [0, 1], [0])
    got = ops.latent_attention(q.to(dtype).to(DEV).view(1, heads, rank).contiguous(), gate=gate.to(dtype).to(DEV).view(1, heads),
                               sink=sink.float().to(DEV), cache=cache, block_table=table, step=step, scale=0.5)
    ops.check_errors()
    ref = _plain_latent_rows(q, lat, sink, gate, 0.5)
    weight_of_needle = torch.softmax((q @ lat.T) * 0.5, dim=1)[:, needle]
    assert float(weight_of_needle.min()) > 0.5                        # the key does stand out
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got[0].double().cpu() - ref).abs().max()) < tol * float(ref.abs().max())


@pytest.mark.parametrize("rank, heads", [(64, 5), (128, 18), (384, 3)])
def test_latent_attention_portions_of_several_requests(rank, heads):
    """Portions of three requests in one step — one deep in its context, one from its first token, one of five rows —
    on the tensor-core kernel, whose blocks are four consecutive rows of ONE request: every row against the plain
    softmax over its own request's latents up to its own position."""
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    g = torch.Generator().manual_seed(rank)
    page = 16
    starts, counts = [300, 0, 37], [70, 131, 5]
    lats = [(torch.randn(st + n, rank, generator=g, dtype=F64) * 0.5).bfloat16() for st, n in zip(starts, counts)]
    pages_of, next_page = [], 0
    for lat in lats:
        n_pages = -(-lat.shape[0] // page)
        pages_of.append(list(range(next_page, next_page + n_pages))[::-1])
        next_page += n_pages
    cache = torch.zeros(next_page + 1, page, rank, dtype=torch.bfloat16, device=DEV)
    width = max(len(p) for p in pages_of)
    table = torch.full((3, width), -1, dtype=torch.int32)
    for r, (lat, pages) in enumerate(zip(lats, pages_of)):
        table[r, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        for j in range(lat.shape[0]):
            cache[pages[j // page], j % page] = lat[j].to(DEV)
    T = sum(counts)
    q = (torch.randn(T, heads, rank, generator=g, dtype=F64) * 0.6).bfloat16()
    gate = (torch.randn(T, heads, generator=g, dtype=F64)).bfloat16()
    sink = torch.randn(heads, generator=g, dtype=F64).float()
    positions, request_of_row, cu = [], [], [0]
    for r, (st, n) in enumerate(zip(starts, counts)):
        positions += list(range(st, st + n))
        request_of_row += [r] * n
        cu.append(cu[-1] + n)
    step = _step(positions, request_of_row, cu, [0, 1, 2])
    assert T > ops.latent_mma_rows_above
    got = ops.latent_attention(q.to(DEV).contiguous(), gate=gate.to(DEV), sink=sink.to(DEV), cache=cache,
                               block_table=table.to(DEV), step=step, scale=0.3).double().cpu()
    ops.check_errors()
    worst = 0.0
    for t in range(T):
        r, p = request_of_row[t], positions[t]
        ref = _plain_latent_rows(q[t].double(), lats[r][:p + 1].double(), sink.double(), gate[t].double(), 0.3)
        worst = max(worst, float((got[t] - ref).abs().max()) / float(ref.abs().max()))
    assert worst < 2e-2, worst


def test_latent_attention_sink_and_window_edges():
    """The sink alone in the denominator (one key), no sink, and a window whose edge the standing-out key is just
    inside and just outside of."""
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    g = torch.Generator().manual_seed(1)
    heads, rank, n, page = 2, 24, 90, 8
    lat = torch.randn(n, rank, generator=g, dtype=F64) * 0.3
    cache = torch.zeros(n // page + 1, page, rank, dtype=torch.float32, device=DEV)
    cache.view(-1, rank)[:n] = lat.float().to(DEV)
    table = torch.arange(n // page + 1, dtype=torch.int32, device=DEV).view(1, -1)
    lat = lat.float().double()

    def run(q, last, sink, window):
        step = _step([last], [0], [0, 1], [0])
        out = ops.latent_attention(q.float().to(DEV).view(1, heads, rank).contiguous(), gate=None,
                                   sink=None if sink is None else sink.float().to(DEV), cache=cache, block_table=table,
                                   step=step, scale=1.0, window=window)
        ops.check_errors()
        return out[0].double().cpu()

    q = torch.randn(heads, rank, generator=g, dtype=F64).float().double()
    sink = torch.tensor([3.0, -2.0], dtype=F64)
    # one key and a sink: the output is the key's latent times 1 / (1 + exp(sink - score))
    for s in (sink, None):
        assert float((run(q, 0, s, 0) - _plain_latent_rows(q, lat[:1], s, None, 1.0)).abs().max()) < 1e-6
    needle, last = 40, 89
    q = q * 0.1 + 6.0 * lat[needle][None, :]
    inside = run(q, last, sink, last - needle + 1)                     # the window's oldest key is the needle
    outside = run(q, last, sink, last - needle)                        # ... is the one after it
    assert float((inside - _plain_latent_rows(q, lat[:last + 1], sink, None, 1.0, window=last - needle + 1)).abs().max()) < 1e-5
    assert float((outside - _plain_latent_rows(q, lat[:last + 1], sink, None, 1.0, window=last - needle)).abs().max()) < 1e-5
    assert float((inside - outside).abs().max()) > 0.1


def test_delta_rule_recalls_a_value_written_long_ago():
    """With a decay of (almost) one, a write strength of one and orthogonal unit keys, the state returns the value
    that was written under a key 200 tokens earlier, across steps: a lost or re-zeroed state would return zero."""
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    heads, kv_heads, D, V, n = 2, 1, 32, 20, 220
    g = torch.Generator().manual_seed(3)
    keys = torch.linalg.qr(torch.randn(D, D, generator=g, dtype=F64)).Q          # orthonormal rows
    k = keys[torch.arange(n) % D]                                                 # key i again every D tokens
    v = torch.randn(n, heads, V, generator=g, dtype=F64)
    q = k.clone()
    qkv = torch.cat([q, k, v.reshape(n, heads * V)], dim=1).float().to(DEV).contiguous()
    ba = torch.cat([torch.full((n, heads), 30.0), torch.full((n, heads), -30.0)], dim=1).float().to(DEV)   # beta = 1, decay = 1
    zeros = torch.zeros(heads, dtype=torch.float32, device=DEV)
    state = torch.zeros(2, heads * D * V, dtype=torch.float32, device=DEV)
    outs, at = [], 0
    for cut in (7, 100, 1, 1, 2, 109):                                           # the state is carried over these steps
        step = _step([0] * cut, [0] * cut, [0, 0, cut], [-1, 1])                  # (a request of padding in front)
        outs.append(ops.gated_delta_rule(qkv[at:at + cut], ba[at:at + cut], decay_log=zeros, decay_bias=zeros, state=state,
                                         step=step, heads=heads, kv_heads=kv_heads, key_dim=D, value_dim=V,
                                         unit_eps=1e-6, q_scale=1.0))
        at += cut
    ops.check_errors()
    out = torch.cat(outs).double().cpu()
    # reading with key i right after writing v under it returns v (delta rule with beta = 1 replaces the old value)
    assert float((out - v).abs().max()) < 1e-4
    assert float(state[0].abs().max()) == 0.0                                     # the other slot was never touched
    S = state[1].view(heads, D, V).double().cpu()
    for i in (0, 5, 31):                                                          # and the state still holds each key's LAST value
        last = max(t for t in range(n) if t % D == i)
        assert float((S.transpose(1, 2) @ keys[i] - v[last]).abs().max()) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, vdim", [(16, 24), (32, 32), (48, 40), (64, 70), (128, 128), (256, 64), (40, 8)])
def test_delta_rule_kernels_of_every_key_size(dim, vdim, dtype):
    """The register kernel's instances (key sizes 16 to 256) and the shared-memory kernel (the other sizes), value sizes
    that are no multiple of a block's 32 columns, two requests of unequal length in two steps, against plain loops."""
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    g = torch.Generator().manual_seed(dim + vdim)
    heads, kv_heads = 4, 2
    lens = [37, 9]
    T = sum(lens)
    QK, VS = kv_heads * dim, heads * vdim
    qkv = (torch.randn(T, 2 * QK + VS, generator=g) * 0.7).to(dtype)
    ba = torch.randn(T, 2 * heads, generator=g).to(dtype)
    decay_log = torch.randn(heads, generator=g) * 0.5 - 1.0
    decay_bias = torch.randn(heads, generator=g) * 0.5
    state = torch.zeros(3, heads * dim * vdim + 5, dtype=torch.float32, device=DEV)
    kw = dict(decay_log=decay_log.to(DEV), decay_bias=decay_bias.to(DEV), state=state, heads=heads, kv_heads=kv_heads,
              key_dim=dim, value_dim=vdim, unit_eps=1e-6, q_scale=dim ** -0.5)
    # step 1: the first 20 rows of request 0 and all of request 1; step 2: the rest of request 0
    rows1 = list(range(20)) + list(range(lens[0], T))
    rows2 = list(range(20, lens[0]))
    sel1, sel2 = torch.tensor(rows1), torch.tensor(rows2)
    out1 = ops.gated_delta_rule(qkv[sel1].to(DEV).contiguous(), ba[sel1].to(DEV).contiguous(),
                                step=_step([0] * len(rows1), [0] * len(rows1), [0, 20, len(rows1)], [2, 0]), **kw)
    out2 = ops.gated_delta_rule(qkv[sel2].to(DEV).contiguous(), ba[sel2].to(DEV).contiguous(),
                                step=_step([0] * len(rows2), [0] * len(rows2), [0, len(rows2)], [2]), **kw)
    ops.check_errors()
    got = torch.zeros(T, heads, vdim, dtype=F64)
    got[sel1] = out1.double().cpu()
    got[sel2] = out2.double().cpu()
    x = qkv.double()
    q = x[:, :QK].view(T, kv_heads, dim)
    k = x[:, QK:2 * QK].view(T, kv_heads, dim)
    v = x[:, 2 * QK:].view(T, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(ba.double()[:, :heads])
    dec = torch.exp(-torch.exp(decay_log.double()) * plain.softplus(ba.double()[:, heads:] + decay_bias.double()))
    ref = torch.zeros(T, heads, vdim, dtype=F64)
    start = 0
    for n in lens:
        for h in range(heads):
            S = torch.zeros(dim, vdim, dtype=F64)
            for t in range(start, start + n):
                kk, qq = k[t, h // 2], q[t, h // 2]
                S = dec[t, h] * S
                S = S + torch.outer(kk, beta[t, h] * (v[t, h] - S.T @ kk))
                ref[t, h] = S.T @ qq
        start += n
    tol = 2e-5 if dtype == torch.float32 else 1e-4            # (the inputs are what the kernel read; only the arithmetic differs)
    assert float((got - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))
    assert float(state[1].abs().max()) == 0.0 and float(state[:, -5:].abs().max()) == 0.0      # nothing beyond the matrices


def test_rglru_keeps_a_state_over_a_thousand_tokens():
    """A channel with a decay next to one: an input at token 0 is still there 1500 tokens later, fed in portions and
    token by token, where a decay rounded to 32-bit before it multiplies would have lost a few percent of it."""
    from pih_b200.kernels import get_ops
    ops = get_ops(torch.device(DEV))
    W, n = 8, 1500
    lam = torch.tensor([-14.0, -10.0, -6.0, -3.0, 0.0, 1.0, 2.0, 3.0], dtype=F64)
    u = torch.zeros(n, W, dtype=F64)
    u[0] = 1.0
    u[700] = -0.5
    gates = torch.zeros(n, 1, 2 * W, dtype=F64)                                  # r = i = sigmoid(0) = 0.5
    y_pre = torch.full((n, W), 2.0, dtype=F64)
    f = lambda t: t.float().to(DEV).contiguous()
    zeros = torch.zeros(W, dtype=torch.float32, device=DEV)
    state = torch.zeros(1, W, dtype=torch.float32, device=DEV)
    outs, at = [], 0
    for cut in [640, 2, 63] + [1] * 40 + [755]:
        step = _step([0] * cut, [0] * cut, [0, cut], [0])
        outs.append(ops.rglru_scan(f(u[at:at + cut]), f(gates[at:at + cut]), f(y_pre[at:at + cut]), y_bias=zeros, r_bias=zeros,
                                   i_bias=zeros, lam=f(lam), decay_scale=8.0, state=state, step=step, blocks=1))
        at += cut
    ops.check_errors()
    log_a = -8.0 * 0.5 * plain.softplus(lam)
    S, ref = torch.zeros(W, dtype=F64), []
    for t in range(n):
        a = torch.exp(log_a)
        S = a * S + torch.sqrt(1 - a * a) * 0.5 * u[t]
        ref.append(S * plain.gelu_tanh(y_pre[t]))
    ref = torch.stack(ref)
    got = torch.cat(outs).double().cpu()
    assert float(ref[-1, 0].abs()) > 1e-4                                        # the slowest channel still remembers
    # (a constant decay rounds the same way at every step: the error of the slowest channel grows with the steps)
    assert float(((got - ref).abs().max(dim=0).values / ref.abs().max(dim=0).values).max()) < 1e-4
    assert float((got[-1, 0] - ref[-1, 0]).abs() / ref[-1, 0].abs()) < 1e-4


def test_long_decoding(dirs):
    """A short prompt and 300 tokens one by one (pages fill and follow one another; the states run on)."""
    from pih_b200.engine.factory import create_runner
    name = "R2"
    requests = traces.make_requests(rm.CONFIGS[name]["vocab"], [310], seed=9)
    steps = traces.tail_decode(requests, tail=300)
    _, model, cache, runner = create_runner(dirs[name], "float32", page_size=8, max_cache_tokens=320, max_requests=1)
    _check(traces.replay(runner, steps), rm.plain_logits(dirs[name], requests), "float32", "long decoding")
    model.rt.ops.check_errors()


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_greedy_generation_through_the_engine(dirs, cuda_graphs):
    """Engine.complete (scheduler, cache, sampler, graphs) against greedy decoding with the plain implementation; three
    requests at once with fewer state slots' worth of room than requests, so they queue."""
    from pih_b200.engine import Engine
    name = "R1"
    cfg, w = rm.load_plain(dirs[name])
    prompts = list(traces.make_requests(rm.CONFIGS[name]["vocab"], [9, 21, 5], seed=13).values())
    new = 12
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(new):
            toks.append(int(plain.forward(cfg, w, toks)[-1].argmax()))
        want.append(toks[len(p):])
    engine = Engine(dirs[name], "float32", page_size=16, max_cache_tokens=256, maximum_batch_sequences=2,
                    maximum_batch_tokens=64, maximum_context_tokens=64, cuda_graphs=cuda_graphs)
    results = engine.complete_batch(prompts, max_tokens=new, temperature=0.0, ignore_eos=True)
    engine.rt.ops.check_errors()
    for r, expect in zip(results, want):
        assert r["token_ids"] == expect


def test_command_lines(dirs, tmp_path):
    """bin/pih-worker makes a random Rigotar model from a configuration file and generates from it; bin/trace_run
    replays a trace on it; both agree with the plain implementation."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from conftest import ROOT
    worker = [sys.executable, os.path.join(ROOT, "bin", "pih-worker")]
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(rm.R2))
    folder = str(tmp_path / "made")
    proc = subprocess.run(worker + ["--random-model", folder, "--config", str(cfg_file), "--seed", "4", "--sigma", "0.15"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    prompt = [5, 17, 3, 200, 9]
    proc = subprocess.run(worker + ["--model", folder, "--generate-tokens", ",".join(map(str, prompt)), "--max-tokens", "7",
                                    "--dtype", "float32", "--ignore-eos"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(proc.stdout.strip().splitlines()[-1])
    cfg, w = rm.load_plain(folder)
    toks = list(prompt)
    for _ in range(7):
        toks.append(int(plain.forward(cfg, w, toks)[-1].argmax()))
    assert res["token_ids"] == toks[len(prompt):]

    requests = traces.make_requests(rm.R2["vocab"], [40, 9, 23], seed=6)
    steps = traces.mixed(requests, seed=1, max_live=3)
    for s_ in steps:
        for e in s_["entries"]:
            e["want"] = e["want"][-1:]                              # the last place of every portion
    out_dir = str(tmp_path / "out")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out_dir,
           "--max-tokens", str(traces.peak_tokens(steps))]
    proc = subprocess.run(cmd, input="\n".join(json.dumps(s_) for s_ in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s_['step']}" for s_ in steps]
    truth = rm.plain_logits(folder, requests)
    at = {rid: 0 for rid in requests}
    for s_ in steps:
        got = np.fromfile(os.path.join(out_dir, f"{s_['step']}.f32"), dtype="<f4").reshape(-1, rm.R2["vocab"])
        for j, e in enumerate(s_["entries"]):
            at[e["id"]] += len(e["tokens"])
            ref = truth[e["id"]][at[e["id"]] - 1].numpy()
            assert np.abs(got[j] - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()), (s_["step"], e["id"])
