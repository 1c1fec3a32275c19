"""The Tuganex design on the GPU against the plain float64 restatement (tests/plain_tuganex.py): each mechanism
alone, every way of cutting requests into steps, batches against requests alone, pages and state slots that are used
again, keys that must be found far back / at page borders / among the first tokens, in prompts and in decoding, long
decoding, and greedy generation through the engine's own entry point."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_tuganex as plain
import traces
import tuganex_models as tm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for i, (n, raw) in enumerate(tm.CONFIGS.items()):
        out[n] = tm.write_model(tmp_path_factory.mktemp(f"tuganex_{n}"), raw, seed=5 + i, sigma=tm.SIGMA[n])
        out[n + "-all"] = tm.write_model(tmp_path_factory.mktemp(f"tuganex_{n}_all"), tm.all_chosen(raw), seed=5 + i,
                                         sigma=tm.SIGMA[n])
    return out


def _ops():
    from pih_b200.kernels import get_ops
    return get_ops(torch.device(DEV))


def _check(got, truth, dtype, what):
    """Per position: the error of the logits (mean taken off, root mean square over the vocabulary) relative to the
    logits' spread.  32-bit: every position of every request.  bfloat16 (models whose routers choose every output), over
    the positions of all requests together: the median within rounding, and at most one position in ten beyond three
    times that."""
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


LENGTHS = {"T1": [70, 45, 131, 33, 64, 50, 1, 2], "T2": [65, 33, 97, 128, 80, 3, 35, 66]}
FAMILIES = ["whole", "tail_decode", "portions", "mixed"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["T1", "T2"])
@pytest.mark.parametrize("family", FAMILIES)
def test_cuttings_against_the_plain_implementation(dirs, name, dtype, family):
    """Whole prompts; most of a prompt and then token by token; portions down to two tokens; up to three live
    requests mixed, with a pool so small and so few state slots that pages and slots are used again."""
    from pih_b200.engine.factory import create_runner
    requests = traces.make_requests(tm.CONFIGS[name]["vocab"], LENGTHS[name], seed=21)
    kw = dict(max_live=3) if family == "mixed" else {}
    steps = getattr(traces, family)(requests, **kw)
    folder = dirs[name] if dtype == "float32" else dirs[name + "-all"]
    _, model, cache, runner = create_runner(folder, dtype, page_size=16 if name == "T1" else 8,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=16), max_requests=3)
    got = traces.replay(runner, steps)
    model.rt.ops.check_errors()
    _check(got, tm.plain_logits(folder, requests), dtype, f"{name} {family} {dtype}")
    cache.check()
    assert all(f == cache.num_pages for f in cache.num_free_pages()) and cache.slots.num_free == 3
    if family == "mixed":
        assert all(g.pool.pages_handed_out > g.pool.num_pages for g in cache.groups)


@pytest.mark.parametrize("kind, changes", [("retention", {}), ("attention", {}),
                                           ("retention", {"heads": 1, "decay": [1.0], "rot": {"dims": 12, "base": 77.0}}),
                                           ("attention", {"heads": 1, "kv_heads": 1, "dim": 40, "vdim": 8,
                                                          "rot": {"dims": 40, "base": 3.0}, "diff": 0.0})])
def test_a_mixer_alone(tmp_path, kind, changes):
    """One layer of one mixer and no feed-forward, whole and token by token; also with one head, a rotation over the
    whole head, a decay of one and a lambda without its constant."""
    from pih_b200.engine.factory import create_runner
    d = tm.write_model(tmp_path / kind, tm.single_layer(kind, **changes), seed=3, sigma=0.2)
    requests = traces.make_requests(120, [40, 7], seed=2)
    truth = tm.plain_logits(d, requests)
    for family in ("whole", "tail_decode"):
        _, model, cache, runner = create_runner(d, "float32", page_size=8, max_cache_tokens=64, max_requests=2)
        _check(traces.replay(runner, getattr(traces, family)(requests)), truth, "float32", f"{kind} {family}")
        model.rt.ops.check_errors()


@pytest.mark.parametrize("mlp", [{"kind": "dense", "ff": 52},
                                 tm._moe(7, 3, 3, 36, groups=(5, 2), shared=28),
                                 tm._moe(4, 0, 4, 20)])
def test_a_feed_forward_alone(tmp_path, mlp):
    """The biased feed-forward, and the routed one with groups, identity experts and a shared expert (and without any
    of them), behind a mixer."""
    from pih_b200.engine.factory import create_runner
    d = tm.write_model(tmp_path / "ff", tm.single_layer("retention", mlp=mlp), seed=4, sigma=0.25)
    requests = traces.make_requests(120, [50, 9], seed=5)
    _, model, cache, runner = create_runner(d, "float32", page_size=8, max_cache_tokens=64, max_requests=2)
    _check(traces.replay(runner, traces.whole(requests)), tm.plain_logits(d, requests), "float32", "feed-forward")
    model.rt.ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("groups, keep", [(1, 1), (4, 2), (6, 1)])
def test_scored_routing_with_decided_scores(dtype, groups, keep):
    """The routed feed-forward as an op with router logits given so that no rounding decides a choice: distinct
    logits, a correction that changes the order and makes choice scores negative, groups, identity experts; every
    row's output against the plain weighted sum of its chosen experts, for many rows and for few."""
    ops = _ops()
    g = torch.Generator().manual_seed(6 + groups)
    rows, hidden, ff, experts, identity, top = 300, 40, 72, 9, 3, 2
    n = experts + identity
    x = (torch.randn(rows, hidden, generator=g) * 0.8).to(dtype)
    wg, wu = [(torch.randn(experts, ff, hidden, generator=g) * 0.2).to(dtype) for _ in range(2)]
    wd = (torch.randn(experts, hidden, ff, generator=g) * 0.2).to(dtype)
    logits = torch.stack([torch.randperm(n, generator=g).float() * 0.7 - 2.0 for _ in range(rows)])
    logits = torch.cat([logits, torch.randn(rows, 1, generator=g)], dim=1)           # one more column, not the router's
    correction = -1.0 - torch.randperm(n, generator=g).float() * 0.11                # all choice scores negative
    f = {"router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}
    w = {"m.router": torch.eye(n, dtype=F64), "m.correction": correction.double()}
    chosen, weights = plain.route(logits[:, :n].double(), f, w, "m.")
    ref = torch.zeros(rows, hidden, dtype=F64)
    xd = x.double()
    for t in range(rows):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            if e >= experts:
                ref[t] += a * xd[t]
            else:
                ref[t] += a * ((plain.silu(xd[t] @ wg[e].double().T) * (xd[t] @ wu[e].double().T)) @ wd[e].double().T)
    assert len(set(chosen.flatten().tolist())) > top and int((chosen >= experts).sum()) > 0
    routing = dict(outputs=n, correction=correction.to(DEV), groups=groups, groups_keep=keep, renormalize=False)
    wgu = torch.cat([wg, wu], dim=1).to(DEV).contiguous()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for count in (rows, 5):
        got = ops.moe_experts(x[:count].to(DEV), logits[:count].to(DEV), wgu, wd.to(DEV).contiguous(), top, routing=routing)
        ops.check_errors()
        assert float((got.double().cpu() - ref[:count]).abs().max()) < tol * float(ref.abs().max()), count
    routing["renormalize"] = True
    got = ops.moe_experts(x.to(DEV), logits.to(DEV), wgu, wd.to(DEV).contiguous(), top, routing=routing).double().cpu()
    scale = (1.0 / weights.sum(-1))[:, None]
    assert float((got - ref * scale).abs().max()) < tol * float((ref * scale).abs().max())


def test_row_wise_kernels():
    """The stream's norm-and-add with a bias, its rounded copy, the activation on both sides of zero, and the gated add."""
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    rows, width = 37, 200
    h = torch.randn(rows, width, generator=g)
    y = torch.randn(rows, width, generator=g) * 3
    bias, weight = torch.randn(width, generator=g), torch.randn(width, generator=g)
    for dtype in (torch.float32, torch.bfloat16):
        hd = h.clone().to(DEV)
        yq = y.to(dtype)
        copy = ops.stream_norm_add(hd, yq.to(DEV), weight.to(DEV), 1e-5, bias=bias.to(DEV), copy_dtype=torch.bfloat16)
        v = yq.double() + bias.double()
        ref = h.double() + plain.rms_unit(v, 1e-5) * weight.double()
        assert float((hd.double().cpu() - ref).abs().max()) < 1e-5
        assert torch.equal(copy.cpu(), hd.cpu().bfloat16())
    for width in (143, 144):                                 # element by element, and 16 bytes a thread
        z = torch.linspace(-6, 6, 7 * width).view(7, width)
        b = torch.randn(width, generator=g) * 0.1
        u = z.double() + b.double()
        ref = torch.where(u > 0, 0.8 * u * u + 0.5 * u, 1.3 * (torch.expm1(u) - u) + 0.5 * u)
        assert float((ops.bias_xielu(z.to(DEV), b.to(DEV), 0.8, 1.3).double().cpu() - ref).abs().max()) < 1e-5
        zb = z.bfloat16()
        ub = zb.double() + b.double()
        refb = torch.where(ub > 0, 0.8 * ub * ub + 0.5 * ub, 1.3 * (torch.expm1(ub) - ub) + 0.5 * ub)
        assert float((ops.bias_xielu(zb.to(DEV), b.to(DEV), 0.8, 1.3).double().cpu() - refb).abs().max()) < 0.2
    gate = torch.randn(rows, 3, generator=g)
    got = ops.add_gated(h.to(DEV), y.to(DEV), gate.to(DEV)[:, 1]).double().cpu()
    assert float((got - (h.double() + torch.sigmoid(gate[:, 1].double())[:, None] * y.double())).abs().max()) < 1e-5
    ops.check_errors()


def test_batches_against_each_request_alone(dirs):
    """Unequal requests side by side in one step — a long portion, a short one, single tokens — give each request
    the bits it gets alone (32-bit: every reduction has an order fixed by the row)."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    name = "T1"
    requests = traces.make_requests(tm.CONFIGS[name]["vocab"], [61, 18, 40, 9], seed=8)
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
                           num_requests=len(slots), host_cu_q=list(cu_q), host_q_start=[positions[c] for c in cu_q[:-1]],
                           q_start=t([positions[c] for c in cu_q[:-1]]), meta=None, attention_plans={})


def _plain_diff_row(q, K, V, scale, lam, eps, out_scale, group):
    """q [heads, 2, dim]; K [n, kv_heads, 2, dim]; V [n, kv_heads, vdim] (float64): the row's output [heads, vdim]."""
    out = []
    for h in range(q.shape[0]):
        g = h // group
        a = [torch.softmax((K[:, g, j] @ q[h, j]) * scale, dim=0) @ V[:, g] for j in range(2)]
        out.append(a[0] - lam * a[1])
    return plain.rms_unit(torch.stack(out), eps) * out_scale


def _paged(K, V, page, dtype, pages=None):
    """The cache tensor [pages, page, width] and block table of one request whose keys and values are given."""
    n = K.shape[0]
    rows = torch.cat([K.reshape(n, -1), V.reshape(n, -1)], dim=1)
    pages = pages if pages is not None else list(range(-(-n // page) + 1))[::-1]
    cache = torch.zeros(max(pages) + 2, page, rows.shape[1], dtype=dtype, device=DEV)
    for j in range(n):
        cache[pages[j // page], j % page] = rows[j].to(dtype).to(DEV)
    return cache, torch.tensor([pages], dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, vdim, heads, kv_heads", [(16, 24, 4, 2), (64, 64, 2, 1), (32, 128, 6, 6), (128, 128, 2, 1),
                                                        (24, 40, 2, 2), (12, 20, 3, 1), (40, 320, 1, 1)])
@pytest.mark.parametrize("needle", [0, 1, 15, 16, 17, 63, 64, 250, 299])
def test_differential_attention_finds_one_key_among_hundreds(needle, dim, vdim, heads, kv_heads, dtype):
    """300 cached keys of which ONE matches the query's first map (its score stands out by construction) and another
    one the second map: the first tokens, both sides of a page border, far back, and the row itself — as a single
    decoded row, and as the last row of a prompt portion of 70 rows.  Random inputs would average such a key away."""
    ops = _ops()
    g = torch.Generator().manual_seed(needle)
    n, page, scale, lam, eps, out_scale = 300, 16, 0.5, 0.35, 1e-5, 0.6
    other = (needle + 100) % n
    K = torch.randn(n, kv_heads, 2, dim, generator=g, dtype=F64) * 0.3
    K[needle, :, 0] = torch.randn(kv_heads, dim, generator=g, dtype=F64)
    K[other, :, 1] = torch.randn(kv_heads, dim, generator=g, dtype=F64)
    V = torch.randn(n, kv_heads, vdim, generator=g, dtype=F64)
    group = heads // kv_heads
    rows = 70
    q = torch.randn(rows, heads, 2, dim, generator=g, dtype=F64) * 0.2
    for h in range(heads):
        q[-1, h, 0] += 4.0 * K[needle, h // group, 0] * (4.0 / math.sqrt(dim))
        q[-1, h, 1] += 4.0 * K[other, h // group, 1] * (4.0 / math.sqrt(dim))
    K, V, q = K.to(dtype).double(), V.to(dtype).double(), q.to(dtype).double()       # what the kernels read
    cache, table = _paged(K, V, page, dtype)
    geometry = dict(heads=heads, kv_heads=kv_heads, key_dim=dim, value_dim=vdim)
    ref = _plain_diff_row(q[-1], K, V, scale, lam, eps, out_scale, group)
    weight_of_needle = torch.softmax((K[:, 0, 0] @ q[-1, 0, 0]) * scale, dim=0)[needle]
    assert float(weight_of_needle) > 0.5                              # the key does stand out
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    # a decoded row
    step = _step([n - 1], [0], [0, 1], [0])
    got = ops.diff_attention(q[-1:].reshape(1, -1).to(dtype).to(DEV).contiguous(), cache=cache, block_table=table, step=step,
                             scale=scale, lam=lam, out_scale=out_scale, norm_eps=eps, window=0, **geometry)
    ops.check_errors()
    assert float((got[0].double().cpu().view(heads, vdim) - ref).abs().max()) < tol * float(ref.abs().max())
    # the last row of a portion
    step = _step(list(range(n - rows, n)), [0] * rows, [0, rows], [0])
    got = ops.diff_attention(q.reshape(rows, -1).to(dtype).to(DEV).contiguous(), cache=cache, block_table=table, step=step,
                             scale=scale, lam=lam, out_scale=out_scale, norm_eps=eps, window=0, **geometry)
    ops.check_errors()
    assert float((got[-1].double().cpu().view(heads, vdim) - ref).abs().max()) < tol * float(ref.abs().max())
    mid = rows // 2                                                    # and a row in the middle sees only its own past
    p = n - rows + mid
    ref_mid = _plain_diff_row(q[mid], K[:p + 1], V[:p + 1], scale, lam, eps, out_scale, group)
    assert float((got[mid].double().cpu().view(heads, vdim) - ref_mid).abs().max()) < tol * float(ref_mid.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_differential_attention_portions_of_several_requests(dtype):
    """Portions of three requests in one step — one deep in its context, one from its first token, one of five rows
    (and a request of a single row): every row against the plain computation over its own request's keys up to its own
    position."""
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    heads, kv_heads, dim, vdim, page = 4, 2, 32, 48, 16
    starts, counts = [300, 0, 37, 99], [70, 131, 5, 1]
    caches, tables, Ks, Vs, next_page = [], [], [], [], 0
    for st, c in zip(starts, counts):
        n = st + c
        K = (torch.randn(n, kv_heads, 2, dim, generator=g, dtype=F64) * 0.5).to(dtype).double()
        V = torch.randn(n, kv_heads, vdim, generator=g, dtype=F64).to(dtype).double()
        pages = list(range(next_page, next_page + -(-n // page)))[::-1]
        next_page += len(pages)
        Ks.append(K), Vs.append(V), tables.append(pages)
    cache = torch.zeros(next_page + 1, page, kv_heads * (2 * dim + vdim), dtype=dtype, device=DEV)
    width = max(len(p) for p in tables)
    table = torch.full((len(starts), width), -1, dtype=torch.int32)
    for r, pages in enumerate(tables):
        table[r, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        rows = torch.cat([Ks[r].reshape(Ks[r].shape[0], -1), Vs[r].reshape(Vs[r].shape[0], -1)], dim=1).to(dtype).to(DEV)
        for j in range(rows.shape[0]):
            cache[pages[j // page], j % page] = rows[j]
    T = sum(counts)
    q = (torch.randn(T, heads, 2, dim, generator=g, dtype=F64) * 0.6).to(dtype).double()
    positions, request_of_row, cu = [], [], [0]
    for r, (st, c) in enumerate(zip(starts, counts)):
        positions += list(range(st, st + c))
        request_of_row += [r] * c
        cu.append(cu[-1] + c)
    step = _step(positions, request_of_row, cu, [0, 1, 2, 3])
    got = ops.diff_attention(q.reshape(T, -1).to(dtype).to(DEV).contiguous(), cache=cache, block_table=table.to(DEV), step=step,
                             scale=0.3, lam=-0.4, out_scale=0.8, norm_eps=1e-5, window=0, heads=heads, kv_heads=kv_heads,
                             key_dim=dim, value_dim=vdim).double().cpu()
    ops.check_errors()
    worst = 0.0
    for t in range(T):
        r, p = request_of_row[t], positions[t]
        ref = _plain_diff_row(q[t], Ks[r][:p + 1], Vs[r][:p + 1], 0.3, -0.4, 1e-5, 0.8, heads // kv_heads)
        worst = max(worst, float((got[t].view(heads, vdim) - ref).abs().max()) / float(ref.abs().max()))
    assert worst < (1e-5 if dtype == torch.float32 else 2e-2), worst


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_differential_attention_window_edges(dtype):
    """A window whose oldest key is the standing-out key, and one that has just moved past it: as a decoded row (whole
    and cut into parts) and as the last row of a portion (the tensor-core kernel in bfloat16)."""
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    heads, kv_heads, dim, vdim, n, page, rows = 2, 1, 16, 32, 200, 8, 40
    needle, last = 131, n - 1
    K = torch.randn(n, kv_heads, 2, dim, generator=g, dtype=F64) * 0.3
    V = torch.randn(n, kv_heads, vdim, generator=g, dtype=F64)
    q = torch.randn(rows, heads, 2, dim, generator=g, dtype=F64) * 0.1
    q[-1, :, 0] += 6.0 * K[needle, 0, 0]
    K, V, q = K.to(dtype).double(), V.to(dtype).double(), q.to(dtype).double()
    cache, table = _paged(K, V, page, dtype)
    geometry = dict(heads=heads, kv_heads=kv_heads, key_dim=dim, value_dim=vdim)
    results = {}
    for window in (last - needle + 1, last - needle):
        ref = _plain_diff_row(q[-1], K[last - window + 1:], V[last - window + 1:], 1.0, 0.3, 1e-5, 0.5, heads)
        one = ops.diff_attention(q[-1:].reshape(1, -1).to(dtype).to(DEV).contiguous(), cache=cache, block_table=table,
                                 step=_step([last], [0], [0, 1], [0]), scale=1.0, lam=0.3, out_scale=0.5, norm_eps=1e-5,
                                 window=window, **geometry)[0]
        many = ops.diff_attention(q.reshape(rows, -1).to(dtype).to(DEV).contiguous(), cache=cache, block_table=table,
                                  step=_step(list(range(n - rows, n)), [0] * rows, [0, rows], [0]), scale=1.0, lam=0.3,
                                  out_scale=0.5, norm_eps=1e-5, window=window, **geometry)[-1]
        ops.check_errors()
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        for got in (one, many):
            assert float((got.double().cpu().view(heads, vdim) - ref).abs().max()) < tol * float(ref.abs().max()), window
        results[window] = one.double().cpu()
    assert float((results[last - needle + 1] - results[last - needle]).abs().max()) > 0.1


def test_queries_and_keys_are_normed_then_rotated_into_their_slots():
    """The kernel in front of the attention: per-map norm with the shared weight, rotation over part of a map at the
    row's own position (also a large one), q in place, k and v into the row's slot; a row of padding writes nothing."""
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    heads, kv_heads, dim, vdim, rot, page = 3, 1, 20, 12, 8, 4
    T = 6
    positions = [0, 1, 5, 1000, 70000, 0]
    slots = [9, 2, 3, 17, 0, -2]
    qkv = torch.randn(T, (heads + kv_heads) * 2 * dim + kv_heads * vdim, generator=g, dtype=F64).float()
    qn, kn = torch.randn(dim, generator=g).float() + 1, torch.randn(dim, generator=g).float() + 1
    freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=F64)
    cache = torch.full((6, page, kv_heads * (2 * dim + vdim)), 7.0, dtype=torch.float32, device=DEV)
    dev = qkv.clone().to(DEV)
    ops.diff_qk_prepare(dev, q_norm=qn.to(DEV), k_norm=kn.to(DEV), eps=1e-5, frequencies=freq.float().to(DEV),
                        positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                        slot_mapping=torch.tensor(slots, dtype=torch.int32, device=DEV), cache=cache, write_kv=True,
                        heads=heads, kv_heads=kv_heads, key_dim=dim, value_dim=vdim)
    ops.check_errors()
    nq, nk = heads * 2 * dim, kv_heads * 2 * dim
    pos = torch.tensor(positions)
    ref_q = plain.rotate(plain.rms_unit(qkv[:, :nq].double().view(T, -1, dim), 1e-5) * qn.double(), pos, rot, 50.0)
    ref_k = plain.rotate(plain.rms_unit(qkv[:, nq:nq + nk].double().view(T, -1, dim), 1e-5) * kn.double(), pos, rot, 50.0)
    # at position 70000 a 32-bit angle is good to about 70000 * 2^-24
    tol = torch.tensor([1e-5, 1e-5, 1e-5, 3e-4, 2e-2, 1e-5], dtype=F64)[:, None]
    assert bool(((dev[:, :nq].double().cpu() - ref_q.reshape(T, -1)).abs() < tol).all())
    flat = cache.view(-1, cache.shape[-1]).double().cpu()
    for t, s in enumerate(slots[:-1]):
        assert bool(((flat[s, :nk] - ref_k[t].reshape(-1)).abs() < tol[t]).all())
        assert torch.equal(flat[s, nk:], qkv[t, nq + nk:].double())
    untouched = [s for s in range(flat.shape[0]) if s not in slots]
    assert bool((flat[untouched] == 7.0).all())


@pytest.mark.parametrize("dim, vdim", [(16, 24), (32, 64), (64, 128), (128, 32), (24, 40)])
def test_retention_recalls_a_value_written_long_ago(dim, vdim):
    """With a decay of one and orthonormal keys the state returns the value that was written under a key many tokens
    earlier, across steps and beside another request: a lost, re-zeroed or mixed-up state would not.  With a decay
    below one it returns that value times the decay to the power of the distance."""
    ops = _ops()
    heads, n = 2, 3 * dim + 5
    g = torch.Generator().manual_seed(3)
    keys = torch.linalg.qr(torch.randn(dim, dim, generator=g, dtype=F64)).Q
    k = keys[torch.arange(n) % dim].repeat(1, heads)                               # key i again every dim tokens
    v = torch.randn(n, heads * vdim, generator=g, dtype=F64)
    qk = torch.cat([k, k], dim=1).float().to(DEV).contiguous()
    vd = v.float().to(DEV).contiguous()
    decays = torch.tensor([1.0, 0.99], dtype=F64)
    state = torch.zeros(3, heads * dim * vdim, dtype=torch.float32, device=DEV)
    state[1] = 5.0                                                                  # another request's slot
    outs, at = [], 0
    for c in (dim + 3, 1, 1, n - dim - 5):                                           # a portion, two single tokens, the rest
        step = _step(list(range(at, at + c)), [0] * c, [0, c], [2])
        outs.append(ops.retention(qk[at:at + c], vd[at:at + c], frequencies=None,
                                  decay_minus_one=(decays - 1.0).float().to(DEV), key_scale=1.0, state=state, step=step,
                                  heads=heads, key_dim=dim, value_dim=vdim))
        at += c
    ops.check_errors()
    got = torch.cat(outs).double().cpu()                                             # [n, heads, vdim]
    vv = v.view(n, heads, vdim)
    for t in (dim + 1, 2 * dim + 7, n - 1):
        past = [j for j in range(t + 1) if j % dim == t % dim]
        for h in range(heads):
            ref = sum(vv[j, h] * float(decays[h]) ** (t - j) for j in past)
            assert float((got[t, h] - ref).abs().max()) < 1e-4 * float(ref.abs().max()), (t, h)
    assert bool((state[1] == 5.0).all()) and bool((state[0] == 0.0).all())


def test_retention_rotates_by_the_position_not_by_the_row():
    """The same tokens at positions 0.. and at positions 1000..: with keys and queries rotated by their positions the
    read-outs agree (a rotation by a common angle cancels), and they differ when only the rows' order is moved."""
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    heads, dim, vdim, n = 2, 16, 8, 12
    qk = torch.randn(n, 2 * heads * dim, generator=g).to(DEV)
    v = torch.randn(n, heads * vdim, generator=g).to(DEV)
    freq = torch.tensor([100.0 ** (-2.0 * i / 8) for i in range(4)], dtype=torch.float32, device=DEV)
    dm1 = torch.tensor([-0.1, -0.01], dtype=torch.float32, device=DEV)

    def run(start):
        state = torch.zeros(1, heads * dim * vdim, dtype=torch.float32, device=DEV)
        return ops.retention(qk, v, frequencies=freq, decay_minus_one=dm1, key_scale=0.25, state=state,
                             step=_step(list(range(start, start + n)), [0] * n, [0, n], [0]), heads=heads, key_dim=dim,
                             value_dim=vdim)

    a, b = run(0), run(1000)
    ops.check_errors()
    assert float((a - b).abs().max()) < 2e-3 * float(a.abs().max()) and float(a.abs().max()) > 0.1


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Sizes, orders of layers, shared caches and constants drawn at random (odd sizes and sizes that only the plain
    kernels take among them): a mixed schedule in 32-bit against the plain implementation position by position, and in
    bfloat16 (every router output chosen) within rounding."""
    from pih_b200.engine.factory import create_runner
    raw = tm.random_config(seed)
    requests = traces.make_requests(raw["vocab"], [70, 45, 33, 18, 1, 2], seed=seed)
    steps = traces.mixed(requests, seed=seed, max_live=3)
    for dtype, cfg in (("float32", raw), ("bfloat16", tm.all_chosen(raw))):
        d = tm.write_model(tmp_path / dtype, cfg, seed=seed, sigma=0.15)
        _, model, cache, runner = create_runner(d, dtype, page_size=16, max_cache_tokens=traces.peak_tokens(steps, round_to=16),
                                                max_requests=3)
        got = traces.replay(runner, steps)
        model.rt.ops.check_errors()
        _check(got, tm.plain_logits(d, requests), dtype, f"seed {seed} {dtype}")
        cache.check()


def test_long_decoding(dirs):
    """A short prompt and 300 tokens one by one (pages fill and follow one another; the states run on)."""
    from pih_b200.engine.factory import create_runner
    name = "T2"
    requests = traces.make_requests(tm.CONFIGS[name]["vocab"], [310], seed=9)
    steps = traces.tail_decode(requests, tail=300)
    _, model, cache, runner = create_runner(dirs[name], "float32", page_size=8, max_cache_tokens=320, max_requests=1)
    _check(traces.replay(runner, steps), tm.plain_logits(dirs[name], requests), "float32", "long decoding")
    model.rt.ops.check_errors()


@pytest.mark.parametrize("cuda_graphs", [False, True])
@pytest.mark.parametrize("name", ["T1", "T2"])
def test_greedy_generation_through_the_engine(dirs, name, cuda_graphs):
    """Engine.complete (scheduler, cache, sampler, graphs, padded steps) against greedy decoding with the plain
    implementation; three requests at once with room for two, so they queue."""
    from pih_b200.engine import Engine
    cfg, w = tm.load_plain(dirs[name])
    prompts = list(traces.make_requests(tm.CONFIGS[name]["vocab"], [9, 21, 5], seed=13).values())
    new = 12
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(new):
            toks.append(int(plain.model_layers(cfg, w, toks)[1][-1].argmax()))
        want.append(toks[len(p):])
    engine = Engine(dirs[name], "float32", page_size=16, max_cache_tokens=256, maximum_batch_sequences=2,
                    maximum_batch_tokens=64, maximum_context_tokens=64, cuda_graphs=cuda_graphs)
    results = engine.complete_batch(prompts, max_tokens=new, temperature=0.0, ignore_eos=True)
    engine.rt.ops.check_errors()
    for r, expect in zip(results, want):
        assert r["token_ids"] == expect


def test_command_lines(dirs, tmp_path):
    """bin/pih-worker makes a random Tuganex model from a configuration file and generates from it; bin/trace_run
    replays a trace on it; both agree with the plain implementation."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from conftest import ROOT
    worker = [sys.executable, os.path.join(ROOT, "bin", "pih-worker")]
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(tm.T2))
    folder = str(tmp_path / "made")
    proc = subprocess.run(worker + ["--random-model", folder, "--config", str(cfg_file), "--seed", "4", "--sigma", "0.15"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    prompt = [5, 17, 3, 200, 9]
    proc = subprocess.run(worker + ["--model", folder, "--generate-tokens", ",".join(map(str, prompt)), "--max-tokens", "7",
                                    "--dtype", "float32", "--ignore-eos"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(proc.stdout.strip().splitlines()[-1])
    cfg, w = tm.load_plain(folder)
    toks = list(prompt)
    for _ in range(7):
        toks.append(int(plain.model_layers(cfg, w, toks)[1][-1].argmax()))
    assert res["token_ids"] == toks[len(prompt):]

    requests = traces.make_requests(tm.T2["vocab"], [40, 9, 23], seed=6)
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
    truth = tm.plain_logits(folder, requests)
    at = {rid: 0 for rid in requests}
    for s_ in steps:
        got = np.fromfile(os.path.join(out_dir, f"{s_['step']}.f32"), dtype="<f4").reshape(-1, tm.T2["vocab"])
        for j, e in enumerate(s_["entries"]):
            at[e["id"]] += len(e["tokens"])
            ref = truth[e["id"]][at[e["id"]] - 1].numpy()
            assert np.abs(got[j] - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()), (s_["step"], e["id"])
