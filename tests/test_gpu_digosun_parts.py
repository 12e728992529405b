"""Digosun's mechanisms one at a time: each kernel against the plain function of the same name.

Attention cases plant one dominating key (its latent and one query are scaled so that its score
stands out) far back among hundreds, on either side of a window's edge and at page borders, in
prompt portions and in single-token steps; sinks are made large enough to matter."""

import pytest
import torch

from somi_inference_b200.cache import CacheManager
from somi_inference_b200.engine.batch import BatchBuilder, StepEntry
from somi_inference_b200.parts.base import CacheNeeds, PagedKVNeeds, StateNeeds
from tests.plain import digosun_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from somi_inference_b200.ops import cuda_ops
    return cuda_ops()


def tol(dtype, f32=2e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def make_batch(ops, requests, *, rank=None, window=None, page_size=8, state=None, dtype=torch.float32,
               seed=0):
    """`requests`: (tokens cached, tokens in this step) each.  Returns manager, batch, order."""
    g = torch.Generator().manual_seed(seed)
    needs = CacheNeeds(paged=None if rank is None else PagedKVNeeds(1, rank, window, value_dim=0),
                       state=state)
    if rank is None:
        needs = CacheNeeds(paged=PagedKVNeeds(1, 8, None, value_dim=0), state=state)
    pages = sum(-(-(c + q) // page_size) for c, q in requests) + 3
    mgr = CacheManager([needs], [None], num_pages=pages, page_size=page_size,
                       max_requests=len(requests) + 1,
                       max_positions=max(c + q for c, q in requests) + page_size, dtype=dtype,
                       device="cuda")
    pool = mgr.groups[0].pool
    taken = pool.take(pool.num_free)
    pool.give_back([taken[i] for i in torch.randperm(len(taken), generator=g).tolist()])
    entries = []
    for i, (c, q) in enumerate(requests):
        mgr.register(i)
        if c:
            mgr.reserve(i, c)
            mgr.commit(i)
        mgr.reserve(i, q)
        entries.append(StepEntry(i, [0] * q, []))
    builder = BatchBuilder(mgr, device="cuda", q_tile_sizes=ops.q_tile_sizes)
    batch, order = builder.build(entries)
    return mgr, batch, order


# ------------------------------------------------------------------ embedding and norms
@pytest.mark.parametrize("width", [48, 256, 1030, 37])
def test_embedding_sinusoid_layernorm(ops, width):
    g = torch.Generator().manual_seed(width)
    table = torch.randn(50, width, generator=g)
    weight = 1 + 0.3 * torch.randn(width, generator=g)
    ids = torch.randint(0, 50, (9,), generator=g)
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 4095, 20000, 7])
    inv = (10000.0 ** (-torch.arange(0, width, 2, dtype=torch.float64) / width)).float()
    out = torch.empty(9, width, device="cuda")
    ops.embed_sinusoid_layernorm(ids.int().cuda(), pos.int().cuda(), table.cuda(), inv.cuda(),
                                 weight.cuda(), 1e-6, out)
    ref = plain.layer_norm(table.double()[ids] + plain.sinusoid(pos, width), weight.double(), 1e-6)
    # a float32 angle of 20000 radians is itself only exact to 1e-3: compare where it is exact
    assert (out.cpu().double() - ref)[:5].abs().max() < 1e-5
    assert (out.cpu().double() - ref).abs().max() < 5e-3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("T, H", [(6, 200), (3, 4100), (40, 202)])
def test_gated_residual_layernorm(ops, dtype, splits, gated, T, H):
    g = torch.Generator().manual_seed(7)
    residual = (3 * torch.randn(T, H, generator=g) + 2.0).cuda()      # a mean to take off
    delta = torch.randn(splits, T, H, generator=g).cuda() if splits > 1 else \
        torch.randn(T, H, generator=g).to(dtype).cuda()
    wide = (2 * torch.randn(T, H + 24, generator=g)).to(dtype).cuda()
    gate = wide[:, 24:] if gated else None                             # rows further apart than H
    weight = (1 + 0.2 * torch.randn(H, generator=g)).to(dtype).cuda()
    before = residual.clone()
    out = torch.empty(T, H, dtype=dtype, device="cuda")
    ops.add_layernorm(residual, delta, gate, weight, 1e-5, out)
    d = delta.double().sum(0) if splits > 1 else delta.double()
    if gated:
        d = d * torch.sigmoid(gate.double())
    r = before.double() + d
    assert (residual.double() - r).abs().max() < 1e-5
    ref = plain.layer_norm(r, weight.double(), 1e-5)
    assert (out.double() - ref).abs().max() < tol(dtype, 1e-5, 3e-2)
    rows = torch.tensor([2, 1], dtype=torch.int32, device="cuda")
    again = residual.clone()
    few = torch.empty(2, H, dtype=dtype, device="cuda")
    ops.add_layernorm(again, None, None, weight, 1e-5, few, rows)
    assert torch.equal(again, residual) and (few.double() - ref[[2, 1]]).abs().max() < tol(dtype, 1e-5, 3e-2)
    if gated:     # the gate's logits as partial sums of a split-K product
        parts = torch.randn(3, T, H, generator=g).cuda()
        r2 = before.clone()
        ops.add_layernorm(r2, delta, parts, weight, 1e-5, out)
        d2 = (delta.double().sum(0) if splits > 1 else delta.double()) * torch.sigmoid(parts.double().sum(0))
        assert (r2.double() - (before.double() + d2)).abs().max() < 1e-5
        ref2 = plain.layer_norm(before.double() + d2, weight.double(), 1e-5)
        assert (out.double() - ref2).abs().max() < tol(dtype, 1e-5, 3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, n, extra", [(5, 77, 19), (3, 4864, 896), (600, 72, 8)])
def test_xielu(ops, dtype, T, n, extra):
    g = torch.Generator().manual_seed(1)
    x = (3 * torch.randn(T, n + extra, generator=g)).to(dtype).cuda()
    x[0, :4] = torch.tensor([0.0, -0.0, 1e-4, -1e-4]).to(dtype)
    for p, q in [(0.3, -1.2), (-4.0, 5.0)]:
        act = torch.tensor([p, q]).cuda()
        out = torch.empty(T, n, dtype=dtype, device="cuda")
        ops.xielu(x, n, act, out)
        ref = plain.xielu(x[:, :n].double().cpu(), torch.tensor(p).double(), torch.tensor(q).double())
        err = (out.double().cpu() - ref).abs() / (1 + ref.abs())
        assert err.max() < tol(dtype, 1e-6, 5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("own", [True, False])
@pytest.mark.parametrize("na", [20, 18, 300])
def test_latent_norms_and_cache_write(ops, dtype, own, na):
    nb = 40 if own else 0
    mgr, batch, _ = make_batch(ops, [(5, 3), (0, 9), (11, 1)], rank=40, page_size=4, dtype=dtype)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(batch.num_tokens, na + nb, generator=g).to(dtype).cuda()
    wa = (1 + 0.2 * torch.randn(na, generator=g)).to(dtype).cuda()
    wb = (1 + 0.2 * torch.randn(40, generator=g)).to(dtype).cuda()
    cache = mgr.view(0).paged.keys
    cache.fill_(7.0)
    out = torch.empty(batch.num_tokens, na, dtype=dtype, device="cuda")
    ops.latent_norm_store(x, na, nb, wa, wb if own else None, 1e-5, out,
                          batch.groups[0].slot_map if own else None, cache if own else None)
    xd = x.double().cpu()
    assert (out.double().cpu() - plain.rms_norm(xd[:, :na], wa.double().cpu(), 1e-5)).abs().max() < tol(dtype, 1e-5)
    # the same from float32 partial sums of the projection
    parts = torch.randn(3, batch.num_tokens, na + nb, generator=g).cuda()
    out2 = torch.empty_like(out)
    cache2 = torch.full_like(cache, 7.0)
    ops.latent_norm_store(parts, na, nb, wa, wb if own else None, 1e-5, out2,
                          batch.groups[0].slot_map if own else None, cache2 if own else None)
    pd = parts.double().sum(0).cpu()
    assert (out2.double().cpu() - plain.rms_norm(pd[:, :na], wa.double().cpu(), 1e-5)).abs().max() < tol(dtype, 1e-5)
    if own:
        got = cache2.reshape(-1, 40).double().cpu()[batch.groups[0].slot_map.cpu().long()]
        assert (got - plain.rms_norm(pd[:, na:], wb.double().cpu(), 1e-5)).abs().max() < tol(dtype, 1e-5)
    flat = cache.reshape(-1, 40).double().cpu()
    slots = batch.groups[0].slot_map.cpu().long()
    if own:
        ref = plain.rms_norm(xd[:, na:], wb.double().cpu(), 1e-5)
        assert (flat[slots] - ref).abs().max() < tol(dtype, 1e-5)
        untouched = torch.ones(flat.shape[0], dtype=torch.bool)
        untouched[slots] = False
        assert (flat[untouched] == 7.0).all()
    else:
        assert (flat == 7.0).all()


# ------------------------------------------------------------------ the short convolution
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_taps_in_portions(ops, dtype, taps):
    """Two sequences fed in portions of unequal sizes (some shorter than the taps reach), in one
    batch; a third starts later in the slot that the first gave back."""
    g = torch.Generator().manual_seed(taps)
    H = 36 if taps != 4 else 1030          # four columns a thread, or (1030) one
    w = (0.5 * torch.randn(H, taps, generator=g))
    seqs = {"a": torch.randn(23, H, generator=g).to(dtype), "b": torch.randn(9, H, generator=g).to(dtype),
            "c": torch.randn(6, H, generator=g).to(dtype)}
    ref = {k: plain.causal_taps(v.double(), w.double()) for k, v in seqs.items()}
    state_needs = StateNeeds({"taps": ((taps - 1, H), dtype)}) if taps > 1 else None
    mgr = CacheManager([CacheNeeds(paged=PagedKVNeeds(1, 8, None, value_dim=0), state=state_needs)],
                       [None], num_pages=64, page_size=4, max_requests=2, max_positions=64,
                       dtype=dtype, device="cuda")
    builder = BatchBuilder(mgr, device="cuda", q_tile_sizes=ops.q_tile_sizes)
    state = mgr.view(0).state.get("taps")
    plan = [{"a": 1, "b": 2}, {"a": 2}, {"a": 1, "b": 5}, {"a": 8, "b": 1}, {"b": 1, "a": 1},
            {"a": 10}, {"c": 2}, {"c": 1}, {"c": 3}]
    fed = {k: 0 for k in seqs}
    for step in plan:
        entries = []
        for rid, n in step.items():
            if not mgr.is_registered(rid):
                mgr.register(rid)
            mgr.reserve(rid, n)
            entries.append(StepEntry(rid, [0] * n, []))
        batch, order = builder.build(entries)
        rows = torch.cat([seqs[entries[i].request][fed[entries[i].request]:fed[entries[i].request] + len(entries[i].tokens)]
                          for i in order]).cuda()
        out = torch.empty_like(rows)
        ops.causal_taps(rows, w.t().contiguous().cuda(), state, batch, out)
        at = 0
        for i in order:
            rid, n = entries[i].request, len(entries[i].tokens)
            got = out[at:at + n].double().cpu()
            assert (got - ref[rid][fed[rid]:fed[rid] + n]).abs().max() < tol(dtype, 1e-5, 4e-2), (rid, fed[rid])
            at += n
            fed[rid] += n
            mgr.commit(rid)
            if fed[rid] == seqs[rid].shape[0]:
                mgr.release(rid)


# ------------------------------------------------------------------ products per head
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [1, 5, 70])
def test_head_products(ops, dtype, T):
    g = torch.Generator().manual_seed(T)
    H, K, N = 3, 20, 44
    w = torch.randn(H, N, K, generator=g).to(dtype).cuda()
    flat = torch.randn(T, H * K, generator=g).to(dtype).cuda()
    y = ops.head_product(flat.view(T, H, K), w, heads_first=True)
    ref = torch.einsum("thk,hnk->htn", flat.view(T, H, K).double(), w.double())
    assert y.shape == (H, T, N) and (y.double() - ref).abs().max() < tol(dtype, 1e-4, 0.2)
    x = torch.randn(H, T, K, generator=g).to(dtype).cuda()
    y = ops.head_product(x, w, heads_first=False)
    ref = torch.einsum("htk,hnk->thn", x.double(), w.double())
    assert y.shape == (T, H, N) and y.is_contiguous()
    assert (y.double() - ref).abs().max() < tol(dtype, 1e-4, 0.2)


# ------------------------------------------------------------------ attention over the latent cache
def run_latent_attention(ops, requests, *, heads, rank, window, page_size, dtype, sinks, plant=None,
                         seed=0, scale=0.3, mma=True):
    """Fill the cache with the latents of whole sequences, run the kernel on the step's rows and
    compare with the plain attention over the same sequences (key = value = latent for every
    head).  `plant(seqs, queries)` may scale latents and queries before they are stored."""
    g = torch.Generator().manual_seed(seed)
    mgr, batch, order = make_batch(ops, requests, rank=rank, window=window, page_size=page_size,
                                   dtype=dtype, seed=seed)
    seqs = [torch.randn(c + q, rank, generator=g).to(dtype) for c, q in requests]
    queries = [torch.randn(c + q, heads, rank, generator=g).to(dtype) for c, q in requests]
    if plant is not None:
        plant(seqs, queries)
    cache = mgr.view(0).paged.keys
    flat = cache.view(-1, rank)
    tables = mgr.groups[0].tables
    # positions whose page the window group already gave back are not in the cache any more
    for i, (c, q) in enumerate(requests):
        slot = mgr.slot(i)
        for p in range(c + q):
            page = int(tables[slot, p // page_size])
            if page >= 0:
                flat[page * page_size + p % page_size] = seqs[i][p].cuda()
    rows = torch.cat([queries[i][requests[i][0]:] for i in order])          # [T, H, R]
    q_dev = rows.transpose(0, 1).contiguous().cuda()                        # [H, T, R]
    out = torch.full_like(q_dev, float("nan"))
    was = ops.use_mma_latent
    ops.use_mma_latent = mma          # bfloat16: the tensor-core kernel, or the one on the CUDA cores
    try:
        ops.latent_attention(q_dev, cache, batch, batch.groups[0], heads, rank, scale, window,
                             None if sinks is None else sinks.cuda(), out)
    finally:
        ops.use_mma_latent = was
    got = out.transpose(0, 1).double().cpu()
    sink = sinks.double() if sinks is not None else torch.full((heads,), -1e30, dtype=torch.float64)
    at = 0
    worst = 0.0
    for i in order:
        c, q = requests[i]
        kv = seqs[i].double()[:, None, :].expand(-1, heads, -1)
        ref = plain.windowed_sink_attention(queries[i].double(), kv, kv, scale, window, sink, first=c)[c:]
        worst = max(worst, (got[at:at + q] - ref).abs().max().item())
        at += q
    return worst


@pytest.mark.parametrize("dtype, mma", [(torch.float32, False), (torch.bfloat16, False),
                                        (torch.bfloat16, True)])
@pytest.mark.parametrize("rank, heads, page_size", [(40, 3, 8), (64, 7, 16), (24, 1, 4), (136, 2, 16),
                                                    (36, 5, 16)])
def test_latent_attention_random(ops, dtype, mma, rank, heads, page_size):
    sinks = torch.tensor([0.5, -2.0, 3.0, 0.0, 1.0, -1.0, 2.0])[:heads]
    for window in (None, 1, 7, 33):
        reqs = [(0, 50), (37, 1), (3, 20), (0, 1), (64, 17), (31, 2), (90, 1)]
        err = run_latent_attention(ops, reqs, heads=heads, rank=rank, window=window,
                                   page_size=page_size, dtype=dtype, sinks=sinks, seed=rank, mma=mma)
        assert err < tol(dtype, 2e-5, 3e-2), (window, err)
    err = run_latent_attention(ops, [(0, 40), (20, 1)], heads=heads, rank=rank, window=9,
                               page_size=page_size, dtype=dtype, sinks=None, mma=mma)
    assert err < tol(dtype, 2e-5, 3e-2)


@pytest.mark.parametrize("rank, heads", [(512, 5), (264, 70), (128, 66), (64, 130)])
def test_latent_attention_wide_and_many_heads(ops, rank, heads):
    """The tensor-core kernel at its widest latent (output columns split over two warps), with
    more heads than one CTA of a single-token request holds, and with single-token requests
    whose keys span several chunks (with a window, and without one over a long context)."""
    sinks = torch.linspace(-2, 2, heads)
    reqs = [(0, 37), (700, 1), (255, 1), (256, 1), (40, 19), (1023, 1), (0, 1)]
    for window in (None, 300, 257, 64):
        err = run_latent_attention(ops, reqs, heads=heads, rank=rank, window=window, page_size=16,
                                   dtype=torch.bfloat16, sinks=sinks, seed=rank, scale=0.12)
        assert err < 3e-2, (window, err)
    err = run_latent_attention(ops, reqs, heads=heads, rank=rank, window=None, page_size=16,
                               dtype=torch.bfloat16, sinks=None, seed=1, scale=0.12)
    assert err < 3e-2


@pytest.mark.parametrize("dtype, mma", [(torch.float32, False), (torch.bfloat16, False),
                                        (torch.bfloat16, True)])
@pytest.mark.parametrize("decode", [False, True])
def test_planted_key_far_back_and_at_window_edges(ops, dtype, mma, decode):
    """One key gets a score far above the rest.  Without a window it lies hundreds of positions
    back; with a window of W it lies exactly W - 1 back (the last key seen) and exactly W back
    (the first key not seen), with the edge on and beside page borders."""
    rank, heads, ps = 32, 2, 16
    sinks = torch.tensor([0.3, -0.7])

    def planter(query_pos, key_pos):
        def plant(seqs, queries):
            direction = torch.zeros(rank)
            direction[5] = 1.0
            seqs[0][key_pos] = (6.0 * direction).to(seqs[0].dtype)
            queries[0][query_pos] = (8.0 * direction)[None, :].expand(heads, -1).to(seqs[0].dtype)
        return plant

    total = 420
    last = total - 1
    reqs = [(last, 1)] if decode else [(total - 100, 100)]
    # far back, no window: the planted key carries (nearly) the whole output
    err = run_latent_attention(ops, reqs, heads=heads, rank=rank, window=None, page_size=ps,
                               dtype=dtype, sinks=sinks, plant=planter(last, 3), mma=mma)
    assert err < tol(dtype, 2e-5, 5e-2)
    for W in (16, 17, 40, 48, 49, 129, 256, 321):
        for back in (W - 1, W):            # just inside, just outside
            err = run_latent_attention(ops, reqs, heads=heads, rank=rank, window=W, page_size=ps,
                                       dtype=dtype, sinks=sinks, plant=planter(last, last - back),
                                       mma=mma)
            assert err < tol(dtype, 2e-5, 5e-2), (W, back, err)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink_counts_once_and_unscaled(ops, dtype):
    """With one visible key (window 1) the output is value * e^s / (e^s + e^sink): the sink enters
    the denominator once, as it is (not multiplied by the scale)."""
    rank, heads = 16, 2
    sinks = torch.tensor([2.0, -1.0])
    for scale in (0.25, 1.0):
        err = run_latent_attention(ops, [(0, 5), (9, 1)], heads=heads, rank=rank, window=1,
                                   page_size=4, dtype=dtype, sinks=sinks, scale=scale)
        assert err < tol(dtype, 2e-5, 3e-2)
    # the same through the closed form, for the single-token request
    g = torch.Generator().manual_seed(0)
    mgr, batch, _ = make_batch(ops, [(6, 1)], rank=rank, window=1, page_size=4, dtype=dtype)
    c = torch.randn(rank, generator=g).to(dtype)
    q = torch.randn(heads, 1, rank, generator=g).to(dtype).cuda()
    cache = mgr.view(0).paged.keys
    cache.view(-1, rank)[int(batch.groups[0].slot_map[0])] = c.cuda()
    out = torch.empty_like(q)
    ops.latent_attention(q, cache, batch, batch.groups[0], heads, rank, 0.5, 1, sinks.cuda(), out)
    s = 0.5 * (q.double().cpu()[:, 0] @ c.double())
    ref = (torch.exp(s) / (torch.exp(s) + torch.exp(sinks.double())))[:, None] * c.double()[None]
    assert (out.double().cpu()[:, 0] - ref).abs().max() < tol(dtype, 1e-5, 3e-2)
