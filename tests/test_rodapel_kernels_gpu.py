"""Each CUDA kernel of the Rodapel family alone against its plain restatement in tests/torch_kernels.py, at sizes that
differ from one another in everything (odd widths, head sizes that are no multiples of 8, one head, value heads wider and
narrower than key heads, one expert, every pair landing on one expert, experts nobody chooses)."""
import math
import types

import pytest
import torch

import torch_kernels as R

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def K():
    from iitj_llm_coopt_b200 import kernels
    return kernels.load()


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def close(got, want, dtype, scale=None):
    want = want.float()
    err = (got.float() - want).abs().max().item()
    ref = scale or max(want.abs().max().item(), 1e-6)
    assert err <= tol(dtype) * ref, (err, ref)


def rnd(*shape, dtype=torch.float32, seed=0, s=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * s).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,width", [(1, 8), (5, 200), (3, 2050), (2, 4099)])
def test_norm_add(K, dtype, tokens, width):
    res, branch, w = rnd(tokens, width, seed=1), rnd(tokens, width, dtype=dtype, seed=2, s=3.0), rnd(width, seed=3) + 1.0
    for accumulate in (True, False):
        r = res.clone()
        cast = torch.empty(tokens, width, dtype=torch.bfloat16, device="cuda")
        K.norm_add(r, branch, w, 1e-5, cast_out=cast, accumulate=accumulate)
        want = R.ref_norm_add(res, branch, w, 1e-5, accumulate)
        close(r, want, torch.float32)
        assert torch.equal(cast, r.to(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
def test_glu_clamped(K, dtype):
    gu = rnd(7, 2 * 37, dtype=dtype, s=3.0)
    act = torch.empty(7, 37, dtype=dtype, device="cuda")
    K.glu_clamped(gu, act, 2.0, 1.702)
    close(act, R.ref_glu_clamped(gu, 2.0, 1.702), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,groups,n,k,a_stride,lda", [(5, 3, 24, 16, 20, 70), (70, 8, 128, 64, 96, 800), (130, 1, 7, 13, 0, 13),
                                                          (33, 4, 48, 200, 33 * 200, 200)])
def test_linear_by_group(K, dtype, rows, groups, n, k, a_stride, lda):
    blocks = groups if a_stride >= rows * lda else 1
    a = rnd(blocks * rows, lda, dtype=dtype, seed=4)
    w = rnd(groups, n, k, dtype=dtype, seed=5, s=k ** -0.5)
    out = torch.zeros(rows, groups * n + 3, dtype=dtype, device="cuda")
    K.linear_by_group(a, w, out, a_stride=a_stride, out_stride=n, out_offset=3)
    want = torch.zeros_like(out, dtype=torch.float32)
    R.TorchKernels().linear_by_group(a, w, want, a_stride=a_stride, out_stride=n, out_offset=3)
    close(out, want, dtype)
    assert (out[:, :3] == 0).all()


@pytest.mark.parametrize("outputs,top", [(14, 3), (5, 5), (100, 8), (3, 1)])
def test_route_topk(K, outputs, top):
    scores, corr = rnd(9, outputs, s=2.0), rnd(outputs, seed=6, s=0.3)
    chosen = torch.empty(9, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(9, top, dtype=torch.float32, device="cuda")
    K.route_topk(scores, corr, chosen, weights)
    c, w = R.ref_route_topk(scores, corr, top)
    assert torch.equal(chosen, c)
    close(weights, w, torch.float32)


def moe_case(K, dtype, tokens, top, experts, identity, width, ff, chosen=None, seed=0):
    g = torch.Generator().manual_seed(seed)
    if chosen is None:
        chosen = torch.stack([torch.randperm(experts + identity, generator=g)[:top] for _ in range(tokens)])
    chosen = chosen.to(torch.int32).cuda()
    weights = torch.rand(tokens, top, generator=g).cuda()
    x = rnd(tokens, width, dtype=dtype, seed=seed + 1)
    w1 = rnd(experts, 2 * ff, width, dtype=dtype, seed=seed + 2, s=width ** -0.5)
    w2 = rnd(experts, width, ff, dtype=dtype, seed=seed + 3, s=ff ** -0.5)
    outs = []
    for kern in (K, R.TorchKernels()):
        rows = tokens * top
        bound = kern.moe_tile_bound(rows, experts)
        plan = kern.moe_plan(chosen, experts, torch.zeros(rows, dtype=torch.int32, device="cuda"),
                             torch.zeros(rows, dtype=torch.int32, device="cuda"), torch.zeros(bound + 1, 4, dtype=torch.int32, device="cuda"))
        act = torch.zeros(rows, ff, dtype=dtype, device="cuda")
        kern.moe_linear(x, w1, act, plan, gather=True, glu=True, limit=1.5, slope=1.702)
        y = torch.zeros(rows, width, dtype=dtype, device="cuda")
        kern.moe_linear(act, w2, y, plan)
        out = torch.zeros(tokens, width, dtype=dtype, device="cuda")
        kern.moe_combine(y, plan, chosen, weights, x, experts, out)
        outs.append((plan, out))
    (pk, ok), (pr, orf) = outs
    assert torch.equal(pk["place"], pr["place"])
    n = int(pr["rows"])
    assert torch.equal(pk["source"][:n], pr["source"][:n])
    assert int(pk["tiles"][0, 0]) == int(pr["tiles"][0, 0]) and int(pk["tiles"][0, 1]) == n
    close(ok, orf, dtype)
    # the experts' row counts for a caller that wants them on the host, and the rows gathered side by side
    rows = tokens * top
    counts = torch.full((experts,), -1, dtype=torch.int32, device="cuda")
    plan = K.moe_plan(chosen, experts, torch.zeros(rows, dtype=torch.int32, device="cuda"), torch.zeros(rows, dtype=torch.int32, device="cuda"),
                      torch.zeros(K.moe_tile_bound(rows, experts) + 1, 4, dtype=torch.int32, device="cuda"), counts=counts)
    assert counts.tolist() == [int((chosen == e).sum()) for e in range(experts)]
    side = torch.full((rows, width), 7.0, dtype=dtype, device="cuda")
    K.gather_rows(x, plan, side)
    assert torch.equal(side[:n], x[plan["source"][:n].long()]) and (side[n:] == 7.0).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_routed_experts(K, dtype):
    moe_case(K, dtype, tokens=11, top=2, experts=10, identity=3, width=40, ff=24)
    moe_case(K, dtype, tokens=150, top=2, experts=3, identity=0, width=64, ff=100, seed=3)           # several tiles per expert
    moe_case(K, dtype, tokens=70, top=1, experts=5, identity=2, width=33, ff=17,
             chosen=torch.full((70, 1), 4), seed=5)                                                  # every pair on one expert
    moe_case(K, dtype, tokens=9, top=2, experts=1, identity=3, width=16, ff=8, seed=7)               # one expert with tensors
    moe_case(K, dtype, tokens=6, top=2, experts=4, identity=2, width=16, ff=8,
             chosen=torch.tensor([[4, 5]] * 6), seed=9)                                              # nobody chooses a real expert


def paged(dtype, requests, lens, page, per_token, seed=0):
    """A shuffled page pool with a block table: returns (cache [pages, page * per_token], table [B, W])."""
    need = [-(-n // page) for n in lens]
    total = sum(need) + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total, generator=g).tolist()
    width = max(need)
    table = torch.zeros(requests, width, dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        table[b, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    cache = torch.full((total, page * per_token), float("nan"), dtype=dtype)       # what was never stored is poison
    return cache.cuda(), table.cuda()


def flat_plan(K, token_request, positions, heads, kv_heads, key_dim, value_dim, window, splits=None):
    """The step plan of the mixers over flat pages (tiles of neighbouring tokens of one request) for the tokens of a test:
    with it, and bfloat16 sizes it takes, `attention_flat` runs on the tensor cores."""
    from iitj_llm_coopt_b200.parts.base import StepShape
    from iitj_llm_coopt_b200.parts.flat_tiles import plan_flat_tiles
    lens, ends = [], []
    for i, (b, p) in enumerate(zip(token_request, positions)):
        if i and token_request[i - 1] == b and positions[i - 1] == p - 1:
            lens[-1] += 1
            ends[-1] = p + 1
        else:
            lens.append(1)
            ends.append(p + 1)
    # runs of one request must carry the request's index: the test's requests are numbered as their first run
    order = []
    for i, b in enumerate(token_request):
        if not i or token_request[i - 1] != b or positions[i - 1] != positions[i] - 1:
            order.append(b)
    plan = plan_flat_tiles(K, StepShape(lens, ends, len(token_request), False, False, "cuda"), heads, kv_heads, key_dim, value_dim, window)
    tiles = torch.tensor(plan.arrays["tiles"], dtype=torch.int32).view(-1, 4)
    tiles[:, 3] = torch.tensor([order[int(r)] for r in tiles[:, 3]], dtype=torch.int32)
    plan.bind({"tiles": tiles.reshape(-1).cuda()})
    if splits is not None:
        plan.splits = splits
    return plan


def meta_for(table, token_request, positions):
    return types.SimpleNamespace(block_table=table, token_request=torch.tensor(token_request, dtype=torch.int32).cuda(),
                                 positions=torch.tensor(positions, dtype=torch.int32).cuda())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,page", [(4, 2, 32, 48, 40, 16), (4, 4, 24, 40, 5, 4), (1, 1, 12, 7, 0, 8),
                                                                 (8, 2, 40, 16, 33, 32), (3, 1, 130, 300, 0, 16)])
def test_headnorm_store_and_attention(K, dtype, heads, kv_heads, dim, vdim, window, page):
    """Two requests: one stores 70 tokens in portions and is asked at every position, one stores 9."""
    lens = [70, 9]
    per = kv_heads * (dim + vdim)
    cache, table = paged(dtype, 2, lens, page, per, seed=dim)
    ref_cache = cache.clone()
    q_gain, k_gain = rnd(dim, seed=7) * 0.1 + 1.0, rnd(dim, seed=8) * 0.1 + 1.0
    cols = heads * dim + per
    RK = R.TorchKernels()
    done = [0, 0]
    for portion in ([33, 9], [2, 0], [35, 0]):
        req, pos = [], []
        for b, n in enumerate(portion):
            req += [b] * n
            pos += list(range(done[b], done[b] + n))
            done[b] += n
        T = len(req)
        slots = torch.tensor([int(table[b, p // page]) * page + p % page for b, p in zip(req, pos)], dtype=torch.int32).cuda()
        qkv = rnd(T, cols, dtype=dtype, seed=done[0], s=2.0)
        gate = rnd(T, heads, seed=done[0] + 1)
        meta = meta_for(table, req, pos)
        a, b_ = qkv.clone(), qkv.clone()
        K.headnorm_store(a, q_gain, k_gain, 1e-5, cache, slots, heads, kv_heads, dim, vdim)
        RK.headnorm_store(b_, q_gain, k_gain, 1e-5, ref_cache, slots, heads, kv_heads, dim, vdim)
        close(a[:, :heads * dim], b_[:, :heads * dim], dtype)
        out = torch.empty(T, heads * vdim, dtype=dtype, device="cuda")
        want = torch.empty(T, heads * vdim, dtype=torch.float32, device="cuda")
        RK.attention_flat(b_, ref_cache, meta, want, heads, kv_heads, dim, vdim, window=window, scale=0.3, gate=gate)
        for plan in (None, flat_plan(K, req, pos, heads, kv_heads, dim, vdim, window), flat_plan(K, req, pos, heads, kv_heads, dim, vdim, window, splits=3)):
            out.fill_(float("nan"))
            K.attention_flat(a, cache, meta, out, heads, kv_heads, dim, vdim, window=window, scale=0.3, gate=gate, plan=plan)
            close(out, want, dtype)
    written = ~torch.isnan(ref_cache.float())
    assert torch.equal(written, ~torch.isnan(cache.float()))
    close(cache.float()[written], ref_cache.float()[written], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot,rotary,rank,page,interleaved", [(8, 48, 16, 16, 96, 16, True), (3, 20, 12, 8, 36, 8, True),
                                                                        (1, 8, 6, 6, 10, 4, False), (5, 16, 16, 0, 24, 16, True),
                                                                        (32, 32, 64, 64, 512, 16, True), (80, 16, 16, 16, 160, 32, True)])
def test_latent_prepare_and_attention(K, dtype, heads, dim, rot, rotary, rank, page, interleaved):
    lens = [50, 3]
    row = rank + rot
    cache, table = paged(dtype, 2, lens, page, row, seed=rank)
    ref_cache = cache.clone()
    gain = rnd(rank, seed=9) * 0.1 + 1.0
    RK = R.TorchKernels()
    done = [0, 0]
    for portion in ([17, 3], [33, 0]):
        req, pos = [], []
        for b, n in enumerate(portion):
            req += [b] * n
            pos += list(range(done[b], done[b] + n))
            done[b] += n
        T = len(req)
        slots = torch.tensor([int(table[b, p // page]) * page + p % page for b, p in zip(req, pos)], dtype=torch.int32).cuda()
        qd = rnd(T, heads * (dim + rot) + row, dtype=dtype, seed=done[0])
        tables = None
        if rotary:
            inv = 1.0 / (10000.0 ** (torch.arange(0, rotary, 2).float() / rotary))
            ang = torch.tensor(pos).float().unsqueeze(1) * inv.unsqueeze(0)
            tables = (ang.cos().cuda().contiguous(), ang.sin().cuda().contiguous())
        qa = rnd(T, heads * row, dtype=dtype, seed=done[0] + 5)          # the absorbed parts stand in already
        qb = qa.clone()
        K.latent_prepare(qd, tables, rotary, interleaved, gain, 1e-5, qa, cache, slots, heads, dim, rot, rank)
        RK.latent_prepare(qd, tables, rotary, interleaved, gain, 1e-5, qb, ref_cache, slots, heads, dim, rot, rank)
        close(qa, qb, dtype)
        meta = meta_for(table, req, pos)
        out = torch.empty(T, heads * rank, dtype=dtype, device="cuda")
        want = torch.empty(T, heads * rank, dtype=torch.float32, device="cuda")
        RK.attention_flat(qb, ref_cache, meta, want, heads, 1, row, rank, shared_value=True, scale=0.2)
        for plan in (None, flat_plan(K, req, pos, heads, 1, row, rank, 0), flat_plan(K, req, pos, heads, 1, row, rank, 0, splits=2)):
            out.fill_(float("nan"))
            K.attention_flat(qa, cache, meta, out, heads, 1, row, rank, shared_value=True, scale=0.2, plan=plan)
            close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,width,rank", [(4, 40, 160, 12), (1, 7, 20, 3), (3, 64, 96, 40), (2, 100, 64, 8), (4, 32, 50, 5)])
def test_wkv(K, dtype, heads, dim, width, rank):
    """Three requests over four state slots; the second step continues two of them from the states the first left."""
    n = heads * dim
    RK = R.TorchKernels()
    mu = torch.rand(5 * width).cuda()
    u, gain = rnd(heads, dim, seed=11, s=0.5), rnd(n, seed=12) * 0.1 + 1.0
    w2, w0 = rnd(n, rank, seed=13, s=0.5), rnd(n, seed=14) - 1.0
    states = [torch.zeros(4, heads, dim, dim, device="cuda") for _ in range(2)]
    befores = [torch.zeros(4, width, device="cuda") for _ in range(2)]
    for step, (lens, slot_ids) in enumerate((([21, 1, 40], [2, 0, 3]), ([1, 18], [3, 2]))):
        T = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
        slots = torch.tensor(slot_ids, dtype=torch.int32).cuda()
        req = torch.tensor([b for b, m in enumerate(lens) for _ in range(m)], dtype=torch.int32).cuda()
        x = rnd(T, width, dtype=dtype, seed=20 + step)
        mixes = [torch.empty(5 * T, width, dtype=dtype, device="cuda"), torch.empty(5 * T, width, dtype=torch.float32, device="cuda")]
        K.token_shift(x, mu, befores[0], slots, req, cu, mixes[0])
        RK.token_shift(x, mu, befores[1], slots, req, cu, mixes[1])
        close(mixes[0], mixes[1], dtype)
        low = rnd(T, rank, seed=30 + step)
        decay = [torch.empty(T, n, device="cuda") for _ in range(2)]
        K.wkv_decay(low, w2, w0, decay[0])
        RK.wkv_decay(low, w2, w0, decay[1])
        close(decay[0], decay[1], torch.float32, scale=1.0)
        rkvg = rnd(4 * T, n, dtype=dtype, seed=40 + step)
        outs = [torch.empty(T, n, dtype=dtype, device="cuda"), torch.empty(T, n, dtype=torch.float32, device="cuda")]
        K.wkv_scan(rkvg, decay[1], u, gain, 1e-5, states[0], slots, cu, outs[0], heads, dim, last_rows=(x, befores[0]))
        RK.wkv_scan(rkvg, decay[1], u, gain, 1e-5, states[1], slots, cu, outs[1], heads, dim, last_rows=(x, befores[1]))
        close(outs[0], outs[1], dtype)
        close(states[0], states[1], torch.float32)
        assert torch.equal(befores[0], befores[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,page,total", [(16, 16, 70), (33, 8, 100), (1, 4, 9), (80, 16, 200), (0, 16, 700)])
def test_planted_keys_at_the_window_s_edges(K, dtype, window, page, total):
    """Random weights would hide a window that is one key off: here every query points along one axis, the key just outside a
    query's window (with no window: key 3, hundreds of positions back) would take all the weight if it were seen (or, with no
    window, must take it), and the first key inside carries a value of its own.  Queries are asked in a prompt portion and as
    single decoded tokens, with windows that start on a page's first and last slot."""
    heads, kv_heads, dim, vdim = 2, 1, 16, 8
    per = kv_heads * (dim + vdim)
    cache, table = paged(dtype, 1, [total], page, per, seed=window)
    g = torch.Generator().manual_seed(5)
    keys = torch.randn(total, dim, generator=g) * 0.1
    vals = torch.randn(total, vdim, generator=g)
    asked = sorted({total - 1, total - 2, min(total - 1, window + page - 1), min(total - 1, window + page), min(total - 1, 2 * page)})
    for p in asked:
        outside, first = (p - window, p - window + 1) if window else (None, 3)
        if outside is not None and outside >= 0:
            keys[outside, 0] = 40.0 + outside % 7
        if first >= 0:
            keys[first, 0] = max(keys[first, 0].item(), 8.0)
            vals[first] = 5.0 + p % 3
    kplane, vplane, ps = R.flat_planes(cache, kv_heads, dim, vdim, False)
    for j in range(total):
        pg, o = int(table[0, j // page]), j % page
        kplane[pg, 0, o] = keys[j].to(dtype)
        vplane[pg, 0, o] = vals[j].to(dtype)
    RK = R.TorchKernels()
    for rows in (asked, [asked[-1]]):                    # a portion of several queries, then one token alone
        q = torch.zeros(len(rows), heads * dim, dtype=dtype, device="cuda")
        q[:, 0], q[:, dim] = 1.0, 0.5
        meta = meta_for(table, [0] * len(rows), rows)
        out = torch.empty(len(rows), heads * vdim, dtype=dtype, device="cuda")
        want = torch.empty(len(rows), heads * vdim, dtype=torch.float32, device="cuda")
        RK.attention_flat(q, cache, meta, want, heads, kv_heads, dim, vdim, window=window, scale=1.0)
        for plan in (None, flat_plan(K, [0] * len(rows), rows, heads, kv_heads, dim, vdim, window),
                     flat_plan(K, [0] * len(rows), rows, heads, kv_heads, dim, vdim, window, splits=4)):
            out.fill_(float("nan"))
            K.attention_flat(q, cache, meta, out, heads, kv_heads, dim, vdim, window=window, scale=1.0, plan=plan)
            close(out, want, dtype)
        if window:
            assert (want[:, :vdim].amax(1) > 1.0).any()       # the planted value shows in the answer
