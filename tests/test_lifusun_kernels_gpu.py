"""Each CUDA kernel of the Lifusun mixers alone against its plain restatement (tests/torch_kernels.py), at sizes that
are no multiples of anything convenient, and with inputs made so that a fault at an edge would show: a key just
outside a chunk that would take all the weight, a far key that a decaying state must still hold, requests that bring
fewer tokens than the convolution has taps, pages in shuffled order."""
import math
from types import SimpleNamespace

import pytest
import torch

import torch_kernels as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from iitj_llm_coopt_b200 import kernels
    return kernels.load()


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def close(got, want, dtype, what=""):
    err = (got.float() - want.float()).abs().max().item() / max(want.float().abs().max().item(), 1e-9)
    assert err <= tol(dtype), (what, err)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps,own", [(3, 1, 12, 20, 4, True), (4, 2, 16, 8, 2, True), (2, 2, 24, 24, 6, False),
                                                              (8, 8, 96, 64, 1, True), (5, 5, 8, 8, 0, True), (3, 1, 5, 7, 3, True)])
def test_conv_norm_store(K, dtype, heads, kv_heads, dim, vdim, taps, own):
    torch.manual_seed(heads * 100 + taps)
    lens = [5, 1, 2, 9]                       # requests that bring fewer tokens than taps - 1 keep part of their old state
    T, B = sum(lens), len(lens)
    C = heads * dim + (kv_heads * (dim + vdim) if own else 0)
    u = torch.randn(T, C, device=DEV).to(dtype)
    bias = torch.randn(C, device=DEV) * 0.3
    taps_w = torch.randn(C, taps, device=DEV) if taps else None
    qg, kg = torch.rand(heads * dim, device=DEV) + 0.5, torch.rand(kv_heads * dim, device=DEV) + 0.5
    back = max(taps - 1, 0)
    state = torch.randn(7, back, C, device=DEV) if back else None
    state[3].zero_() if back else None        # slot 3: a new request (zeros before its first token)
    slots_b = [5, 3, 0, 6]
    page, pages = 4, 12
    cache = torch.zeros(pages, kv_heads * page * (dim + vdim), device=DEV, dtype=dtype) if own else None
    perm = torch.randperm(pages * page)[:T].tolist()
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    treq = [b for b, n in enumerate(lens) for _ in range(n)]
    want_q, want_k, want_v, new = R.ref_conv_norm_store(u, bias, taps_w, qg, kg, state, slots_b, cu, heads, kv_heads, dim, vdim, 1e-5, own)
    q_out = torch.empty(T, heads * dim, device=DEV, dtype=dtype)
    st = state.clone() if back else None
    K.conv_norm_store(u, bias, taps_w, qg, kg if own else None, st, i32(slots_b), i32(treq), i32(cu), q_out, cache,
                      i32(perm) if own else None, heads, kv_heads, dim, vdim, 1e-5)
    close(q_out, want_q, dtype, "q")
    if own:
        kp = cache[:, :kv_heads * page * dim].view(pages, kv_heads, page, dim)
        vp = cache[:, kv_heads * page * dim:].view(pages, kv_heads, page, vdim)
        for t in range(T):
            p, o = divmod(perm[t], page)
            close(kp[p, :, o].reshape(-1), want_k[t], dtype, "k")
            close(vp[p, :, o].reshape(-1), want_v[t], dtype, "v")
    for slot, rows in new.items():
        assert torch.allclose(st[slot], rows, atol=1e-6), "state"
    if back:
        assert torch.equal(st[1], state[1])                # a slot of no request of the step is left alone


def paged_case(dtype, heads, kv_heads, dim, vdim, page, seqs, seed=0):
    """Keys and values of `seqs` = [(context length, rows of the step)] in shuffled pages; every request brings its last rows."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-n // page) for n, _ in seqs) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    cache = torch.randn(total_pages, kv_heads * page * (dim + vdim), generator=g).to(DEV).to(dtype)
    width = max(-(-n // page) for n, _ in seqs)
    table, treq, pos = [], [], []
    for b, (n, rows) in enumerate(seqs):
        mine = [order.pop() for _ in range(-(-n // page))]
        table.append(mine + [0] * (width - len(mine)))
        treq += [b] * rows
        pos += list(range(n - rows, n))
    meta = SimpleNamespace(block_table=i32(table), token_request=i32(treq), positions=i32(pos))
    q = torch.randn(len(pos), heads * dim, generator=g).to(DEV).to(dtype)
    return cache, meta, q


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page,chunk", [(4, 2, 16, 24, 16, 16), (6, 6, 32, 32, 8, 32), (1, 1, 12, 20, 4, 128),
                                                                (20, 5, 8, 16, 4, 8), (8, 4, 96, 80, 16, 48), (40, 8, 64, 128, 16, 0),
                                                                (3, 3, 40, 8, 32, 48)])
def test_talking_attention(K, dtype, heads, kv_heads, dim, vdim, page, chunk):
    # prompt portions that start and end inside chunks and pages beside single decoded tokens at, before and after edges
    c = chunk or 64
    seqs = [(3 * c + 5, 2 * c + 3), (c, 1), (c + 1, 1), (c - 1, 1), (1, 1), (2 * c + c // 2, 7), (5 * c, 1)]
    cache, meta, q = paged_case(dtype, heads, kv_heads, dim, vdim, page, seqs, seed=heads)
    talk = (torch.eye(heads) + 0.3 * torch.randn(heads, heads)).to(DEV)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], device=DEV)
    scale = dim ** -0.5
    want = R.ref_talking_attention(q, cache, meta.block_table, meta.token_request, meta.positions, talk, slopes, heads, kv_heads,
                                   dim, vdim, page, chunk, scale)
    out = torch.empty(q.shape[0], heads * vdim, device=DEV, dtype=dtype)
    K.talking_attention(q, cache, meta, talk, slopes, out, heads, kv_heads, dim, vdim, chunk, scale)
    close(out, want, dtype)


def tiles_of(seqs, tile=16):
    out, row = [], 0
    for b, (n, rows) in enumerate(seqs):
        for s in range(0, rows, tile):
            out.append([row + s, min(tile, rows - s), n - rows + s, b])
        row += rows
    return i32(out)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page,chunk", [(4, 2, 16, 24, 16, 16), (6, 6, 32, 32, 8, 32), (1, 1, 16, 8, 4, 128),
                                                                (20, 5, 48, 16, 4, 8), (8, 4, 96, 80, 16, 48), (32, 8, 128, 128, 16, 64),
                                                                (3, 3, 64, 8, 32, 100), (32, 4, 64, 64, 32, 64)])
def test_talking_attention_tiles_on_the_tensor_core(K, heads, kv_heads, dim, vdim, page, chunk):
    """The form that takes a tile of queries at a time (bfloat16): portions that start and end inside chunks, tiles that
    cross a chunk's edge, tiles of one row, beside single decoded tokens; against the restatement and the one-token kernel."""
    c = chunk
    seqs = [(3 * c + 5, 2 * c + 3), (c, 1), (c + 1, 1), (1, 1), (2 * c + c // 2 + 40, 37), (5 * c, 1), (17, 17), (c + 9, 16)]
    cache, meta, q = paged_case(torch.bfloat16, heads, kv_heads, dim, vdim, page, seqs, seed=heads + chunk)
    talk = (torch.eye(heads) + 0.3 * torch.randn(heads, heads)).to(DEV)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], device=DEV)
    scale = dim ** -0.5
    assert K.lib.llm_talking_attention_mma_supported(heads, kv_heads, dim, vdim, chunk, cache.shape[1])
    want = R.ref_talking_attention(q, cache, meta.block_table, meta.token_request, meta.positions, talk, slopes, heads, kv_heads,
                                   dim, vdim, page, chunk, scale)
    out = torch.full((q.shape[0], heads * vdim), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.talking_attention(q, cache, meta, talk, slopes, out, heads, kv_heads, dim, vdim, chunk, scale, tiles=tiles_of(seqs))
    close(out, want, torch.bfloat16)
    one = torch.empty_like(out)
    K.talking_attention(q, cache, meta, talk, slopes, one, heads, kv_heads, dim, vdim, chunk, scale)
    close(out, one, torch.bfloat16, "against the one-token kernel")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_talking_attention_edges_of_a_chunk(K, dtype):
    """The key just before a chunk's first position lines up with every query and would take all the weight if it were
    seen; the chunk's first key (just inside) carries a value nothing else has and must be seen by every later query of
    the chunk, the last one included."""
    heads, kv_heads, dim, vdim, page, chunk = 4, 2, 16, 16, 8, 24
    n = 3 * chunk
    cache, meta, q = paged_case(dtype, heads, kv_heads, dim, vdim, page, [(n, n)], seed=3)
    kp = cache[:, :kv_heads * page * dim].view(-1, kv_heads, page, dim)
    vp = cache[:, kv_heads * page * dim:].view(-1, kv_heads, page, vdim)
    table = meta.block_table[0].tolist()
    q[:] = 0.5
    for start in (chunk, 2 * chunk):
        out_p, out_o = divmod(start - 1, page)
        kp[table[out_p], :, out_o] = 40.0              # just outside: score 40 * 0.5 * 16 above the rest
        vp[table[out_p], :, out_o] = 1000.0
        in_p, in_o = divmod(start, page)
        vp[table[in_p], :, in_o] = -7.0                # just inside
    talk = torch.eye(heads, device=DEV)
    slopes = torch.full((heads,), 0.01, device=DEV)
    want = R.ref_talking_attention(q, cache, meta.block_table, meta.token_request, meta.positions, talk, slopes, heads, kv_heads,
                                   dim, vdim, page, chunk, 0.25)
    out = torch.empty(n, heads * vdim, device=DEV, dtype=dtype)
    K.talking_attention(q, cache, meta, talk, slopes, out, heads, kv_heads, dim, vdim, chunk, 0.25,
                        tiles=tiles_of([(n, n)]) if dtype == torch.bfloat16 else None)      # bfloat16: the tensor-core form
    others = torch.ones(n, dtype=torch.bool, device=DEV)
    others[[chunk - 1, 2 * chunk - 1]] = False           # (the planted key's own position sees it: the last key of its own chunk)
    assert out[others].float().abs().max() < 100         # no query of the next chunk saw the key just outside
    assert (out[chunk:2 * chunk - 1].float().min(dim=1).values < -0.05).all()     # every query of the chunk saw its first key
    close(out, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,rot", [(2, 32, 48, 32), (1, 20, 12, 10), (3, 24, 40, 24), (4, 8, 16, 0), (2, 64, 128, 32), (2, 160, 40, 64), (40, 32, 128, 32), (80, 32, 128, 0), (2, 18, 10, 6), (3, 7, 5, 0)])
def test_retention_scan(K, dtype, heads, dim, vdim, rot):
    torch.manual_seed(dim)
    lens = [37, 1, 2, 18]
    T = sum(lens)
    cols = 2 * heads * (dim + vdim)
    proj = torch.randn(T, cols, device=DEV).to(dtype)
    half = rot // 2
    pos = torch.cat([torch.arange(100, 100 + lens[0]), torch.tensor([0]), torch.tensor([63, 64]), torch.arange(0, lens[3])]).to(DEV)
    cos = sin = None
    if half:
        ang = pos.float().unsqueeze(1) * (1.0 / (10000.0 ** (torch.arange(half, device=DEV).float() / half)))
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    decay = torch.tensor(([0.9, 0.99, 0.999, 0.5] * 20)[:heads], device=DEV)
    state = torch.randn(6, heads, vdim, dim, device=DEV)
    state[2].zero_()
    slots, cu = [4, 2, 0, 5], [0, 37, 38, 40, 58]
    want, new = R.ref_retention(proj, cos, sin, rot, decay, state, slots, cu, heads, dim, vdim, dim ** -0.5)
    st = state.clone()
    o = torch.empty(T, heads * vdim, device=DEV)
    K.retention(proj, (cos, sin) if half else None, rot, decay, st, i32(slots), i32(cu), o, heads, dim, vdim, dim ** -0.5, write=True)
    close(o, want, torch.float32, "o")
    for slot, S in new.items():
        close(st[slot], S, torch.float32, "state")
    assert torch.equal(st[1], state[1]) and torch.equal(st[3], state[3])
    st2 = state.clone()
    K.retention(proj, (cos, sin) if half else None, rot, decay, st2, i32(slots), i32(cu), o, heads, dim, vdim, dim ** -0.5, write=False)
    assert torch.equal(st2, state)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,rot,lens", [(3, 32, 16, 16, [700, 300, 5, 129]), (2, 64, 64, 64, [257]), (1, 20, 12, 10, [1000, 1]),
                                                     (16, 64, 64, 64, [4100])])
def test_retention_long_portions_in_segments(K, dtype, heads, dim, vdim, rot, lens):
    """Portions long enough to be walked in segments side by side and mended in a second pass, beside short ones that
    are not; states that are not zero at the start; the state afterwards."""
    torch.manual_seed(sum(lens))
    T, B = sum(lens), len(lens)
    proj = (torch.randn(T, 2 * heads * (dim + vdim), device=DEV) * 0.5).to(dtype)
    half = rot // 2
    pos = torch.cat([torch.arange(50 * b, 50 * b + n) for b, n in enumerate(lens)]).to(DEV)
    ang = pos.float().unsqueeze(1) * (1.0 / (10000.0 ** (torch.arange(half, device=DEV).float() / half)))
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    decay = torch.tensor(([0.9, 0.99, 0.999, 0.9995] * 4)[:heads], device=DEV)
    state = torch.randn(B + 2, heads, vdim, dim, device=DEV)
    slots = list(range(B, 0, -1))
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    want, new = R.ref_retention(proj, cos, sin, rot, decay, state, slots, cu, heads, dim, vdim, dim ** -0.5)
    st = state.clone()
    o = torch.empty(T, heads * vdim, device=DEV)
    K.retention(proj, (cos, sin), rot, decay, st, i32(slots), i32(cu), o, heads, dim, vdim, dim ** -0.5, write=True, longest=max(lens))
    close(o, want, torch.float32, "o")
    for slot, S in new.items():
        close(st[slot], S, torch.float32, "state")
    assert torch.equal(st[0], state[0]) and torch.equal(st[B + 1], state[B + 1])


def test_retention_plain_form_in_segments(K):
    """Sizes that are no multiples of 4 take the form without a register tile; long portions of it are walked in segments too."""
    test_retention_long_portions_in_segments(K, torch.float32, 3, 18, 10, 6, [700, 300, 5, 129])
    before = K.retention_segments
    K.retention_segments = 4          # the measurement switch: the plain form for sizes the register tile would take
    try:
        test_retention_long_portions_in_segments(K, torch.bfloat16, 3, 32, 16, 16, [700, 300, 5, 129])
    finally:
        K.retention_segments = before


def test_retention_keeps_a_far_key(K):
    """600 tokens; only the first one has a key that the last query lines up with, and a value nothing else has: what the
    last token reads is that value, decayed 599 times."""
    heads, dim, vdim, T = 1, 16, 8, 600
    proj = torch.zeros(T, 2 * heads * (dim + vdim), device=DEV)
    proj[:, dim:2 * dim] = 0.01 * torch.randn(T, dim, device=DEV)
    proj[:, 2 * dim:2 * dim + vdim] = 0.01 * torch.randn(T, vdim, device=DEV)
    proj[0, dim:2 * dim] = 4.0
    proj[0, 2 * dim:2 * dim + vdim] = torch.arange(1, vdim + 1, device=DEV).float()
    proj[T - 1, :dim] = 1.0
    decay = torch.tensor([1 - 2.0 ** -11], device=DEV)
    state = torch.zeros(2, heads, vdim, dim, device=DEV)
    o = torch.empty(T, vdim, device=DEV)
    want, _ = R.ref_retention(proj, None, None, 0, decay, state, [1], [0, T], heads, dim, vdim, 0.25)
    # in three portions, the state carried in between
    for lo, hi in ((0, 1), (1, 333), (333, T)):
        K.retention(proj[lo:hi].contiguous(), None, 0, decay, state, i32([1]), i32([0, hi - lo]), o[lo:hi], heads, dim, vdim, 0.25,
                    longest=hi - lo)         # (the portions of 332 and 267 tokens are walked in segments)
    expect = 4.0 * 0.25 * dim * float(decay) ** (T - 1) * torch.arange(1, vdim + 1).float()
    assert (o[T - 1].cpu() - expect).abs().max() < 0.05 * expect.max()
    close(o, want, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim", [(2, 32), (3, 40), (5, 8), (2, 128)])
def test_headnorm_gate(K, dtype, heads, vdim):
    T = 9
    o = torch.randn(T, heads * vdim, device=DEV) * 3
    proj = torch.randn(T, 50 + heads * vdim, device=DEV).to(dtype)
    out = torch.empty(T, heads * vdim, device=DEV, dtype=dtype)
    K.headnorm_gate(o, proj, 50, out, heads, vdim, 1e-5)
    close(out, R.ref_headnorm_gate(o, proj[:, 50:], heads, vdim, 1e-5), dtype)
