"""Each mechanism of the Damadra layers alone, on the device, against the plain statement of
tests/plain_damadra.py: the scaled embedding with its rounded copy, the norm on a sublayer's output with the
residual sum (single rows and stacks of partial sums), the preparation of queries, keys and values (norm per head
or over the whole projection, warm-up with position, values that are the keys, the stores into pages), the
attention with a learned bias by distance (a far key among hundreds, keys just inside and just outside the window,
page borders; prompt portions and single tokens; plain and tensor-core kernels), and the router with identity
experts, the gated squared-relu activation and the identity share."""
from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

import plain_damadra as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gen(seed):
    return torch.Generator().manual_seed(seed)


# ------------------------------------------------------------------ embedding, output norm
def test_scaled_embedding_and_its_rounded_copy():
    from reinfer_b200 import ops
    g = _gen(1)
    table = torch.randn(37, 24, generator=g).to(torch.bfloat16)
    ids = torch.tensor([3, 36, 0, 3, 17], dtype=torch.int32)
    out = torch.empty(5, 24, device=DEV)
    rounded = torch.empty(5, 24, dtype=torch.bfloat16, device=DEV)
    ops.embed_gather(table.to(DEV), ids.to(DEV), out, scale=7.5, rounded=rounded)
    ref = table[ids.long()].float() * 7.5
    assert torch.equal(out.cpu(), ref) and torch.equal(rounded.cpu(), ref.to(torch.bfloat16))
    ops.embed_gather(table.to(DEV), ids.to(DEV), out)                  # scale 1, no copy: the rows themselves
    assert torch.equal(out.cpu(), table[ids.long()].float())


@pytest.mark.parametrize("h", [52, 64, 200, 1030, 4096])
@pytest.mark.parametrize("parts", [1, 3])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_output_norm_adds_to_the_stream(h, parts, wdtype):
    from reinfer_b200 import ops
    g = _gen(h + parts)
    rows, eps, mult = 5, 1e-5, 0.7
    x = torch.randn(rows, h, generator=g)
    y = torch.randn(parts, rows, h, generator=g) * 3
    w = (torch.randn(h, generator=g) * 0.2 + 1).to(wdtype)
    ref = x.double() + mult * plain.rms(y.double().sum(0), eps) * w.double()
    xd = x.to(DEV)
    rounded = torch.empty(rows, h, dtype=torch.bfloat16, device=DEV)
    ops.residual_outnorm(xd, y.to(DEV) if parts > 1 else y[0].to(DEV), w.to(DEV), eps, mult, rounded=rounded)
    assert (xd.cpu().double() - ref).abs().max() < 2e-5
    assert torch.equal(rounded.cpu(), xd.cpu().to(torch.bfloat16))
    # with a multiple of other rows joining y before the norm
    a = torch.rand(rows, generator=g)
    for sdt in (torch.float32, torch.bfloat16):
        src = torch.randn(rows, h, generator=g).to(sdt)
        ref2 = x.double() + mult * plain.rms(y.double().sum(0) + a.double()[:, None] * src.double(), eps) * w.double()
        x2 = x.to(DEV)
        ops.residual_outnorm(x2, y.to(DEV) if parts > 1 else y[0].to(DEV), w.to(DEV), eps, mult, extra=(a.to(DEV), src.to(DEV)))
        assert (x2.cpu().double() - ref2).abs().max() < 2e-5
    # a row's result does not depend on the rows beside it
    x1 = x[2:3].to(DEV).contiguous()
    ops.residual_outnorm(x1, y[:, 2:3].contiguous().to(DEV) if parts > 1 else y[0, 2:3].contiguous().to(DEV), w.to(DEV), eps, mult)
    assert torch.equal(x1.cpu()[0], xd.cpu()[2])


# ------------------------------------------------------------------ queries, keys and values
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("QH,KH,d,dv,whole,vkeys,temp", [(6, 3, 16, 24, False, False, (0.4, 5)), (4, 2, 16, 16, True, True, None),
                                                         (3, 3, 12, 20, False, False, None), (8, 1, 32, 16, False, False, (0.6, 1)),
                                                         (70, 70, 8, 8, False, False, (0.3, 64)), (2, 1, 40, 40, True, True, (0.2, 3))])
def test_heads_are_prepared_and_stored(dtype, QH, KH, d, dv, whole, vkeys, temp):
    from reinfer_b200 import ops
    g = _gen(QH * d + dv)
    T, page, eps = 9, 4, 1e-5
    width = (QH + KH) * d + (0 if vkeys else KH * dv)
    x = (torch.randn(T, width, generator=g) * 2).to(dtype)
    qw = torch.randn(QH * d if whole else d, generator=g) * 0.2 + 1
    kw = torch.randn(KH * d if whole else d, generator=g) * 0.2 + 1
    positions = torch.tensor([0, 1, 4, 5, 63, 64, 127, 128, 700], dtype=torch.int32)
    slots = torch.tensor([5, 0, 22, 23, 9, -1, 13, 2, 31], dtype=torch.int32)          # one padding row stores nothing
    pages = 8
    cache = torch.full((pages, KH * page * (d + dv)), 77.0, dtype=dtype, device=DEV)
    q_out = torch.empty(T, QH, d, dtype=dtype, device=DEV)
    ops.norm_heads_append(x.to(DEV), qw.to(DEV), kw.to(DEV), positions.to(DEV), slots.to(DEV), q_out, cache, QH, KH, d, dv,
                          QH * d if whole else d, KH * d if whole else d, vkeys, page, eps, temp=temp)
    xd = x.double()
    q, k = xd[:, :QH * d], xd[:, QH * d:(QH + KH) * d]
    v = k if vkeys else xd[:, (QH + KH) * d:]
    if whole:
        qn, kn = plain.rms(q, eps) * qw.double(), plain.rms(k, eps) * kw.double()
    else:
        qn = (plain.rms(q.view(T, QH, d), eps) * qw.double()).view(T, -1)
        kn = (plain.rms(k.view(T, KH, d), eps) * kw.double()).view(T, -1)
    if temp is not None:
        warm = 1.0 + temp[0] * torch.log(torch.floor((positions.double() + 1) / temp[1]) + 1)
        qn = qn * warm[:, None]
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (q_out.double().cpu().view(T, -1) - qn).abs().max() <= tol * qn.abs().max()
    c = cache.double().cpu()
    touched = torch.zeros_like(c, dtype=torch.bool)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        pg, off = s // page, s % page
        for hh in range(KH):
            a = (hh * page + off) * d
            assert (c[pg, a:a + d] - kn[t, hh * d:(hh + 1) * d]).abs().max() <= tol * kn.abs().max()
            b = KH * page * d + (hh * page + off) * dv
            assert (c[pg, b:b + dv] - v[t, hh * dv:(hh + 1) * dv]).abs().max() <= tol * v.abs().max()
            touched[pg, a:a + d] = True
            touched[pg, b:b + dv] = True
    assert (c[~touched] == 77.0).all()                      # nothing else was written
    # a layer that reads another's keys and values prepares its queries only
    q_only = torch.empty(T, QH, d, dtype=dtype, device=DEV)
    ops.norm_heads_append(x[:, :QH * d].contiguous().to(DEV), qw.to(DEV), None, positions.to(DEV), None, q_only, None, QH, KH, d, dv,
                          QH * d if whole else d, KH * d if whole else d, vkeys, page, eps, temp=temp)
    assert torch.equal(q_only, q_out)


# ------------------------------------------------------------------ attention with a bias by distance
def _paged(k, v, page, KH, dk, dv, pages_total, table):
    """Scatter k [n, KH, dk], v [n, KH, dv] into a cache [pages][K | V] by a block table (-1: the page was given back)."""
    cache = torch.full((pages_total, KH * page * (dk + dv)), float("nan"), dtype=k.dtype)
    for pos in range(k.shape[0]):
        pg, off = table[pos // page], pos % page
        if pg < 0:
            continue
        for h in range(KH):
            a = (h * page + off) * dk
            cache[pg, a:a + dk] = k[pos, h]
            b = KH * page * dk + (h * page + off) * dv
            cache[pg, b:b + dv] = v[pos, h]
    return cache


def _bias_table(rel, far):
    rows = rel.shape[0]
    return torch.stack([rel[plain.distance_bucket(n, rows, far)] for n in range(far + 1)]).float().t().contiguous()     # [heads, distances]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("QH,KH,dk,dv,window,page,rows,far", [(6, 3, 16, 24, 0, 8, 8, 30), (4, 2, 16, 16, 11, 8, 10, 30),
                                                              (3, 3, 12, 20, 0, 4, 6, 21), (8, 1, 32, 16, 0, 16, 20, 300),
                                                              (4, 1, 32, 32, 16, 16, 32, 300), (4, 2, 128, 64, 0, 64, 32, 200),
                                                              (4, 4, 64, 64, 100, 64, 16, 150), (2, 2, 24, 24, 1, 8, 4, 9),
                                                              (2, 1, 64, 128, 70, 16, 12, 64), (4, 2, 128, 128, 0, 64, 32, 200),
                                                              (4, 4, 128, 128, 100, 16, 16, 150), (8, 1, 128, 128, 64, 8, 8, 20)])
def test_biased_attention_sees_what_it_should(dtype, QH, KH, dk, dv, window, page, rows, far):
    """Keys made to stand out (a large key along a direction every query has a share of): the very first key of the
    request (far back, hundreds of keys away for the causal form), and for the windowed form the key just inside
    and the key just outside the window of chosen rows.  The one that may be seen must win its row, the other must not
    be seen; whole prompt, token by token, and in pieces that end at page borders and inside pages."""
    from reinfer_b200 import ops
    g = _gen(40 + window + dk)
    n = 330 if not window else 3 * window + 37
    q = torch.randn(n, QH, dk, generator=g)
    k = torch.randn(n, KH, dk, generator=g)
    v = torch.randn(n, KH, dv, generator=g)
    q[:, :, 0] = 2.0
    rel = torch.randn(rows, QH, generator=g)
    scale = 0.3
    marked = []
    if not window:
        k[0, :, 0] = 30.0                                        # far back: seen by every row
    else:
        for i in (window + 5, 2 * window + 9, n - 1):
            k[i - window + 1, :, 0] = 30.0                       # just inside row i's window (its oldest key)
            k[i - window, :, 0] = 45.0                           # just outside
            marked.append(i)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    n_pages = -(-n // page)
    table = torch.randperm(n_pages + 3, generator=g)[:n_pages].tolist()
    cache = _paged(k, v, page, KH, dk, dv, n_pages + 3, table).to(DEV)
    bt = torch.tensor([table], dtype=torch.int32, device=DEV)
    group = SimpleNamespace(block_table=bt, page_size=page)
    bias = _bias_table(rel, far).to(DEV)
    ref = plain.softmax_attention(q.double(), k.double(), v.double(), scale, plain.distance_bias(n, rel.double(), far), window or None)
    tol = 1e-5 if dtype == torch.float32 else 2e-2

    def run(lo, hi):
        T = hi - lo
        ctx = SimpleNamespace(tok_entry=torch.zeros(T, dtype=torch.int32, device=DEV),
                              positions=torch.arange(lo, hi, dtype=torch.int32, device=DEV),
                              n_decode=1 if T == 1 else 0, n_entries=1, q_start=[0, T], start_pos=[lo], max_kv_len=hi, decode_kv_tiles=None,
                              cu_q=torch.tensor([0, T], dtype=torch.int32, device=DEV),
                              kv_len=torch.tensor([hi], dtype=torch.int32, device=DEV))
        out = torch.empty(T, QH, dv, dtype=dtype, device=DEV)
        ops.biased_attention(ctx, q[lo:hi].contiguous().to(DEV), cache, group, out, QH, KH, dk, dv, window, scale, bias)
        return out.double().cpu()

    whole = run(0, n)
    assert (whole - ref).abs().max() <= tol * ref.abs().max()
    one_by_one = torch.cat([run(i, i + 1) for i in range(n)])
    assert (one_by_one - ref).abs().max() <= tol * ref.abs().max()
    cuts = [0, 2, page, 2 * page + 1, 3 * page, n // 2, n // 2 + 2, n - page - 1, n]
    cuts = sorted(set(c for c in cuts if 0 <= c <= n))
    pieces = torch.cat([run(a, b) for a, b in zip(cuts, cuts[1:])])
    assert (pieces - ref).abs().max() <= tol * ref.abs().max()
    # the plain statement itself: the marked key takes its row (else the test would show nothing)
    if not window:
        assert (ref[n - 1, 0] - v[0, 0].double()).abs().max() < 1e-3 * v.abs().max()
    elif window > 1:
        for i in marked:
            assert (ref[i, 0] - v[i - window + 1, 0].double()).abs().max() < 1e-3 * v.abs().max()


@pytest.mark.parametrize("d,page,window", [(16, 8, 11), (128, 16, 8), (128, 64, 40), (64, 16, 20)])
def test_pages_behind_the_window_are_not_read(d, page, window):
    """A windowed request whose early pages went back to the pool (-1 in its table; the pool's memory holds NaN there):
    nothing of them reaches the result, in a portion and in single tokens, in every kernel - also not through what an
    earlier launch left in shared memory (a launch over a cache of NaN runs first: a skipped copy must not leave its
    place in a tile to whatever was there)."""
    from reinfer_b200 import ops
    g = _gen(3 + d)
    QH, KH, n = 4, 2, 200
    for dtype in (torch.float32, torch.bfloat16):
        q = torch.randn(n, QH, d, generator=g).to(dtype)
        k = torch.randn(n, KH, d, generator=g).to(dtype)
        v = torch.randn(n, KH, d, generator=g).to(dtype)
        rel = torch.randn(8, QH, generator=g)
        lo = 150                                              # tokens 150.. are run; keys before 150 - window + 1 are out of every window
        table = list(range(-(-n // page)))
        for p in range((lo - window + 1) // page):
            table[p] = -1
        assert table[(lo - window + 1) // page] >= 0
        cache = _paged(k, v, page, KH, d, d, len(table), table).to(DEV)
        poison = torch.full_like(cache, float("nan"))
        bt = torch.tensor([table], dtype=torch.int32, device=DEV)
        full = torch.arange(len(table), dtype=torch.int32, device=DEV).view(1, -1)
        bias = _bias_table(rel, 30).to(DEV)
        ref = plain.softmax_attention(q.double(), k.double(), v.double(), 0.25, plain.distance_bias(n, rel.double(), 30), window)
        for a, b in ((lo, n), (lo, lo + 1), (n - 1, n), (lo + 3, lo + 9)):
            T = b - a
            ctx = SimpleNamespace(tok_entry=torch.zeros(T, dtype=torch.int32, device=DEV),
                                  positions=torch.arange(a, b, dtype=torch.int32, device=DEV), n_decode=1 if T == 1 else 0, n_entries=1,
                                  q_start=[0, T], start_pos=[a], max_kv_len=b, decode_kv_tiles=None,
                                  cu_q=torch.tensor([0, T], dtype=torch.int32, device=DEV), kv_len=torch.tensor([b], dtype=torch.int32, device=DEV))
            out = torch.empty(T, QH, d, dtype=dtype, device=DEV)
            ops.biased_attention(ctx, q[a:b].contiguous().to(DEV), poison, SimpleNamespace(block_table=full, page_size=page), out, QH, KH, d, d,
                                 window, 0.25, bias)
            ops.biased_attention(ctx, q[a:b].contiguous().to(DEV), cache, SimpleNamespace(block_table=bt, page_size=page), out, QH, KH, d, d,
                                 window, 0.25, bias)
            err = (out.double().cpu() - ref[a:b]).abs().max()
            assert err <= (1e-5 if dtype == torch.float32 else 2e-2) * ref.abs().max(), (dtype, a, b, err)


def test_a_batch_of_unequal_requests_equals_each_alone():
    """Three requests in one launch - two single tokens at different lengths and a portion - against each by itself."""
    from reinfer_b200 import ops
    g = _gen(9)
    QH, KH, dk, dv, page, rows, far = 6, 2, 32, 16, 8, 12, 40
    lens = [77, 130, 52]
    new = [1, 1, 20]
    rel = torch.randn(rows, QH, generator=g)
    bias = _bias_table(rel, far).to(DEV)
    for dtype in (torch.float32, torch.bfloat16):
        qs = [torch.randn(n, QH, dk, generator=g).to(dtype) for n in lens]
        ks = [torch.randn(n, KH, dk, generator=g).to(dtype) for n in lens]
        vs = [torch.randn(n, KH, dv, generator=g).to(dtype) for n in lens]
        pages = [-(-n // page) for n in lens]
        perm = torch.randperm(sum(pages) + 2, generator=g).tolist()
        tables, at = [], 0
        for p in pages:
            tables.append(perm[at:at + p])
            at += p
        cache = torch.full((sum(pages) + 2, KH * page * (dk + dv)), float("nan"), dtype=dtype)
        for kk, vv, tb in zip(ks, vs, tables):
            part = _paged(kk, vv, page, KH, dk, dv, cache.shape[0], tb)
            for pg in tb:
                cache[pg] = part[pg]
        cache = cache.to(DEV)
        width = max(pages)
        bt = torch.full((3, width), -1, dtype=torch.int32)
        for e, tb in enumerate(tables):
            bt[e, :len(tb)] = torch.tensor(tb, dtype=torch.int32)
        group = SimpleNamespace(block_table=bt.to(DEV), page_size=page)
        q_cat = torch.cat([qq[n - m:] for qq, n, m in zip(qs, lens, new)]).contiguous().to(DEV)
        cu = [0, 1, 2, 22]
        ctx = SimpleNamespace(tok_entry=torch.tensor([0, 1] + [2] * 20, dtype=torch.int32, device=DEV),
                              positions=torch.tensor([lens[0] - 1, lens[1] - 1] + list(range(lens[2] - 20, lens[2])), dtype=torch.int32, device=DEV),
                              n_decode=2, n_entries=3, q_start=cu, start_pos=[lens[0] - 1, lens[1] - 1, lens[2] - 20], max_kv_len=max(lens),
                              decode_kv_tiles=None, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                              kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV))
        out = torch.empty(22, QH, dv, dtype=dtype, device=DEV)
        ops.biased_attention(ctx, q_cat, cache, group, out, QH, KH, dk, dv, 0, 0.2, bias)
        out = out.double().cpu()
        at = 0
        for qq, kk, vv, n, m in zip(qs, ks, vs, lens, new):
            ref = plain.softmax_attention(qq.double(), kk.double(), vv.double(), 0.2, plain.distance_bias(n, rel.double(), far), None)[n - m:]
            assert (out[at:at + m] - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * ref.abs().max()
            at += m


# ------------------------------------------------------------------ mixture of experts
@pytest.mark.parametrize("n,E,top", [(7, 5, 3), (3, 3, 1), (4, 2, 4), (12, 8, 4), (40, 33, 6), (2, 2, 2)])
def test_router_choice_and_weights(n, E, top):
    from reinfer_b200 import ops
    g = _gen(n * 10 + top)
    T = 50
    z = torch.randn(T, n, generator=g) * 2
    corr = torch.randn(n, generator=g) * 0.5
    gates, ident = ops.moe_route(z.to(DEV), corr.to(DEV), E, top)
    s = torch.softmax(z.double(), dim=-1)
    chosen = torch.topk(s + corr.double(), top, dim=-1).indices
    ref_g = torch.zeros(T, n, dtype=torch.float64)
    ref_g.scatter_(1, chosen, torch.gather(s, 1, chosen))
    assert (gates.double().cpu() - ref_g[:, :E]).abs().max() < 1e-6
    assert ((gates.cpu() != 0) == (ref_g[:, :E] != 0)).all()
    if n > E:
        assert (ident.double().cpu() - ref_g[:, E:].sum(1)).abs().max() < 1e-6
    else:
        assert ident is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("h,n,E,top", [(52, 3, 3, 1), (64, 7, 5, 3), (96, 4, 2, 4), (256, 12, 8, 4), (1000, 37, 30, 5)])
def test_router_product_and_choice_in_one(dtype, h, n, E, top):
    """The fused router against the plain route(): the same experts, the same weights; and a token's row alone gives
    the same bits as in the batch."""
    from reinfer_b200 import ops
    g = _gen(h + n)
    T = 40
    x = torch.randn(T, h, generator=g).to(dtype)
    w = (torch.randn(n, h, generator=g) * 3 / h ** 0.5).to(dtype)
    corr = torch.randn(n, generator=g) * 0.2
    gates, ident = ops.moe_router(x.to(DEV), w.to(DEV), corr.to(DEV), E, top)
    W = {"p.router": w.double(), "p.correction": corr.double()}
    chosen, weight = plain.route(x.double(), W, "p.", {"top": top})
    ref = torch.zeros(T, n, dtype=torch.float64)
    ref.scatter_(1, chosen, weight)
    assert (gates.double().cpu() - ref[:, :E]).abs().max() < 2e-6
    assert ((gates.cpu() != 0) == (ref[:, :E] != 0)).all()
    if n > E:
        assert (ident.double().cpu() - ref[:, E:].sum(1)).abs().max() < 2e-6
    g1, i1 = ops.moe_router(x[17:18].contiguous().to(DEV), w.to(DEV), corr.to(DEV), E, top)
    assert torch.equal(g1[0], gates[17]) and (ident is None or torch.equal(i1[0], ident[17]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ff", [10, 16])
def test_gated_squared_relu_and_identity_share(dtype, ff):
    from reinfer_b200 import ops
    g = _gen(5)
    T, E, h = 6, 3, 20
    u = (torch.randn(T, E * ff, generator=g) * 2).to(dtype)
    gates = torch.rand(T, E, generator=g)
    gates[gates < 0.4] = 0.0
    act = ops.relu2_gate(u.to(DEV), gates.to(DEV), ff)
    ref = torch.relu(u.double()) ** 2 * gates.double().repeat_interleave(ff, dim=1)
    assert (act.double().cpu() - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-2) * ref.abs().max()
    assert (act.cpu()[ref == 0] == 0).all()                  # an expert that was not chosen adds exact zeros
    dst = torch.randn(T, h, generator=g)
    a = torch.rand(T, generator=g)
    src = torch.randn(T, h, generator=g).to(dtype)
    d1 = dst.clone().to(DEV)
    ops.rows_axpy(d1, a.to(DEV), src.to(DEV))
    assert (d1.cpu() - (dst + a[:, None] * src.float())).abs().max() < 1e-6
    ops.rows_axpy(d1, a.to(DEV), src.to(DEV), store=True)
    assert (d1.cpu() - a[:, None] * src.float()).abs().max() < 1e-6
