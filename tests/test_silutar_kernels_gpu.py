"""Each mechanism of the statistics-free / recurrent layers alone, on the device, against the plain
statement of tests/plain_silutar.py: Dynamic Tanh, learned positions, soft cap, short convolution
with its window in the slots, the three matrix-state recurrences (portions, batches, slots used
again, a memory hundreds of tokens old), the per-head output stage, and the chunk attention with its
distance penalty (keys just inside and just outside a chunk made to stand out)."""
from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch

import plain_silutar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _tables(lengths, slots):
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    return (torch.tensor(cu, dtype=torch.int32, device=DEV), torch.tensor(slots, dtype=torch.int32, device=DEV))


# ------------------------------------------------------------------ pointwise
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dyt_with_partial_sums_and_row_gather(dtype):
    from reinfer_b200 import ops
    g = _gen(1)
    T, h = 37, 200
    x = torch.randn(T, h, generator=g) * 2
    delta = torch.randn(3, T, h, generator=g)
    w, b, a = torch.randn(h, generator=g), torch.randn(h, generator=g), torch.tensor([0.7])
    wd, bd, ad = (t.to(dtype).to(DEV) for t in (w, b, a))
    xd = x.to(DEV)
    out = torch.empty(T, h, dtype=dtype, device=DEV)
    ops.dyt(xd, delta.to(DEV), wd, bd, ad, out)
    xs = x.double() + delta.double().sum(0)
    ref = plain.dyt(xs, wd.double().cpu(), bd.double().cpu(), ad.double().cpu())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (xd.double().cpu() - xs).abs().max() < 1e-5                      # the sum was written back
    assert (out.double().cpu() - ref).abs().max() <= tol * ref.abs().max()
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device=DEV)
    out2 = torch.empty(4, h, dtype=dtype, device=DEV)
    ops.dyt(xd, None, wd, bd, ad, out2, rows)
    assert torch.equal(out2, out[rows.long()])


def test_embedding_with_positions_and_soft_cap():
    from reinfer_b200 import ops
    g = _gen(2)
    table, pos = torch.randn(50, 24, generator=g).to(DEV), torch.randn(30, 24, generator=g).to(DEV)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    p = torch.tensor([0, 29, 7, 8], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 24, dtype=torch.float32, device=DEV)
    ops.embed_gather(table, ids, out, pos_table=pos, positions=p)
    assert torch.equal(out, table[ids.long()] + pos[p.long()])
    x = torch.randn(5, 33, generator=g).to(DEV) * 40
    y = x.clone()
    ops.softcap(y, 15.0)
    assert (y.double() - 15.0 * torch.tanh(x.double() / 15.0)).abs().max() < 1e-5
    assert y.abs().max() <= 15.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_gate(dtype):
    from reinfer_b200 import ops
    g = _gen(3)
    T, H, dv = 9, 3, 40
    o = torch.randn(T, H, dv, generator=g).to(DEV)
    gate_full = torch.randn(T, H * dv + 16, generator=g).to(dtype).to(DEV)
    gate = gate_full[:, 8:8 + H * dv]                               # a strided view, as a slice of a fused projection is
    for w, fn in ((torch.randn(dv, generator=g), "silu"), (torch.randn(H * dv, generator=g), "sigmoid")):
        out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
        ops.head_norm_gate(o, w.to(DEV), gate, out, H, dv, 1e-5, fn, out_scale=0.7)
        gd = gate.double().cpu().view(T, H, dv)
        act = plain.silu(gd) if fn == "silu" else plain.sigmoid(gd)
        wv = w.double().view(1, -1, dv) if w.numel() == H * dv else w.double()
        ref = (plain.rms_unit(o.double().cpu(), 1e-5) * wv * act * 0.7).view(T, H * dv)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert (out.double().cpu() - ref).abs().max() <= tol * ref.abs().max()


# ------------------------------------------------------------------ short convolution
@pytest.mark.parametrize("taps", [1, 2, 3, 5])
@pytest.mark.parametrize("silu", [False, True])
def test_short_convolution_over_portions_batches_and_reused_slots(taps, silu):
    from reinfer_b200 import ops
    g = _gen(10 + taps)
    C = 150
    w = torch.randn(C, taps, generator=g)
    state = torch.full((4, taps - 1, C), 7.0, device=DEV)           # rubbish until a request is admitted
    seqs = {"a": torch.randn(150, C, generator=g), "b": torch.randn(9, C, generator=g), "c": torch.randn(71, C, generator=g)}
    cuts = {"a": [3, 2, 70, 1, 1, 66, 7], "b": [1, 2, 2, 1, 3], "c": [65, 2, 2, 2]}
    slot = {"a": 2, "b": 0, "c": 2}                                  # c takes a's slot afterwards
    got = {r: [] for r in seqs}
    done = {r: 0 for r in seqs}
    for group in (["a", "b"], ["c"]):
        for r in group:
            state[slot[r]].zero_()
        k = 0
        while any(done[r] < len(seqs[r]) for r in group):
            live = [r for r in group if done[r] < len(seqs[r])]
            lens = [cuts[r][min(k, len(cuts[r]) - 1)] if k < len(cuts[r]) else len(seqs[r]) - done[r] for r in live]
            lens = [min(n, len(seqs[r]) - done[r]) for n, r in zip(lens, live)]
            u = torch.cat([seqs[r][done[r]:done[r] + n] for r, n in zip(live, lens)]).to(DEV)
            wide = torch.zeros(u.shape[0], C + 10, device=DEV)
            wide[:, 5:5 + C] = u                                       # rows strided
            y = torch.empty_like(u)
            cu, sl = _tables(lens, [slot[r] for r in live])
            ops.shortconv(wide[:, 5:5 + C], w.to(DEV), state, y, cu, sl, len(live), max(lens), silu)
            at = 0
            for r, n in zip(live, lens):
                got[r].append(y[at:at + n].cpu())
                at += n
                done[r] += n
            k += 1
    for r, u in seqs.items():
        ref = plain.short_conv(u.double(), w.double())
        if silu:
            ref = plain.silu(ref)
        assert (torch.cat(got[r]).double() - ref).abs().max() < 1e-5, r


# ------------------------------------------------------------------ recurrences
def _gate64(kind, z, param, rate=None):
    if kind == "sigmoid_root":
        return plain.sigmoid(z) ** param                   # param = 1 / tau
    if kind == "exp_sigmoid":
        return torch.exp(-param * plain.sigmoid(z))
    return torch.exp(-torch.exp(rate)[None, :, None] * plain.softplus(z))


FORMS = [("diagonal", "sigmoid_root"), ("delta_old_state", "exp_sigmoid"), ("delta_gated_state", "exp_softplus")]


@pytest.mark.parametrize("form,gate", FORMS)
@pytest.mark.parametrize("H,Hk,dk,dv", [(2, 2, 8, 8), (4, 2, 40, 24), (2, 1, 72, 40), (1, 1, 136, 33)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_recurrence_over_portions_batches_and_reused_slots(form, gate, H, Hk, dk, dv, dtype):
    from reinfer_b200 import ops
    if form != "delta_gated_state":
        Hk = H                                              # only that form groups its key heads
    g = _gen(100 + dk)
    lengths = {"a": 45, "b": 7, "c": 23}
    cuts = {"a": [20, 2, 1, 1, 17, 4], "b": [1, 1, 2, 3], "c": [2, 19, 2]}
    slot = {"a": 1, "b": 3, "c": 1}
    unit = form == "delta_gated_state"
    param = {"sigmoid_root": 1.0 / 4.0, "exp_sigmoid": math.exp(-0.5), "exp_softplus": 0.0}[gate]
    q_scale = dk ** -0.5 if form != "delta_old_state" else 1.0
    zb = torch.randn(H * dk, generator=g)
    ab = torch.randn(H * dk, generator=g)
    rate = torch.randn(H, generator=g) * 0.5 - 1.0
    data = {}
    for r, n in lengths.items():
        data[r] = dict(q=torch.randn(n, Hk * dk, generator=g).to(dtype), k=torch.randn(n, Hk * dk, generator=g).to(dtype),
                       v=torch.randn(n, H * dv, generator=g).to(dtype), z=torch.randn(n, H * dk, generator=g) * 2 + 1,
                       a=torch.randn(n, H * dk, generator=g).to(dtype), b=torch.randn(n, H, generator=g).to(dtype))
    state = torch.full((5, H, dk, dv), float("nan"), device=DEV)
    got = {r: [] for r in lengths}
    done = {r: 0 for r in lengths}
    for group in (["a", "b"], ["c"]):
        for r in group:
            state[slot[r]].zero_()
        k = 0
        while any(done[r] < lengths[r] for r in group):
            live = [r for r in group if done[r] < lengths[r]]
            lens = [min(cuts[r][k] if k < len(cuts[r]) else lengths[r], lengths[r] - done[r]) for r in live]
            cat = lambda key: torch.cat([data[r][key][done[r]:done[r] + n] for r, n in zip(live, lens)]).to(DEV)
            cu, sl = _tables(lens, [slot[r] for r in live])
            out = torch.empty(sum(lens), H, dv, device=DEV)
            ops.recurrence(form, gate, cat("q"), cat("k"), cat("v"), cat("z"), zb.to(DEV), state, out, cu, sl, len(live),
                           H, Hk, dk, dv, gate_param=param, q_scale=q_scale, unit_qk=unit,
                           a_pre=cat("a") if form == "delta_old_state" else None, a_bias=ab.to(DEV) if form == "delta_old_state" else None,
                           b_pre=cat("b") if form == "delta_gated_state" else None, rate=rate.to(DEV) if gate == "exp_softplus" else None)
            at = 0
            for r, n in zip(live, lens):
                got[r].append(out[at:at + n].cpu())
                at += n
                done[r] += n
            k += 1
    for r, n in lengths.items():
        d = {k_: v_.double() for k_, v_ in data[r].items()}
        q, k = d["q"].view(n, Hk, dk), d["k"].view(n, Hk, dk)
        if unit:
            q, k = plain.l2_unit(q), plain.l2_unit(k)
        q = q * q_scale
        v = d["v"].view(n, H, dv)
        gt = _gate64(gate, (d["z"] + zb.double()).view(n, H, dk), param, rate.double())
        heads = []
        for h in range(H):
            kh = h // (H // Hk)
            if form == "diagonal":
                heads.append(plain.scan_gla(q[:, kh], k[:, kh], v[:, h], gt[:, h]))
            elif form == "delta_old_state":
                a = plain.sigmoid(d["a"] + ab.double()).view(n, H, dk)
                heads.append(plain.scan_general_delta(q[:, kh], k[:, kh], v[:, h], gt[:, h], a[:, h]))
            else:
                heads.append(plain.scan_gated_delta(q[:, kh], k[:, kh], v[:, h], gt[:, h], plain.sigmoid(d["b"])[:, h]))
        ref = torch.stack(heads, 1)
        err = (torch.cat(got[r]).double() - ref).abs().max() / ref.abs().max()
        assert err < 2e-5, (r, err.item())                  # the inputs are the same rounded values on both sides


@pytest.mark.parametrize("form,gate", FORMS)
def test_a_memory_hundreds_of_tokens_old_is_read_back(form, gate):
    """One key channel hardly decays; token 3 writes a value there that no later token touches (their keys are zero in
    that channel, so neither a write nor a removal reaches it); 600 tokens later a query on that channel reads it
    back, among noise from everything since.  Portions and single tokens; every form of the recurrence."""
    from reinfer_b200 import ops
    g = _gen(7)
    n, dk, dv = 640, 16, 32
    q = torch.randn(n, dk, generator=g) * 0.1
    k = torch.randn(n, dk, generator=g)
    v = torch.randn(n, dv, generator=g)
    z = torch.randn(n, dk, generator=g)
    a = torch.randn(n, dk, generator=g)
    b = torch.randn(n, 1, generator=g) + 2.0
    k[:, 5] = 0.0
    k[3] = 0.0
    k[3, 5] = 6.0
    q[603] = 0.0
    q[603, 5] = 50.0
    # the gate of channel 5 within 1e-7 of one: sigmoid(14)^(1/16), exp(-c sigmoid(-30)), exp(-e^rate softplus(-30))
    z[:, 5] = 14.0 if gate == "sigmoid_root" else -30.0
    param = {"sigmoid_root": 1.0 / 16.0, "exp_sigmoid": math.exp(-0.5), "exp_softplus": 0.0}[gate]
    rate = torch.tensor([-0.5])
    unit = form == "delta_gated_state"
    state = torch.zeros(1, 1, dk, dv, device=DEV)
    outs = []
    at = 0
    for m in [100, 1, 1, 250, 2, 286]:                          # portions and single tokens
        cu, sl = _tables([m], [0])
        out = torch.empty(m, 1, dv, device=DEV)
        sel = slice(at, at + m)
        ops.recurrence(form, gate, q[sel].to(DEV), k[sel].to(DEV), v[sel].to(DEV), z[sel].to(DEV), None,
                       state, out, cu, sl, 1, 1, 1, dk, dv, gate_param=param, q_scale=1.0, unit_qk=unit,
                       a_pre=a[sel].to(DEV) if form == "delta_old_state" else None,
                       b_pre=b[sel].to(DEV) if unit else None, rate=rate.to(DEV) if gate == "exp_softplus" else None,
                       max_q_len=m)
        outs.append(out.cpu())
        at += m
    got = torch.cat(outs)[:, 0].double()
    gt = _gate64(gate, z.double().view(n, 1, dk), param, rate.double())[:, 0]
    qd, kd = q.double(), k.double()
    if unit:
        qd, kd = plain.l2_unit(qd), plain.l2_unit(kd)
    if form == "diagonal":
        ref = plain.scan_gla(qd, kd, v.double(), gt)
    elif form == "delta_old_state":
        ref = plain.scan_general_delta(qd, kd, v.double(), gt, plain.sigmoid(a.double()))
    else:
        ref = plain.scan_gated_delta(qd, kd, v.double(), gt, plain.sigmoid(b.double())[:, 0])
    # what token 3 wrote: k v^T, for the gated delta form the unit key times beta (v - 0)
    wrote = 6.0 * v[3].double() if not unit else plain.sigmoid(b[3].double()) * v[3].double()
    far = (50.0 if not unit else 1.0) * wrote
    assert (ref[603] - far).abs().max() < 0.05 * far.abs().max()       # the row is that memory
    assert (got - ref).abs().max() < 1e-4 * ref.abs().max()
    assert (got[603] - ref[603]).abs().max() < 1e-4 * far.abs().max()


# ------------------------------------------------------------------ chunk attention
def _paged(k, v, page, KH, dk, dv, pages_total, table):
    """Scatter k [n, KH, dk], v [n, KH, dv] into a cache [pages][K | V] by a block table."""
    cache = torch.full((pages_total, KH * page * (dk + dv)), float("nan"), dtype=k.dtype)
    for pos in range(k.shape[0]):
        pg, off = table[pos // page], pos % page
        for h in range(KH):
            a = (h * page + off) * dk
            cache[pg, a:a + dk] = k[pos, h]
            b = KH * page * dk + (h * page + off) * dv
            cache[pg, b:b + dv] = v[pos, h]
    return cache


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("QH,KH,dk,dv,chunk,page", [(4, 2, 16, 24, 24, 8), (2, 2, 64, 64, 64, 16), (3, 1, 40, 8, 5, 8),
                                                    (4, 2, 128, 128, 64, 16), (2, 1, 128, 128, 128, 8)])
def test_chunk_attention_sees_its_chunk_and_nothing_else(dtype, QH, KH, dk, dv, chunk, page):
    """Keys at the first position of every chunk and at the last position before it are made to stand out (a large key
    along a direction every query has a share of): the one inside must win, the one outside must not be seen, in a
    prompt portion and token by token."""
    from reinfer_b200 import ops
    g = _gen(40 + chunk)
    n = 3 * chunk + 2
    q = torch.randn(n, QH, dk, generator=g)
    k = torch.randn(n, KH, dk, generator=g)
    v = torch.randn(n, KH, dv, generator=g)
    q[:, :, 0] = 2.0
    for c in range(1, 4):
        if c * chunk < n:
            k[c * chunk, :, 0] = 9.0                 # just inside chunk c
        k[c * chunk - 1, :, 0] = 12.0                # the last key of chunk c-1: not for chunk c
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    r1, r2 = torch.rand(QH, generator=g) + 0.2, torch.rand(QH, generator=g) + 0.3
    scale = 0.4
    n_pages = -(-n // page)
    table = torch.randperm(n_pages + 3, generator=g)[:n_pages].tolist()
    cache = _paged(k, v, page, KH, dk, dv, n_pages + 3, table).to(DEV)
    bt = torch.tensor([table], dtype=torch.int32, device=DEV)
    group = SimpleNamespace(block_table=bt, page_size=page)
    ref = torch.stack([plain.chunk_attention(q[:, h].double(), k[:, h // (QH // KH)].double(), v[:, h // (QH // KH)].double(),
                                             scale, r1[h].double(), r2[h].double(), chunk) for h in range(QH)], 1) * 0.6
    tol = 1e-5 if dtype == torch.float32 else 2e-2

    def run(lo, hi):
        T = hi - lo
        ctx = SimpleNamespace(tok_entry=torch.zeros(T, dtype=torch.int32, device=DEV),
                              positions=torch.arange(lo, hi, dtype=torch.int32, device=DEV),
                              n_decode=1 if T == 1 else 0, n_entries=1, q_start=[0, T], start_pos=[lo], max_kv_len=hi, decode_kv_tiles=None,
                              cu_q=torch.tensor([0, T], dtype=torch.int32, device=DEV),
                              kv_len=torch.tensor([hi], dtype=torch.int32, device=DEV))
        out = torch.empty(T, QH, dv, dtype=dtype, device=DEV)
        ops.chunk_attention(ctx, q[lo:hi].contiguous().to(DEV), cache, group, out, QH, KH, dk, dv, chunk, scale,
                            (r1.to(DEV), r2.to(DEV)), 0.6)
        return out.double().cpu()

    whole = run(0, n)
    assert (whole - ref).abs().max() <= tol * ref.abs().max()
    one_by_one = torch.cat([run(i, i + 1) for i in range(n)])
    assert (one_by_one - ref).abs().max() <= tol * ref.abs().max()
    pieces = torch.cat([run(a, b) for a, b in ((0, 2), (2, chunk + 1), (chunk + 1, 2 * chunk - 1), (2 * chunk - 1, n))])
    assert (pieces - ref).abs().max() <= tol * ref.abs().max()
    # the standing-out key inside the chunk takes most of the weight of its chunk's first rows
    kv0 = v[chunk, 0].double() * 0.6
    assert (ref[chunk, 0] - kv0).abs().max() < 1e-9
