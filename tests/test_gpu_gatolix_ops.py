"""Every mechanism of the Gatolix layer alone, on the GPU, against the plain oracle (oracle/gatolix_ref.py): norms on
both sides of a sublayer, element-wise activations, the rotary table, what a token writes into the latent pool, windowed
attention over the pool (prompt portions and single rows, pages in any order, loud keys just inside and just outside the
window), routing and the bounded experts."""
import math

import pytest
import torch

import gatolix_ref as R

pytestmark = pytest.mark.gpu
F64 = torch.float64
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dt):
    return 2e-5 if dt == torch.float32 else 2e-2


def _close(got, want, dt, what=""):
    err = float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-6))
    assert err <= _tol(dt), f"{what}: relative error {err:.3e}"


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D", [50, 200, 1000, 4096, 8192])
def test_sandwich_norm(cuda, dt, D):
    from b200attn import ops
    g = torch.Generator().manual_seed(D)
    T, eps = 7, 1e-5
    x = torch.randn(T, D, generator=g) * 3 + 1
    y = (torch.randn(T, D, generator=g) * 2 - 0.5).to(dt)
    pw, pb, qw, qb = (torch.randn(D, generator=g) for _ in range(4))
    xd = x.to(cuda)
    h = ops.sandwich_norm(xd, y.to(cuda), pw.to(cuda), pb.to(cuda), qw.to(cuda), qb.to(cuda), eps=eps, h_dtype=dt)
    x1 = x.double() + R.layer_norm(y.double(), pw.double(), pb.double(), eps)
    assert float((xd.cpu().double() - x1).abs().max()) <= 1e-5 * float(x1.abs().max())          # the residual stays fp32
    _close(h, R.layer_norm(x1, qw.double(), qb.double(), eps), dt, "read-out")
    # read-out alone; write-back alone; plain add; RMS kind without bias
    xd = x.to(cuda)
    _close(ops.sandwich_norm(xd, pre_w=qw.to(cuda), pre_b=qb.to(cuda), eps=eps, h_dtype=dt),
           R.layer_norm(x.double(), qw.double(), qb.double(), eps), dt, "read-out alone")
    assert torch.equal(xd.cpu(), x)
    assert ops.sandwich_norm(xd, y.to(cuda), pw.to(cuda), None, eps=eps) is None
    _close(xd, x.double() + R.layer_norm(y.double(), pw.double(), torch.zeros(D, dtype=F64), eps), torch.float32, "write-back")
    xd = x.to(cuda)
    h = ops.sandwich_norm(xd, y.to(cuda), None, None, qw.to(cuda), None, eps=eps, norm_kind=ops.NORM_RMS, h_dtype=dt)
    _close(h, R.rms_norm(x.double() + y.double(), qw.double(), eps), dt, "add + rms")


@pytest.mark.parametrize("dt", DTYPES)
def test_elementwise(cuda, dt):
    from b200attn import ops
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(5, 70, generator=g) * 4).to(dt)
    _close(ops.relu_sq(a.to(cuda)), torch.relu(a.double()) ** 2, dt, "relu^2")
    gu = (torch.randn(6, 2 * 37, generator=g) * 4).to(dt)                    # values on both sides of the limits
    gg, uu = gu.double()[:, :37], gu.double()[:, 37:]
    for limit in (0.5, 3.0):
        gc, uc = gg.clamp(max=limit), uu.clamp(-limit, limit)
        _close(ops.glu_and_mul(gu.to(cuda), ops.GLU_CLAMPED, 1.702, limit), gc * torch.sigmoid(1.702 * gc) * (uc + 1), dt, "bounded glu")
    _close(ops.glu_and_mul(gu.to(cuda)), gg * torch.sigmoid(gg) * uu, dt, "silu glu")
    z = (torch.randn(3, 99, generator=g) * 40).to(dt)
    zd = z.to(cuda)
    ops.softcap_(zd, 25.0)
    _close(zd, 25.0 * torch.tanh(z.double() / 25.0), dt, "soft cap")


@pytest.mark.parametrize("scaling", [None, {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0},
                                     {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0}])
def test_rotary_table(cuda, scaling):
    from b200attn import ops
    dims, base, P = 12, 300.0, 200
    tab = ops.rotary_table(P, dims, base, scaling, cuda).cpu().double()
    f, mag = R.rotary_frequencies(dims, base, scaling)
    for pos in (0, 1, 7, 63, 64, 199):
        want = [math.cos(pos * fi) * mag for fi in f] + [math.sin(pos * fi) * mag for fi in f]
        assert tab[pos].tolist() == pytest.approx(want, abs=2e-6)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,dn,dr,dims,Rk", [(3, 20, 12, 8, 36), (4, 16, 16, 16, 64), (1, 8, 4, 4, 10)])
def test_latent_prep(cuda, dt, H, dn, dr, dims, Rk):
    from b200attn import ops
    g = torch.Generator().manual_seed(H)
    T, bs, nb, eps = 9, 4, 6, 1e-5
    scaling = {"factor": 3.0, "original": 16, "fast": 3.0, "slow": 1.0}
    tab = ops.rotary_table(64, dims, 50.0, scaling, cuda)
    f, mag = R.rotary_frequencies(dims, 50.0, scaling)
    goff = H * (dn + dr)
    proj = torch.randn(T, goff + H + Rk + dr, generator=g).to(dt)
    pos = torch.tensor([5, 0, 1, 2, 3, 40, 41, 63, 7], dtype=torch.int32)
    slots = torch.tensor([3, 0, 1, 2, 7, -1, 23, 22, 12], dtype=torch.int64)
    nw = torch.randn(Rk, generator=g)
    cache = torch.full((nb, bs, Rk + dr), 9.0, dtype=dt, device=cuda)
    qa = ops.latent_prep(proj.to(cuda), H, dn, dr, dims, Rk, 0, goff + H, nw.to(cuda), eps, pos.to(cuda), tab, slots.to(cuda), cache)
    flat = cache.view(nb * bs, Rk + dr).cpu().double()
    pd = proj.double()
    for t in range(T):
        q = pd[t, :goff].view(H, dn + dr)
        _close(qa[t, :, Rk:], R.rotate(q[:, dn:], int(pos[t]), f, mag, dims), dt, "query rotation")
        if slots[t] < 0:
            continue
        d = pd[t, goff + H:]
        _close(flat[slots[t], :Rk], R.rms_norm(d[:Rk], nw.double(), eps), dt, "latent")
        _close(flat[slots[t], Rk:], R.rotate(d[Rk:], int(pos[t]), f, mag, dims), dt, "shared key part")
    untouched = [s for s in range(nb * bs) if s not in slots.tolist()]
    assert bool((flat[untouched] == 9.0).all())
    # a layer that reads another layer's pool writes nothing
    before = cache.clone()
    ops.latent_prep(proj.to(cuda)[:, :goff + H].contiguous(), H, dn, dr, dims, Rk, 0, -1, None, eps, pos.to(cuda), tab, None, None)
    assert torch.equal(cache, before)


def _paged(rows, bs, cuda, dt, seed):
    """rows [Tk, Dc] -> pool with the pages in a shuffled order (and pages of other owners in between) + block table."""
    Tk, Dc = rows.shape
    nb = (Tk + bs - 1) // bs
    perm = torch.randperm(2 * nb + 3, generator=torch.Generator().manual_seed(seed))[:nb]
    pool = torch.full((2 * nb + 3, bs, Dc), 50.0, dtype=dt)                  # foreign pages hold loud numbers
    for b in range(nb):
        part = rows[b * bs:(b + 1) * bs]
        pool[perm[b], :part.shape[0]] = part.to(dt)
    return pool.to(cuda), perm.to(torch.int32)


def _attend(cuda, dt, H, Rk, dr, window, seqs, bs=16, loud=(), seed=0):
    """seqs: [(context tokens, rows in this step)].  Returns (got, want) over all rows of the step."""
    from b200attn import ops
    g = torch.Generator().manual_seed(seed + H)
    Dc, scale = Rk + dr, 0.3
    pools, tables, cu, ctx, qs, gates, wants = [], [], [0], [], [], [], []
    for si, (nctx, nq) in enumerate(seqs):
        Tk = nctx + nq
        rows = torch.randn(Tk, Dc, generator=g).to(dt)
        q = torch.randn(nq, H, Dc, generator=g).to(dt)
        gate = (torch.randn(nq, H, generator=g) * 2).to(dt)
        for (s, row, key, amp) in loud:                                      # make one (query row, key) score stand out
            if s == si:
                unit = torch.randn(Dc, generator=g)
                unit = unit / unit.norm()
                rows[key] = (unit * amp).to(dt)
                q[row] = (unit * amp).to(dt)
        k = rows.double()[:, None, :].expand(Tk, H, Dc)
        want = R.windowed_attention(q.double(), k, k[:, :, :Rk], scale, window, first_pos=nctx)
        wants.append(want * torch.sigmoid(gate.double())[:, :, None])
        pool, bt = _paged(rows, bs, cuda, dt, seed + si)
        pools.append(pool), tables.append(bt), qs.append(q), gates.append(gate)
        cu.append(cu[-1] + nq), ctx.append(nctx)
    # one pool for the step: concatenate the per-sequence pools and shift their page numbers
    off, max_nb = 0, max(t.shape[0] for t in tables)
    bts = torch.zeros(len(seqs), max_nb, dtype=torch.int32)
    for i, (p, t) in enumerate(zip(pools, tables)):
        bts[i, :t.shape[0]] = t + off
        off += p.shape[0]
    batch = ops.SeqBatch(torch.tensor(cu, dtype=torch.int32, device=cuda), torch.tensor(ctx, dtype=torch.int32, device=cuda),
                         bts.to(cuda), None, len(seqs), cu[-1])
    gate_wide = torch.cat([torch.zeros(cu[-1], 3, dtype=dt), torch.cat(gates)], 1).to(cuda)       # a column slice of a wider row
    got = ops.latent_attention(torch.cat(qs).to(cuda).contiguous(), torch.cat(pools), batch, Rk, scale, window,
                               gate=gate_wide[:, 3:])
    return got, torch.cat(wants)


SHAPES = [(3, 36, 12), (16, 64, 16), (8, 128, 48), (5, 64, 16), (2, 256, 64), (20, 64, 32), (72, 64, 16), (4, 512, 64)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,Rk,dr", SHAPES)
@pytest.mark.parametrize("window", [0, 1, 16, 37])
def test_latent_attention_prompts_and_single_rows(cuda, dt, H, Rk, dr, window):
    """Whole prompts, portions with context (starting inside a page and inside a window), single rows, in one batch."""
    seqs = [(0, 45), (23, 31), (70, 1), (0, 1), (41, 2), (100, 1), (15, 70)]
    got, want = _attend(cuda, dt, H, Rk, dr, window, seqs, seed=window)
    _close(got, want, dt, f"H={H} R={Rk} dr={dr} window={window}")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,Rk,dr", [(8, 128, 48), (2, 256, 64), (4, 512, 64), (20, 128, 16), (16, 64, 16), (3, 36, 12)])
@pytest.mark.parametrize("window", [0, 1, 16, 37, 300])
def test_latent_attention_decode_batches(cuda, dt, H, Rk, dr, window):
    """Batches in which every sequence brings one row (what a decode step is): few rows, so the keys of a row are shared
    out over warps and CTAs.  Contexts from nothing to several hundred tokens, one loud key at each window's first and
    last-but-one position."""
    seqs = [(0, 1), (1, 1), (15, 1), (16, 1), (63, 1), (64, 1), (65, 1), (200, 1), (511, 1), (640, 1)]
    loud = []
    for i, (nctx, _) in enumerate(seqs):
        if window and nctx - window + 1 >= 0 and i % 2 == 0:
            loud.append((i, 0, nctx - window + 1, 9.0))                       # the last key the window keeps
        elif window and nctx - window >= 0:
            loud.append((i, 0, nctx - window, 9.0))                           # the first key it has dropped
    got, want = _attend(cuda, dt, H, Rk, dr, window, seqs, loud=loud, seed=window + H)
    _close(got, want, dt, f"decode batch H={H} R={Rk} dr={dr} window={window}")
    got, want = _attend(cuda, dt, H, Rk, dr, window, seqs[6:8], seed=5)       # two rows: more shares per row
    _close(got, want, dt, "small decode batch")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,Rk,dr", [(3, 36, 12), (16, 64, 16), (8, 128, 48)])
@pytest.mark.parametrize("edge", ["inside", "outside"])
def test_latent_attention_loud_key_at_the_window_edge(cuda, dt, H, Rk, dr, edge):
    """A key whose score dwarfs all others sits on the last position the window keeps, or one before it: in a prompt
    portion, in a single row, and with the edge on a page border (page size 16: keys 31 | 32, 47 | 48)."""
    window = 20
    cases = []
    # (context, rows, query row) -> the query's position p; the edge key is p - window + 1 (inside) or p - window (outside)
    for nctx, nq, row in ((0, 90, 60), (40, 30, 11), (66, 1, 0), (0, 90, 51), (47, 20, 4), (67, 1, 0), (19, 1, 0), (20, 1, 0)):
        p = nctx + row
        key = p - window + (1 if edge == "inside" else 0)
        if key >= 0:
            cases.append(((nctx, nq), (row, key)))
    seqs = [c[0] for c in cases]
    loud = [(i, c[1][0], c[1][1], 12.0) for i, c in enumerate(cases)]
    got, want = _attend(cuda, dt, H, Rk, dr, window, seqs, loud=loud, seed=7)
    _close(got, want, dt, f"loud key {edge} the window")
    # the loud key decides the row when it is in sight: the two runs must differ there
    if edge == "inside":
        got2, want2 = _attend(cuda, dt, H, Rk, dr, window - 1, seqs, loud=loud, seed=7)
        _close(got2, want2, dt, "window one shorter")
        assert float((want - want2).abs().max()) > 0.1


@pytest.mark.parametrize("dt", DTYPES)
def test_latent_attention_far_key_and_padding(cuda, dt):
    """Without a window a loud key 1000 positions back decides a decoded row; with one it is out of sight.  Rows of a
    padding sequence (negative context) come back as zeros."""
    from b200attn import ops
    for window in (0, 300):
        got, want = _attend(cuda, dt, 4, 64, 16, window, [(1100, 1), (1090, 12)], loud=[(0, 0, 97, 10.0), (1, 5, 3, 10.0)], seed=3)
        _close(got, want, dt, f"far key, window {window}")
    qa = torch.randn(3, 2, 24, device=cuda).to(dt)
    pool = torch.randn(4, 16, 24, device=cuda).to(dt)
    batch = ops.SeqBatch(torch.tensor([0, 1, 2, 3], dtype=torch.int32, device=cuda),
                         torch.tensor([5, -1, 0], dtype=torch.int32, device=cuda), torch.zeros(3, 2, dtype=torch.int32, device=cuda),
                         None, 3, 3)
    out = ops.latent_attention(qa, pool, batch, 16, 0.5, 8)
    assert bool((out[1] == 0).all()) and bool((out[0] != 0).any())
    _close(out[2], pool[0, 0, :16].double().cpu().expand(2, 16), dt, "a first token sees itself")


@pytest.mark.parametrize("H,dn,dr,dv", [(3, 16, 16, 32), (2, 24, 8, 16), (5, 8, 24, 48), (4, 128, 64, 128), (1, 8, 8, 80)])
@pytest.mark.parametrize("window", [0, 1, 40, 64, 150])
def test_gather_and_window_attention(cuda, H, dn, dr, dv, window):
    """Prompt portions over keys and values held per head: pool rows gathered from shuffled pages (from each window's first
    position on, or from further back), keys = per-head part + shared part, a loud key on the window's edge."""
    from b200attn import ops
    g = torch.Generator().manual_seed(H * 7 + window)
    bf, Rk, bs, scale = torch.bfloat16, 24, 16, 0.25
    seqs = [(0, 130), (70, 65), (201, 3), (0, 1), (33, 64)]                  # (context, rows)
    pools, tables, wants, qs, gates, kns, vs = [], [], [], [], [], [], []
    cu_q, ctx, cu_k, k_lo = [0], [], [0], []
    for si, (nctx, nq) in enumerate(seqs):
        Tk = nctx + nq
        lat = torch.randn(Tk, Rk + dr, generator=g).to(bf)                   # pool rows: [latent | shared key part]
        kn = torch.randn(Tk, H, dn, generator=g).to(bf)
        v = torch.randn(Tk, H, dv, generator=g).to(bf)
        q = torch.randn(nq, H, dn + dr, generator=g).to(bf)
        gate = (torch.randn(nq, H, generator=g) * 2).to(bf)
        if window and nctx + nq // 2 - window + 1 >= 0:                      # loud key on the last position the window keeps
            row, key = nq // 2, nctx + nq // 2 - window + 1
            unit = torch.randn(dn + dr, generator=g)
            unit = unit / unit.norm() * 9.0
            q[row] = unit.to(bf)
            kn[key] = unit[:dn].to(bf)
            lat[key, Rk:] = unit[dn:].to(bf)
        k = torch.cat([kn.double(), lat[:, None, Rk:].double().expand(Tk, H, dr)], -1)
        want = R.windowed_attention(q.double(), k, v.double(), scale, window, first_pos=nctx)
        wants.append(want * torch.sigmoid(gate.double())[:, :, None])
        first = 0 if si % 2 else (max(0, nctx - window + 1) if window else 0)            # gather from the edge, or from 0
        pool, bt = _paged(lat, bs, cuda, bf, si)
        pools.append(pool), tables.append(bt), qs.append(q), gates.append(gate)
        kns.append(kn[first:]), vs.append(v[first:])
        cu_q.append(cu_q[-1] + nq), ctx.append(nctx), cu_k.append(cu_k[-1] + Tk - first), k_lo.append(first)
    off, max_nb = 0, max(t.shape[0] for t in tables)
    bts = torch.zeros(len(seqs), max_nb, dtype=torch.int32)
    for i, (p, t) in enumerate(zip(pools, tables)):
        bts[i, :t.shape[0]] = t + off
        off += p.shape[0]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=cuda)          # noqa: E731
    d_cu_k, d_k_lo = i32(cu_k), i32(k_lo)
    lat_g = ops.latent_gather(torch.cat(pools), bts.to(cuda), d_cu_k, d_k_lo, len(seqs), cu_k[-1])
    assert lat_g.shape == (cu_k[-1], Rk + dr)
    qall = torch.cat(qs).to(cuda)
    gate_wide = torch.cat([torch.zeros(cu_q[-1], 5, dtype=bf), torch.cat(gates)], 1).to(cuda)
    got = ops.window_attention(qall[:, :, :dn], qall[:, :, dn:].contiguous(), torch.cat(kns).to(cuda).contiguous(), lat_g[:, Rk:],
                               torch.cat(vs).to(cuda).contiguous(), i32(cu_q), i32(ctx), d_cu_k, d_k_lo, len(seqs), scale, window,
                               gate=gate_wide[:, 5:])
    _close(got, torch.cat(wants), bf, f"H={H} {dn}+{dr}/{dv} window={window}")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("T,D,E,top", [(9, 48, 5, 2), (1, 64, 8, 8), (1500, 32, 3, 1), (40, 200, 40, 6)])
def test_route_softmax_over_all_with_correction(cuda, dt, T, D, E, top):
    from b200attn import ops
    g = torch.Generator().manual_seed(E)
    h = torch.randn(T, D, generator=g).to(dt)
    wr = (torch.randn(E, D, generator=g) * 2 * D ** -0.5).to(dt)
    corr = torch.randn(E, generator=g) * 0.3                                 # large enough to change the choice
    ids, wts = ops.moe_route(h.to(cuda), wr.to(cuda), corr.to(cuda), top, scoring=ops.ROUTE_SOFTMAX_ALL)
    w = {"l0.mlp.router": wr, "l0.mlp.correction": corr}
    want_ids, want_w = R.route(h.double(), w, "l0", top)
    s = torch.softmax(h.double() @ wr.double().T, -1)
    plain = torch.topk(s, top, -1).indices
    assert T < 9 or not torch.equal(plain.sort(-1).values, want_ids.sort(-1).values)           # the correction matters here
    margin = torch.topk(s + corr.double(), min(top + 1, E), -1).values
    sure = torch.ones(T, dtype=torch.bool) if top == E else (margin[:, top - 1] - margin[:, top]) > 1e-5   # inputs are exact in both types
    assert int(sure.sum()) >= T * 0.8
    assert torch.equal(ids.cpu().long()[sure].sort(-1).values, want_ids[sure].sort(-1).values)
    order_g, order_w = ids.cpu().long().argsort(-1), want_ids.argsort(-1)
    gw, ww = torch.gather(wts.cpu().double(), -1, order_g), torch.gather(want_w, -1, order_w)
    assert float((gw[sure] - ww[sure]).abs().max()) <= (1e-5 if dt == torch.float32 else 2e-2)
    assert top == E or float(wts.sum(-1).max()) < 1.0                        # not renormalised


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("T,D,F,E,top,limit", [(11, 48, 40, 5, 2, 0.5), (1, 64, 24, 3, 3, 7.0), (2100, 32, 16, 4, 1, 1.5)])
def test_bounded_experts(cuda, dt, T, D, F, E, top, limit):
    from b200attn import ops
    g = torch.Generator().manual_seed(T)
    h = (torch.randn(T, D, generator=g) * 2).to(dt)
    w = {}
    for e in range(E):
        w[f"l0.mlp.e{e}.gate"] = (torch.randn(F, D, generator=g) * D ** -0.5).to(dt)
        w[f"l0.mlp.e{e}.up"] = (torch.randn(F, D, generator=g) * D ** -0.5).to(dt)
        w[f"l0.mlp.e{e}.down"] = (torch.randn(D, F, generator=g) * F ** -0.5).to(dt)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g)
    gu = torch.stack([torch.cat([w[f"l0.mlp.e{e}.gate"], w[f"l0.mlp.e{e}.up"]]) for e in range(E)]).to(cuda)
    dn = torch.stack([w[f"l0.mlp.e{e}.down"] for e in range(E)]).to(cuda)
    y = ops.moe_experts(h.to(cuda), ids.to(cuda), wts.to(cuda), gu[:, :F], gu[:, F:], dn, w_gate_up=gu, glu=ops.GLU_CLAMPED,
                        glu_alpha=1.702, glu_limit=limit)
    n = min(T, 40)
    want = torch.zeros(n, D, dtype=F64)
    for t in range(n):
        for j in range(top):
            want[t] += wts[t, j].double() * R.expert(h[t:t + 1].double(), w, "l0", int(ids[t, j]), limit)[0]
    _close(y[:n], want, dt, "experts")
    # a token's result does not depend on the batch around it
    y1 = ops.moe_experts(h[:1].to(cuda), ids[:1].to(cuda), wts[:1].to(cuda), gu[:, :F], gu[:, F:], dn, w_gate_up=gu,
                         glu=ops.GLU_CLAMPED, glu_alpha=1.702, glu_limit=limit)
    _close(y1, y[:1].double().cpu(), dt, "alone against in the batch")
