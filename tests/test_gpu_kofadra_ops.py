"""Every new mechanism alone, against the plain oracle (oracle/kofadra_ref.py): residual streams + norm, the gated
delta-rule mixer's stages with state carried across calls, block-masked sink attention over scattered pages, the router
and the grouped expert products.  fp32 compares tightly; bf16 against the same oracle fed the rounded inputs."""
import math

import pytest
import torch

import kofadra_ref as R

pytestmark = pytest.mark.gpu

F64 = torch.float64


def _ops():
    from b200attn import ops
    return ops


def _close(got, want, tol, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / (want.abs().max() + 1e-30))
    assert err <= tol, f"{what}: relative error {err:.3e} above {tol:.1e}"


def _batch(cuda, lens, ctx, slots, tables=None):
    ops = _ops()
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=cuda)      # noqa: E731
    return ops.SeqBatch(i32(cu), i32(ctx), None if tables is None else i32(tables), i32(slots), len(lens), cu[-1])


# ------------------------------------------------------------------------------------------------ streams + norm
@pytest.mark.parametrize("S,D", [(1, 48), (2, 200), (3, 64), (5, 33), (9, 40)])
@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_hc_step(cuda, S, D, kind, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(S * 100 + D)
    T = 6
    x = torch.randn(T, S, D, generator=g) * 3 + 0.7
    y = torch.randn(T, D, generator=g).to(dtype)
    mix, out_w, in_w = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    w = 1 + 0.2 * torch.randn(D, generator=g)
    xd = x.to(cuda)
    h = ops.hc_step(xd, y.to(cuda), mix.to(cuda), out_w.to(cuda), in_w.to(cuda), w.to(cuda), 1e-5,
                    ops.NORM_LAYER if kind == "layer" else ops.NORM_RMS, h_dtype=dtype)
    x2 = torch.einsum("sj,tsd->tjd", mix.to(F64), x.to(F64)) + out_w.to(F64).view(1, S, 1) * y.to(F64).unsqueeze(1)
    u = (in_w.to(F64).view(1, S, 1) * x2).sum(1)
    want = R.layer_norm(u, w.to(F64), 1e-5) if kind == "layer" else R.rms_div(u, 1e-5) * w.to(F64)
    _close(xd, x2, 1e-6, "streams")
    _close(h, want, 1e-5 if dtype == torch.float32 else 1e-2, "read-out")
    # read-out alone (no write-back) leaves the streams untouched; write-back alone returns nothing
    before = xd.clone()
    h2 = ops.hc_step(xd, in_w=in_w.to(cuda), norm_w=w.to(cuda), eps=1e-5, h_dtype=dtype,
                     norm_kind=ops.NORM_LAYER if kind == "layer" else ops.NORM_RMS)
    assert torch.equal(before, xd) and torch.equal(h2, h)
    assert ops.hc_step(xd, y.to(cuda), mix.to(cuda), out_w.to(cuda)) is None and not torch.equal(before, xd)


def test_plain_residual_is_the_one_stream_default(cuda):
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    x, y, w = torch.randn(4, 1, 40, generator=g), torch.randn(4, 40, generator=g), torch.rand(40, generator=g) + 0.5
    xd = x.to(cuda)
    h = ops.hc_step(xd, y.to(cuda), norm_w=w.to(cuda), eps=1e-6, h_dtype=torch.float32)
    _close(xd[:, 0], x[:, 0] + y, 1e-6)
    _close(h, R.layer_norm((x[:, 0] + y).to(F64), w.to(F64), 1e-6), 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_streams(cuda, dtype):
    ops = _ops()
    emb = torch.randn(19, 24).to(dtype)
    tok = torch.tensor([3, 18, 0, 3], dtype=torch.int64)
    x = ops.embed_streams(emb.to(cuda), tok.to(cuda), 3, 2.5)
    assert x.shape == (4, 3, 24) and x.dtype == torch.float32
    for s in range(3):
        _close(x[:, s], emb.float()[tok] * 2.5, 1e-7)


# ------------------------------------------------------------------------------------------------ delta rule
def _delta_oracle(proj, conv_w, A_log, dt_bias, norm_w, H, G, dk, dv, eps):
    """One sequence, all stages in fp64: returns qkv (normalised), beta, decay, o, gated output."""
    T = proj.shape[0]
    C = 2 * G * dk + H * dv
    z = R.silu(R.causal_conv(proj[:, :C], conv_w))
    q = z[:, :G * dk].view(T, G, dk)
    k = z[:, G * dk:2 * G * dk].view(T, G, dk)
    v = z[:, 2 * G * dk:].view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    gate = proj[:, C:C + H * dv].view(T, H, dv)
    beta = torch.sigmoid(proj[:, C + H * dv:C + H * dv + H])
    decay = torch.exp(-torch.exp(A_log) * R.softplus(proj[:, C + H * dv + H:C + H * dv + 2 * H] + dt_bias))
    o = torch.zeros(T, H, dv, dtype=F64)
    for h in range(H):
        o[:, h], _ = R.delta_rule(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], beta[:, h], decay[:, h])
    out = R.rms_div(o, eps) * norm_w * R.silu(gate)
    return torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1), beta, decay, o, out.reshape(T, H * dv)


@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 16, 24, 3), (2, 2, 40, 72, 1), (3, 1, 8, 8, 6), (2, 1, 128, 64, 4),
                                            (1, 1, 200, 40, 2), (1, 1, 30, 6, 3), (1, 1, 300, 8, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_delta_mixer_stages_with_state_across_calls(cuda, H, G, dk, dv, taps, dtype):
    """Two sequences of unequal length fed in portions (down to one and two tokens), their slots swapped relative to
    their order and dirty from an earlier occupant: every stage equals the oracle run over the whole sequences."""
    ops = _ops()
    g = torch.Generator().manual_seed(dk * 7 + taps)
    C = 2 * G * dk + H * dv
    P = C + H * dv + 2 * H
    lens = [23, 12]
    proj = [(torch.randn(n, P, generator=g) * 1.5).to(dtype) for n in lens]
    conv_w = torch.randn(C, taps, generator=g) * taps ** -0.5
    A_log, dt_bias, norm_w = torch.randn(H, generator=g) - 1, torch.randn(H, generator=g), 1 + 0.1 * torch.randn(dv, generator=g)
    want = [_delta_oracle(p.to(F64), conv_w.to(F64), A_log.to(F64), dt_bias.to(F64), norm_w.to(F64), H, G, dk, dv, 1e-5)
            for p in proj]
    state = torch.full((3, H, dk, dv), 7.0, device=cuda)                       # dirty slots
    conv_state = torch.full((3, taps - 1, C), -5.0, dtype=dtype, device=cuda) if taps > 1 else None
    portions = [[9, 1, 2, 11], [5, 2, 1, 4]]
    slots = [2, 0]
    at = [0, 0]
    got = [[[] for _ in range(5)] for _ in lens]
    for step in range(4):
        ns = [portions[i][step] for i in range(2)]
        rows = torch.cat([proj[i][at[i]:at[i] + ns[i]] for i in range(2)]).to(cuda)
        b = _batch(cuda, ns, at, slots)
        qkv, beta, decay = ops.delta_prep(rows, C + H * dv, C + H * dv + H, H, G, dk, dv, taps, conv_w.to(cuda),
                                          A_log.to(cuda), dt_bias.to(cuda), b, conv_state)
        o = ops.delta_scan(qkv, beta, decay, H, G, dk, dv, b, state)
        out = ops.delta_out(o, rows, C, norm_w.to(cuda), 1e-5)
        r0 = 0
        for i in range(2):
            for j, t in enumerate((qkv, beta, decay, o, out)):
                got[i][j].append(t[r0:r0 + ns[i]].float().cpu())
            r0 += ns[i]
            at[i] += ns[i]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for i in range(2):
        for j, name in enumerate(("qkv", "beta", "decay", "o", "gated output")):
            _close(torch.cat(got[i][j]).view(want[i][j].shape), want[i][j], tol, f"sequence {i} {name}")


def test_delta_state_keeps_a_far_token(cuda):
    """With decay ~ 1 and one early token written at full strength, a query 400 tokens later (fed one by one through
    the slot) still reads it: a state that is lost or re-zeroed anywhere on the way shows as a zero output."""
    ops = _ops()
    H = G = 1
    dk, dv, T = 16, 8, 420
    qkv = torch.zeros(T, 2 * dk + dv)
    qkv[:, dk] = 1.0                                   # every key is e0 ...
    qkv[5, dk], qkv[5, dk + 3] = 0.0, 1.0              # ... but token 5's, which is e3 and carries the value
    qkv[5, 2 * dk:] = torch.arange(1, dv + 1)
    qkv[T - 1, 3] = 1.0                                # the last query asks for e3
    beta, decay = torch.ones(T, 1), torch.full((T, 1), 0.9999)
    state = torch.zeros(1, 1, dk, dv, device=cuda)
    outs = []
    at = 0
    for n in [100] + [1] * 319 + [1]:
        b = _batch(cuda, [n], [at], [0])
        outs.append(ops.delta_scan(qkv[at:at + n].to(cuda), beta[at:at + n].to(cuda), decay[at:at + n].to(cuda), H, G, dk, dv,
                                   b, state))
        at += n
    assert at == T
    want, _ = R.delta_rule(qkv[:, :dk].to(F64), qkv[:, dk:2 * dk].to(F64), qkv[:, 2 * dk:].to(F64), beta[:, 0].to(F64),
                           decay[:, 0].to(F64))
    assert float(want[T - 1].abs().min()) > 0.5
    _close(torch.cat(outs)[:, 0], want, 1e-5)


# ------------------------------------------------------------------------------------------------ attention
def _attn_setup(cuda, dtype, H, G, dk, dv, bs, lens, seed):
    g = torch.Generator().manual_seed(seed)
    qkv = [(torch.randn(n, H * dk + G * dk + G * dv, generator=g)).to(dtype) for n in lens]
    nb_each = [(n + bs - 1) // bs for n in lens]
    perm = torch.randperm(sum(nb_each) + 3, generator=g).tolist()             # scattered pages
    tables, k = [], 0
    for nb in nb_each:
        tables.append(perm[k:k + nb] + [0] * (max(nb_each) - nb))
        k += nb
    kc = torch.full((len(perm), G, bs, dk), float("nan"), dtype=dtype, device=cuda)
    vc = torch.full((len(perm), G, bs, dv), float("nan"), dtype=dtype, device=cuda)
    return qkv, tables, kc, vc


def _attn_oracle(qkv, q_w, k_w, H, G, dk, dv, eps, scale, chunk):
    T = qkv.shape[0]
    q = R.rms_div(qkv[:, :H * dk].view(T, H, dk), eps) * q_w
    k = R.rms_div(qkv[:, H * dk:(H + G) * dk].view(T, G, dk), eps) * k_w
    v = qkv[:, (H + G) * dk:].view(T, G, dv)
    return torch.stack([R.sink_attention(q[:, h], k[:, h // (H // G)], v[:, h // (H // G)], scale, chunk or None)
                        for h in range(H)], 1)


@pytest.mark.parametrize("H,G,dk,dv,bs,chunk", [(4, 1, 24, 16, 16, 8), (2, 2, 16, 40, 16, 20), (3, 3, 96, 8, 8, 64),
                                                (2, 1, 8, 24, 16, 0), (5, 5, 40, 8, 32, 5),
                                                # head sizes the tensor-core prompt kernel takes (bf16, portions of >= 16 rows)
                                                (4, 2, 64, 32, 16, 24), (2, 1, 128, 128, 16, 100), (2, 2, 32, 96, 8, 0),
                                                (4, 4, 96, 96, 16, 64), (2, 1, 64, 64, 16, 7),
                                                # more than eight query heads per kv head; sizes only the warp kernel takes
                                                (12, 1, 16, 8, 16, 10), (2, 1, 12, 20, 16, 6), (1, 1, 8, 320, 16, 9)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_chunk_attention_in_portions_over_scattered_pages(cuda, H, G, dk, dv, bs, chunk, dtype):
    """Two sequences: prompt portions that end inside a page and inside a mask block, then single rows; queries and
    keys at chosen places are scaled so that ONE score dominates -- a key just inside the block's edge, one just
    outside it, and one far back."""
    ops = _ops()
    lens = [75, 37]
    qkv, tables, kc, vc = _attn_setup(cuda, dtype, H, G, dk, dv, bs, lens, seed=dk + chunk)
    q_w, k_w = 1 + 0.1 * torch.randn(dk), 1 + 0.1 * torch.randn(dk)
    c = chunk or 10 ** 9
    for i in (len(qkv[0]) - 1, 41, 30):                 # loud pairs in sequence 0: (query i, key j)
        lo = (i // c) * c
        d = torch.randn(dk)                             # after the per-head norm what counts is the shared direction
        qkv[0][i, :H * dk] = d.repeat(H).to(dtype)
        for j in {lo, max(lo - 1, 0), 2}:
            qkv[0][j, H * dk:(H + G) * dk] = d.repeat(G).to(dtype)
    want = [_attn_oracle(x.to(F64), q_w.to(F64), k_w.to(F64), H, G, dk, dv, 1e-5, 0.7, chunk) for x in qkv]
    portions = [[13, 50] + [1] * 12, [30, 2] + [1] * 5 + [0] * 7]
    at, got = [0, 0], [[], []]
    for step in range(14):
        ns = [portions[i][step] for i in range(2)]
        live = [i for i in range(2) if ns[i]]
        rows = torch.cat([qkv[i][at[i]:at[i] + ns[i]] for i in live]).to(cuda)
        slots = torch.tensor([tables[i][p // bs] * bs + p % bs for i in live for p in range(at[i], at[i] + ns[i])],
                             dtype=torch.int64, device=cuda)
        b = _batch(cuda, [ns[i] for i in live], [at[i] for i in live], [0] * len(live), [tables[i] for i in live])
        q = ops.qknorm_cache(rows, H, G, dk, dv, q_w.to(cuda), k_w.to(cuda), 1e-5, slots, kc, vc)
        o = ops.chunk_attention(q, kc, vc, b, 0.7, chunk, sink=1.0, sink_logit=0.0)
        r0 = 0
        for i in live:
            got[i].append(o[r0:r0 + ns[i]].float().cpu())
            r0 += ns[i]
            at[i] += ns[i]
    for i in range(2):
        assert at[i] == lens[i]
        _close(torch.cat(got[i]), want[i], 2e-5 if dtype == torch.float32 else 3e-2, f"sequence {i}")


def test_sink_and_padding_rows(cuda):
    """Scores far below zero: the sink takes nearly all the mass and the output shrinks accordingly; without a sink the
    same inputs give a convex combination.  A sequence marked as padding writes zeros."""
    ops = _ops()
    H = G = 1
    dk = dv = 8
    T = 6
    q = torch.ones(T, 1, dk, device=cuda)
    kc = torch.zeros(2, 1, 4, dk, device=cuda)
    vc = torch.ones(2, 1, 4, dv, device=cuda)
    kc[:] = -1.0                                                   # score = -8 * scale for every pair
    b = _batch(cuda, [T], [0], [0], [[1, 0]])
    with_sink = ops.chunk_attention(q, kc, vc, b, 0.5, 0, sink=1.0)
    no_sink = ops.chunk_attention(q, kc, vc, b, 0.5, 0, sink=0.0)
    for i in range(T):
        e = (i + 1) * math.exp(-4.0)
        assert abs(float(with_sink[i, 0, 0]) - e / (1 + e)) < 1e-6 and abs(float(no_sink[i, 0, 0]) - 1.0) < 1e-6
    pad = ops.chunk_attention(q, kc, vc, _batch(cuda, [T], [-1], [0], [[1, 0]]), 0.5, 0, sink=1.0)
    assert float(pad.abs().max()) == 0.0


# ------------------------------------------------------------------------------------------------ experts
@pytest.mark.parametrize("T,D,F,E,top", [(1, 48, 20, 5, 2), (7, 64, 96, 3, 3), (70, 50, 18, 4, 1), (150, 40, 72, 12, 3),
                                         (33, 256, 64, 40, 4), (1100, 64, 16, 10, 3), (1027, 36, 8, 3, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_and_experts(cuda, T, D, F, E, top, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn(T, D, generator=g).to(dtype)
    W = {"m.router": (torch.randn(E, D, generator=g) * D ** -0.5 * 3).to(dtype), "m.router.b": torch.randn(E, generator=g)}
    for e in range(E):
        W[f"m.e{e}.gate"] = (torch.randn(F, D, generator=g) * D ** -0.5).to(dtype)
        W[f"m.e{e}.up"] = (torch.randn(F, D, generator=g) * D ** -0.5).to(dtype)
        W[f"m.e{e}.down"] = (torch.randn(D, F, generator=g) * F ** -0.5).to(dtype)
    W64 = {k: v.to(F64) for k, v in W.items()}
    idx, wt = R.moe_route(h.to(F64), W64, "m", top)
    ids, wts = ops.moe_route(h.to(cuda), W["m.router"].to(cuda), W["m.router.b"].to(cuda), top)
    z = h.to(F64) @ W64["m.router"].t() + W64["m.router.b"]
    gap = torch.sort(z, -1, descending=True).values
    clear = (gap[:, :top] - gap[:, 1:top + 1]).min(-1).values > 1e-3 if top < E else torch.ones(T, dtype=torch.bool)
    assert clear.float().mean() > 0.8                               # rows without a near tie must agree exactly
    assert torch.equal(ids.cpu().long()[clear], idx[clear])
    _close(wts.cpu()[clear], wt[clear], 1e-5 if dtype == torch.float32 else 1e-2, "router weights")
    stack = lambda leaf: torch.stack([W[f"m.e{e}.{leaf}"] for e in range(E)]).to(cuda)      # noqa: E731
    # the grouped products are checked on the oracle's own choice, so that a near tie cannot hide in them
    y = ops.moe_experts(h.to(cuda), idx.to(torch.int32).to(cuda), wt.float().to(cuda), stack("gate"), stack("up"), stack("down"))
    want = torch.zeros(T, D, dtype=F64)
    for t in range(T):
        for j in range(top):
            e = int(idx[t, j])
            a = R.silu(W64[f"m.e{e}.gate"] @ h[t].to(F64)) * (W64[f"m.e{e}.up"] @ h[t].to(F64))
            want[t] += wt[t, j] * (W64[f"m.e{e}.down"] @ a)
    _close(y, want, 2e-5 if dtype == torch.float32 else 3e-2, "experts")
    # gate and up as views of the stacked [E, 2F, D] tensor (how the model holds them), and, for a batch large enough,
    # the grouped-GEMM path: same result
    gu = torch.cat([stack("gate"), stack("up")], 1).contiguous()
    y2 = ops.moe_experts(h.to(cuda), idx.to(torch.int32).to(cuda), wt.float().to(cuda), gu[:, :F], gu[:, F:], stack("down"),
                         w_gate_up=gu)
    _close(y2, want, 2e-5 if dtype == torch.float32 else 3e-2, "experts (stacked)")


def test_experts_large_batch_takes_the_grouped_gemm(cuda, monkeypatch):
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    T, D, F, E, top = 700, 64, 40, 7, 3
    assert T * top >= ops.MOE_GROUPED_GEMM_MIN_PAIRS
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).to(cuda)
    wr = (torch.randn(E, D, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
    gu = (torch.randn(E, 2 * F, D, generator=g) * D ** -0.5).to(torch.bfloat16).to(cuda)
    wd = (torch.randn(E, D, F, generator=g) * F ** -0.5).to(torch.bfloat16).to(cuda)
    ids, wts = ops.moe_route(h, wr, None, top)
    fast = ops.moe_experts(h, ids, wts, gu[:, :F], gu[:, F:], wd, w_gate_up=gu)
    monkeypatch.setattr(ops, "MOE_GROUPED_GEMM_MIN_PAIRS", 10 ** 9)
    own = ops.moe_experts(h, ids, wts, gu[:, :F], gu[:, F:], wd, w_gate_up=gu)
    _close(fast, own, 2e-2, "grouped GEMM against the tiled kernels")
    want = torch.zeros(T, D, dtype=F64)
    hf, guf, wdf = h.double().cpu(), gu.double().cpu(), wd.double().cpu()
    for t in range(0, T, 37):
        for j in range(top):
            e = int(ids[t, j])
            a = R.silu(guf[e, :F] @ hf[t]) * (guf[e, F:] @ hf[t])
            want[t] += float(wts[t, j]) * (wdf[e] @ a)
    _close(fast.cpu()[::37], want[::37], 3e-2, "grouped GEMM against the oracle")


def test_experts_do_not_depend_on_the_batch(cuda):
    """A token's result is the same bits alone and among 90 others (same tiles per row, same summation order)."""
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    D, F, E, top = 64, 48, 6, 2
    h = torch.randn(91, D, generator=g).to(torch.bfloat16).to(cuda)
    wr = torch.randn(E, D, generator=g).to(torch.bfloat16).to(cuda)
    wg, wu = (torch.randn(E, F, D, generator=g) * D ** -0.5).to(torch.bfloat16).to(cuda), \
        (torch.randn(E, F, D, generator=g) * D ** -0.5).to(torch.bfloat16).to(cuda)
    wd = (torch.randn(E, D, F, generator=g) * F ** -0.5).to(torch.bfloat16).to(cuda)
    ids, wts = ops.moe_route(h, wr, None, top)
    full = ops.moe_experts(h, ids, wts, wg, wu, wd)
    for t in (0, 45, 90):
        alone = ops.moe_experts(h[t:t + 1], ids[t:t + 1].contiguous(), wts[t:t + 1].contiguous(), wg, wu, wd)
        assert torch.equal(alone[0], full[t])
