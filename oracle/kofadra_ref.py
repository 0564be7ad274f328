"""Plain CPU restatement of the Kofadra decoder, one function per mechanism (test infrastructure only).

Everything runs token by token or with explicit loops in float64 on whole sequences; nothing here is shared with
the product path under vllm-backend-public_b200/ (which never imports this file).  `weights` maps the checkpoint's
tensor names to tensors; `cfg` is the parsed config.json dictionary.

Notation: T tokens, D model width, H query heads, G key/value heads, dk / dv per-head key and value sizes,
S residual streams, E experts.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(biased variance + eps) * w over the last axis."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_div(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------------------------------ mixers
def causal_conv(x, w):
    """x [T, C], w [C, taps]; y[t, c] = sum_j w[c, taps-1-j] * x[t-j, c], zeros before the sequence."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            if t - j >= 0:
                y[t] += w[:, taps - 1 - j] * x[t - j]
    return y


def delta_rule(q, k, v, beta, g):
    """Gated delta rule for ONE head.  q, k [T, dk]; v [T, dv]; beta, g [T].  Returns o [T, dv] and the last state."""
    T, dk = q.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=q.dtype)
    o = torch.zeros(T, dv, dtype=q.dtype)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        o[t] = S.t() @ q[t]
    return o, S


def delta_mixer(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """h [T, D] -> [T, D].  p = '<layer>.mix'."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ W[p + ".q"].t(), W[p + ".q.conv"])).view(T, G, dk)
    k = silu(causal_conv(h @ W[p + ".k"].t(), W[p + ".k.conv"])).view(T, G, dk)
    v = silu(causal_conv(h @ W[p + ".v"].t(), W[p + ".v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + ".b"].t())                                        # [T, H]
    g = torch.exp(-torch.exp(W[p + ".A_log"]) * softplus(h @ W[p + ".a"].t() + W[p + ".dt_bias"]))
    gate = silu(h @ W[p + ".g"].t()).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        kv = hh // (H // G)
        o, _ = delta_rule(q[:, kv], k[:, kv], v[:, hh], beta[:, hh], g[:, hh])
        out[:, hh] = rms_div(o, eps) * W[p + ".norm"] * gate[:, hh]
    return out.reshape(T, H * dv) @ W[p + ".o"].t()


def sink_attention(q, k, v, scale: float, chunk: Optional[int]):
    """ONE head.  q, k [T, dk]; v [T, dv].  Position i sees j <= i within its own block of `chunk` positions (all j <= i
    when chunk is None); the softmax denominator carries one extra unit term (a key of score 0 without a value)."""
    T = q.shape[0]
    o = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for i in range(T):
        lo = (i // chunk) * chunk if chunk else 0
        s = (k[lo:i + 1] @ q[i]) * scale
        mx = max(float(s.max()), 0.0)
        e = torch.exp(s - mx)
        o[i] = (e.unsqueeze(1) * v[lo:i + 1]).sum(0) / (math.exp(-mx) + e.sum())
    return o


def attention_mixer(h, W, p: str, m: dict, eps: float):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_div((h @ W[p + ".q"].t()).view(T, H, dk), eps) * W[p + ".q.norm"]
    k = rms_div((h @ W[p + ".k"].t()).view(T, G, dk), eps) * W[p + ".k.norm"]
    v = (h @ W[p + ".v"].t()).view(T, G, dv)
    chunk = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        kv = hh // (H // G)
        out[:, hh] = sink_attention(q[:, hh], k[:, kv], v[:, kv], m["scale"], chunk)
    return out.reshape(T, H * dv) @ W[p + ".o"].t()


# ------------------------------------------------------------------------------------------------ feed-forward
def moe_route(h, W, p: str, top: int):
    """Indices [T, top] and weights [T, top]: the `top` largest router logits, softmax over those only."""
    z = h @ W[p + ".router"].t() + W[p + ".router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe(h, W, p: str, f: dict):
    idx, wt = moe_route(h, W, p, f["router"]["top"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            a = silu(W[f"{p}.e{e}.gate"] @ h[t]) * (W[f"{p}.e{e}.up"] @ h[t])
            y[t] += wt[t, j] * (W[f"{p}.e{e}.down"] @ a)
    return y


# ------------------------------------------------------------------------------------------------ whole model
def layer_runs(cfg: dict) -> List[int]:
    """Layer index of every layer run, in execution order (a looped span repeats as a whole)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens, dtype=F64, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the summed residual stream after every layer run)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams")
    x0 = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    xs = x0.unsqueeze(0).repeat(S or 1, 1, 1)                                        # [S, T, D]
    trail = []
    for li in layer_runs(cfg):
        L = cfg["layers"][li]
        p = f"l{li}"
        for q_, sub in ((1, "mix"), (2, "mlp")):
            if sub == "mlp" and not L.get("mlp"):
                continue
            if S:
                hin, hout, hmix = W[f"{p}.hc{q_}.in"], W[f"{p}.hc{q_}.out"], W[f"{p}.hc{q_}.mix"]
            else:
                hin, hout, hmix = torch.ones(1, dtype=dtype), torch.ones(1, dtype=dtype), torch.ones(1, 1, dtype=dtype)
            u = (hin.view(-1, 1, 1) * xs).sum(0)
            hn = layer_norm(u, W[f"{p}.norm{q_}"], eps)
            if sub == "mix":
                fn = delta_mixer if L["type"] == "delta" else attention_mixer
                y = fn(hn, W, p + ".mix", L["mixer"], eps)
            else:
                if L["mlp"]["kind"] != "moe":
                    raise ValueError(L["mlp"]["kind"])
                y = moe(hn, W, p + ".mlp", L["mlp"])
            xs = torch.einsum("st,sij->tij", hmix, xs) + hout.view(-1, 1, 1) * y.unsqueeze(0)
        trail.append(xs.sum(0))
    x = layer_norm(xs.sum(0), W["final.norm"], eps)
    logits = x @ W["head"].t()
    return (logits, torch.stack(trail)) if return_layers else logits


# ------------------------------------------------------------------------------------------------ random models
def random_model(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 weights (every name the loader expects) for a config, scaled so that activations stay O(1)."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def rnd(*shape, std):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    W = {"embed": rnd(cfg["vocab"], D, std=1.0 / cfg["embedding"]["scale"]), "head": rnd(cfg["vocab"], D, std=D ** -0.5),
         "final.norm": 1 + rnd(D, std=0.1)}
    S = cfg.get("streams")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        W[p + ".norm1"] = 1 + rnd(D, std=0.1)
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            W[p + ".mix.q"] = rnd(H * dk, D, std=D ** -0.5)
            W[p + ".mix.k"] = rnd(G * dk, D, std=D ** -0.5)
            W[p + ".mix.v"] = rnd(G * dv, D, std=D ** -0.5)
            W[p + ".mix.q.norm"] = 1 + rnd(dk, std=0.1)
            W[p + ".mix.k.norm"] = 1 + rnd(dk, std=0.1)
        else:
            taps = m["conv"]
            W[p + ".mix.q"] = rnd(G * dk, D, std=D ** -0.5)
            W[p + ".mix.k"] = rnd(G * dk, D, std=D ** -0.5)
            W[p + ".mix.v"] = rnd(H * dv, D, std=D ** -0.5)
            for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                W[f"{p}.mix.{n}.conv"] = rnd(c, taps, std=taps ** -0.5)
            W[p + ".mix.b"] = rnd(H, D, std=D ** -0.5)
            W[p + ".mix.a"] = rnd(H, D, std=D ** -0.5)
            W[p + ".mix.A_log"] = rnd(H, std=0.5) - 1.0
            W[p + ".mix.dt_bias"] = rnd(H, std=0.5)
            W[p + ".mix.norm"] = 1 + rnd(dv, std=0.1)
            W[p + ".mix.g"] = rnd(H * dv, D, std=D ** -0.5)
        W[p + ".mix.o"] = rnd(D, H * dv, std=(H * dv) ** -0.5)
        f = L.get("mlp")
        if f:
            W[p + ".norm2"] = 1 + rnd(D, std=0.1)
            ff, E = f["expert"]["ff"], f["router"]["experts"]
            for e in range(E):
                W[f"{p}.mlp.e{e}.gate"] = rnd(ff, D, std=D ** -0.5)
                W[f"{p}.mlp.e{e}.up"] = rnd(ff, D, std=D ** -0.5)
                W[f"{p}.mlp.e{e}.down"] = rnd(D, ff, std=ff ** -0.5)
            W[p + ".mlp.router"] = rnd(E, D, std=4.0 * D ** -0.5)
            W[p + ".mlp.router.b"] = rnd(E, std=1.0)
        if S:
            for q_ in (1, 2) if f else (1,):
                W[f"{p}.hc{q_}.in"] = rnd(S, std=0.2) + 1.0 / S
                W[f"{p}.hc{q_}.out"] = rnd(S, std=0.2) + 1.0
                W[f"{p}.hc{q_}.mix"] = (torch.eye(S) + torch.randn(S, S, generator=g) * 0.1).to(torch.bfloat16)
    return W
