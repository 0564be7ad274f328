"""Plain CPU restatement of the Gatolix decoder, one function per mechanism (test infrastructure only).

Everything runs with explicit loops in float64 on whole sequences; nothing here is shared with the product path under
vllm-backend-public_b200/ (which never imports this file).  `weights` maps the checkpoint's tensor names to tensors;
`cfg` is the parsed config.json dictionary.

Notation: T tokens, D model width, H heads, dn / dr per-head unrotated and rotated query/key sizes, dv per-head value
size, R latent size, W window, E experts.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ norms
def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(biased variance + eps) * w + b over the last axis."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


# ------------------------------------------------------------------------------------------------ rotation
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """Angle per position step of every pair i < dims / 2, and the factor on cos and sin.  With `scaling`
    {factor, original, fast, slow}: pairs that turn fast keep their frequency, pairs that turn slowly are divided by
    `factor`, a linear ramp over the pair index in between."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, pos: int, freqs: List[float], mag: float, dims: int):
    """x [..., n]: the first `dims` entries are rotated pairwise (2i with 2i + 1) by pos * freqs[i]; the rest pass."""
    y = x.clone()
    for i in range(dims // 2):
        a = pos * freqs[i]
        c, s = math.cos(a) * mag, math.sin(a) * mag
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        y[..., 2 * i] = u * c - v * s
        y[..., 2 * i + 1] = v * c + u * s
    return y


# ------------------------------------------------------------------------------------------------ mixer
def latent_kv(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float):
    """What a layer that owns a down-projection caches per token: the normed latent c [T, R] and the rotated shared key
    part [T, dr]."""
    R, dr = m["kv_rank"], m["rot_dim"]
    rot = m["rot"]
    freqs, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    d = h @ w[p + ".mix.dkv"].to(F64).T
    c = rms_norm(d[:, :R], w[p + ".mix.dkv.norm"].to(F64), eps)
    kr = torch.stack([rotate(d[t, R:R + dr], t, freqs, mag, rot["dims"]) for t in range(h.shape[0])])
    return c, kr


def windowed_attention(q, k, v, scale: float, window: int, first_pos: int = 0):
    """q [Tq, H, dk] at positions first_pos .. first_pos + Tq - 1; k [Tk, H, dk], v [Tk, H, dv] at positions 0 .. Tk - 1.
    A query at position i attends to keys max(0, i - window + 1) .. i (window 0: keys 0 .. i), plain softmax over them.
    Returns [Tq, H, dv]."""
    Tq, H, _ = q.shape
    out = torch.zeros(Tq, H, v.shape[2], dtype=q.dtype)
    for t in range(Tq):
        i = first_pos + t
        first = max(0, i - window + 1) if window else 0
        for hh in range(H):
            s = (k[first:i + 1, hh] @ q[t, hh]) * scale
            pr = torch.softmax(s, 0)
            out[t, hh] = pr @ v[first:i + 1, hh]
    return out


def latent_attention(h, m: dict, w: Dict[str, torch.Tensor], p: str, c, kr):
    """h [T, D] -> [T, D].  Keys and values are rebuilt per head from the latent c (key = [W_uk c | shared rotated part]);
    head outputs are gated by sigmoid(W_g h)."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    rot = m["rot"]
    freqs, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    window = (m.get("mask") or {}).get("size") or 0
    q = (h @ w[p + ".mix.q"].to(F64).T).view(T, H, dn + dr).clone()
    for t in range(T):
        q[t, :, dn:] = rotate(q[t, :, dn:], t, freqs, mag, rot["dims"])
    gate = torch.sigmoid(h @ w[p + ".mix.g"].to(F64).T)                      # [T, H]
    kn = (c @ w[p + ".mix.uk"].to(F64).T).view(T, H, dn)
    k = torch.cat([kn, kr[:, None, :].expand(T, H, dr)], -1)
    v = (c @ w[p + ".mix.uv"].to(F64).T).view(T, H, dv)
    out = windowed_attention(q, k, v, m["scale"], window) * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + ".mix.o"].to(F64).T


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h, w, p: str):
    """W_down relu(W_up h)^2."""
    a = torch.relu(h @ w[p + ".mlp.up"].to(F64).T)
    return (a * a) @ w[p + ".mlp.down"].to(F64).T


def expert(h, w, p: str, e: int, limit: float):
    g = torch.clamp(h @ w[f"{p}.mlp.e{e}.gate"].to(F64).T, max=limit)
    u = torch.clamp(h @ w[f"{p}.mlp.e{e}.up"].to(F64).T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[f"{p}.mlp.e{e}.down"].to(F64).T


def route(h, w, p: str, top: int):
    """Softmax over all experts; the `top` largest of score + correction are chosen, weighted by the plain score."""
    s = torch.softmax(h @ w[p + ".mlp.router"].to(F64).T, -1)
    choice = s + w[p + ".mlp.correction"].to(F64)
    ids = torch.topk(choice, top, dim=-1).indices
    return ids, torch.gather(s, -1, ids)


def moe_ff(h, f: dict, w, p: str):
    ids, wts = route(h, w, p, f["router"]["top"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            y[t] += wts[t, j] * expert(h[t:t + 1], w, p, int(ids[t, j]), float(f["expert"]["limit"]))[0]
    return y


# ------------------------------------------------------------------------------------------------ model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None):
    """Logits [T, vocab] (float64) of one sequence from position 0; `layers_out` collects the residual after each layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"].to(F64)[torch.tensor(tokens)]
    kv = {}

    def ln(name, v):
        return layer_norm(v, w[name].to(F64), w[name + ".b"].to(F64), eps)

    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        if L["type"] != "latent_attention":
            raise ValueError(L["type"])
        h = ln(p + ".norm1", x)
        src = m.get("kv_from")
        if src is None:
            kv[i] = latent_kv(h, m, w, p, eps)
            src = i
        x = x + ln(p + ".norm1b", latent_attention(h, m, w, p, *kv[src]))
        f = L.get("mlp")
        if f:
            h = ln(p + ".norm2", x)
            y = dense_ff(h, w, p) if f["kind"] == "dense" else moe_ff(h, f, w, p)
            x = x + ln(p + ".norm2b", y)
        if layers_out is not None:
            layers_out.append(x.clone())
    z = ln("final.norm", x) @ w["head"].to(F64).T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


# ------------------------------------------------------------------------------------------------ random checkpoints
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "final.norm": (D,), "final.norm.b": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        p, m, f = f"l{i}", L["mixer"], L.get("mlp")
        H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if f else ()):
            out[f"{p}.{n}"] = (D,)
            out[f"{p}.{n}.b"] = (D,)
        out[p + ".mix.q"] = (H * (dn + dr), D)
        if m.get("kv_from") is None:
            out[p + ".mix.dkv"] = (R + dr, D)
            out[p + ".mix.dkv.norm"] = (R,)
        out.update({p + ".mix.uk": (H * dn, R), p + ".mix.uv": (H * dv, R), p + ".mix.g": (H, D), p + ".mix.o": (D, H * dv)})
        if f and f["kind"] == "dense":
            out.update({p + ".mlp.up": (f["ff"], D), p + ".mlp.down": (D, f["ff"])})
        elif f:
            F = f["expert"]["ff"]
            for e in range(f["router"]["experts"]):
                out.update({f"{p}.mlp.e{e}.gate": (F, D), f"{p}.mlp.e{e}.up": (F, D), f"{p}.mlp.e{e}.down": (D, F)})
            out.update({p + ".mlp.router": (f["router"]["experts"], D), p + ".mlp.correction": (f["router"]["experts"],)})
    return out


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 tensors by checkpoint name: matrices ~ N(0, 1 / fan-in), norm weights near one, small biases."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        t = torch.randn(*shape, generator=g)
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "b":
            t = 0.1 * t
        elif leaf == "correction":
            t = 0.05 * t
        elif len(shape) == 1:
            t = 1.0 + 0.1 * t
        elif name == "embed":
            pass
        elif leaf == "router":
            t = t * 2.0 * shape[1] ** -0.5
        else:
            t = t * shape[1] ** -0.5
        w[name] = t.to(torch.bfloat16)
    return w
