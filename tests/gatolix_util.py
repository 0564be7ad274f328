"""Helpers of the Gatolix tests: small configurations that differ from each other in every size and option."""
from typing import Optional

import gatolix_ref as R
from kofadra_util import TOL, make_engine, rel_err, replay, save_checkpoint, tokens  # noqa: F401  (shared test helpers)

YARN = {"factor": 3.0, "original": 64, "fast": 8.0, "slow": 2.0}


def mixer(heads, dim, rot_dim, vdim, kv_rank, window=None, scale=None, base=10000.0, scaling=None, dims=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
         "rot": {"base": base, "dims": dims if dims is not None else rot_dim}}
    if scaling:
        m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def layer(m, mlp=None):
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def config(width, vocab, layers, eps=1e-5, softcap: Optional[float] = 20.0):
    c = {"architecture": "Gatolix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}
    if softcap:
        c["logit_softcap"] = softcap
    return c


def cfg_a():      # odd vocabulary; a window below a page, one of 20, one layer without a window; a layer without feed-forward;
    # a pool read by the next layer; only part of the rotated entries turn in layer 2; sizes that are no multiples of 8
    return config(64, 97, [
        layer(mixer(4, 16, 8, 24, 48, window=8, scaling=YARN), dense(72)),
        layer(mixer(2, 8, 8, 12, 48, window=20, scaling=YARN, kv_from=0)),
        layer(mixer(3, 20, 12, 10, 36, scale=0.2, base=500.0, dims=8), moe(5, 2, 40, 0.5)),
        layer(mixer(3, 6, 12, 18, 36, window=33, scale=0.3, base=500.0, dims=8, kv_from=2), dense(30))])


def cfg_b():      # one head, a window of one token (a position sees only itself), no frequency scaling, no soft cap, one expert
    # chosen of three and every expert chosen
    return config(48, 130, [
        layer(mixer(1, 16, 16, 16, 32, window=1), moe(3, 1, 32, 2.0)),
        layer(mixer(2, 8, 4, 8, 16, window=16, base=100.0), moe(2, 2, 16, 0.25)),
        layer(mixer(2, 8, 4, 8, 16, window=17, base=100.0, kv_from=1), moe(4, 3, 24, 6.0))], eps=1e-6, softcap=None)


def cfg_c():      # sizes the tensor-core attention kernel takes in bf16 (latent a multiple of 64, rotated part a multiple of
    # 16), sixteen and eight heads, windows that end inside a key tile, three layers on one pool
    return config(128, 256, [
        layer(mixer(16, 16, 16, 16, 64, window=40, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}), dense(96)),
        layer(mixer(8, 32, 16, 24, 64, window=70, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}, kv_from=0),
              moe(8, 3, 32, 1.5)),
        layer(mixer(4, 8, 16, 8, 64, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}, kv_from=0), moe(6, 2, 16, 3.0)),
        layer(mixer(8, 16, 32, 32, 128, window=64), moe(4, 4, 64, 1.0))], softcap=5.0)


def cfg_d():      # a window longer than any test sequence, no feed-forward in the last layer, a wide latent
    return config(32, 50, [layer(mixer(2, 8, 8, 8, 160, window=4096, scaling={"factor": 2.0, "original": 16, "fast": 2.0, "slow": 1.0}),
                                 dense(16)),
                           layer(mixer(5, 4, 2, 6, 8, window=3))], softcap=50.0)


def cfg_e():      # nothing is a multiple of four: width 30, odd value size, latent 22, six rotated entries, expert width 10
    return config(30, 77, [
        layer(mixer(3, 6, 6, 5, 22, window=11, scaling={"factor": 5.0, "original": 24, "fast": 3.0, "slow": 0.25}), moe(3, 2, 10, 0.75)),
        layer(mixer(2, 10, 6, 7, 22, window=5, scaling={"factor": 5.0, "original": 24, "fast": 3.0, "slow": 0.25}, kv_from=0), dense(21)),
        layer(mixer(1, 2, 2, 3, 6, base=3.0))], eps=1e-4, softcap=8.0)


def cfg_f():      # head sizes for which long prompt portions rebuild keys and values per head (bf16): a pool read with and
    # without a window, a latent that only the warp kernel takes for the short rows beside it
    y = {"factor": 4.0, "original": 48, "fast": 6.0, "slow": 1.5}
    return config(64, 120, [
        layer(mixer(4, 16, 16, 32, 64, window=100, scaling=y), dense(48)),
        layer(mixer(2, 48, 16, 16, 64, scaling=y, kv_from=0), moe(4, 2, 32, 1.25)),
        layer(mixer(3, 8, 24, 48, 40, window=37, base=200.0), moe(3, 1, 24, 2.5)),
        layer(mixer(5, 40, 24, 16, 40, window=64, base=200.0, kv_from=2), dense(40))], softcap=12.0)


CONFIGS = {"a": cfg_a, "b": cfg_b, "c": cfg_c, "d": cfg_d, "e": cfg_e}


def oracle_logits(cfg: dict, weights, toks):
    return R.forward(cfg, weights, toks)
