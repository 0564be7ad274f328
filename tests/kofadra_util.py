"""Helpers of the Kofadra tests: small configurations, checkpoints on disk, schedules replayed through the engine."""
import json
from pathlib import Path
from typing import Dict, List, Sequence, Tuple

import torch

import kofadra_ref as R


def attn(heads, kv_heads, dim, vdim, chunk=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if chunk:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, taps, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}, "mlp": mlp}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(width, vocab, layers, streams=None, loop=None, eps=1e-5, scale=4.0):
    c = {"architecture": "Kofadra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
         "embedding": {"scale": scale}}
    if streams is not None:
        c["streams"] = streams
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# Four geometries that differ from each other in every size, in layer order and in which optional parts they have.
def cfg_a():      # odd vocabulary, G < H, a looped span, a layer without feed-forward, a chunk that is no multiple of a page
    return config(64, 97, [delta(4, 2, 16, 24, 3, moe(5, 2, 40)), attn(4, 1, 24, 16, chunk=8, scale=0.3),
                           attn(2, 2, 16, 16, chunk=20, mlp=moe(4, 3, 24)), delta(2, 1, 32, 16, 2, moe(3, 1, 16))],
                  streams=2, loop=(1, 3, 2))


def cfg_b():      # plain residual (no stream tensors), no loop, one expert of three, a layer with plain causal attention
    return config(48, 130, [attn(3, 3, 16, 16, chunk=16, mlp=moe(3, 1, 32)), delta(3, 3, 16, 16, 4, moe(3, 2, 20)),
                            attn(2, 1, 8, 24, mlp=moe(2, 2, 16))], eps=1e-6, scale=1.0)


def cfg_c():      # one stream with its tensors, a loop of one pass, every expert chosen, head sizes that are no power of two
    return config(80, 64, [delta(2, 2, 40, 72, 1, moe(2, 2, 48)), attn(5, 5, 40, 8, chunk=5, scale=0.2, mlp=moe(6, 2, 8))],
                  streams=1, loop=(0, 2, 1))


def cfg_d():      # four streams, the whole stack looped three times, long convolution
    return config(32, 50, [delta(2, 1, 8, 8, 6, moe(4, 2, 16)), attn(2, 2, 8, 8, chunk=32, mlp=moe(4, 1, 16))], streams=4,
                  loop=(0, 2, 3))


def cfg_e():      # head sizes the tensor-core prompt kernel takes in bf16 (multiples of 32), dk != dv, three streams
    return config(96, 200, [attn(4, 2, 32, 64, chunk=24, scale=0.25, mlp=moe(8, 2, 32)), delta(2, 2, 32, 32, 4, moe(8, 3, 24)),
                            attn(2, 1, 64, 32, chunk=40)], streams=3, loop=(0, 1, 2))


def save_checkpoint(path: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    from safetensors.torch import save_file
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(path / "model.safetensors"))
    return path


def make_engine(model_dir: Path, dtype: str, max_tokens: int = 512, block_size: int = 16, max_num_seqs: int = 4,
                eager: bool = False, num_blocks=None):
    from b200attn.engine import LLMEngine
    from b200attn.model import resolve_config
    cfg = resolve_config(str(model_dir))
    nb = (max_tokens + block_size - 1) // block_size
    return LLMEngine(cfg, torch.device("cuda", 0), max_num_seqs=max_num_seqs, max_model_len=nb * block_size,
                     block_size=block_size, num_blocks=(num_blocks or nb) + 1, max_num_batched_tokens=nb * block_size,
                     weights_dir=model_dir, dtype=dtype, enforce_eager=eager)


def replay(engine, requests: Dict[str, Sequence[int]], schedule: List[List[Tuple[str, int]]]) -> Dict[str, torch.Tensor]:
    """Feed `requests` step by step ([(id, how many of its next tokens)] per step), ask for the logits of every
    position, release a request with its last token.  Returns id -> [len, vocab]."""
    at = {k: 0 for k in requests}
    got: Dict[str, list] = {k: [] for k in requests}
    for step in schedule:
        entries, end = [], []
        for rid, n in step:
            lo, hi = at[rid], at[rid] + n
            assert hi <= len(requests[rid])
            entries.append((rid, list(requests[rid][lo:hi]), list(range(n))))
            at[rid] = hi
            if hi == len(requests[rid]):
                end.append(rid)
        lg = engine.replay_step(entries, end)
        off = 0
        for rid, n in step:
            got[rid].append(lg[off:off + n])
            off += n
    assert all(at[k] == len(requests[k]) for k in requests)
    return {k: torch.cat(v) for k, v in got.items()}


def rel_err(got: torch.Tensor, want: torch.Tensor, dtype: str = "float32") -> float:
    """Per position: rms of the difference over the vocabulary (mean removed) / rms of the expected logits.
    float32: the worst position.  bfloat16: the 80th percentile -- in 16 bits a router logit within rounding of the next
    one may pick another expert at a few positions of these tiny random models, which is a close call and not a fault;
    every mechanism's logic is pinned by the float32 runs of the same schedules."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    e = d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()
    return float(e.max()) if dtype == "float32" else float(torch.quantile(e, 0.8))


TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def oracle_logits(cfg: dict, weights, toks) -> torch.Tensor:
    return R.forward(cfg, weights, toks)
