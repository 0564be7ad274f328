"""Kofadra decoder on the b200attn ops: a stack of pre-norm layers over fp32 hyper-connected residual streams, each
layer one sequence mixer (chunk-masked sink attention without rotation, or a gated delta-rule recurrence behind short
convolutions) and an optional routed mixture of gated experts; a span of layers may run several times with shared
weights, every pass keeping its own cache or state.

The model plugs into the same engine as LlamaModel (b200attn.engine.LLMEngine): paged K/V pools addressed through the
scheduler's block tables and slot mapping, recurrent state in the scheduler's per-sequence state slots, one forward over
[decode rows | prompt chunks], logits for the sampled rows.  Projections and the vocabulary head are library GEMMs
(torch -> cuBLAS); everything between them is this repo's kernels (csrc/hyper_norm.cu, delta_rule.cu,
chunk_attention.cu, moe.cu).  There is no CPU path.

Geometry, layer order, the loop, every size and constant come from the checkpoint's config.json
(`architecture: "Kofadra"`); weights from its *.safetensors, or random from a seed.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from . import ops

ARCHITECTURE = "Kofadra"


@dataclass
class MixerSpec:
    kind: str                  # "attention" | "delta"
    heads: int
    kv_heads: int
    dim: int                   # per-head query / key size
    vdim: int                  # per-head value size
    taps: int = 1              # delta: short convolution length
    chunk: int = 0             # attention: block-local causal mask (0 = plain causal)
    scale: float = 1.0         # attention: score scale


@dataclass
class MoESpec:
    experts: int
    top: int
    ff: int


@dataclass
class LayerSpec:
    mixer: MixerSpec
    mlp: Optional[MoESpec]


@dataclass
class KofadraConfig:
    name: str
    vocab: int
    hidden: int
    layer_specs: List[LayerSpec]
    eps: float = 1e-6
    streams: int = 0                       # 0: one plain residual (no hyper-connection tensors in the checkpoint)
    embed_scale: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    max_position: int = 1 << 20            # no positional table: only the cache bounds a sequence
    family: str = "kofadra"

    @property
    def runs(self) -> List[int]:
        """Layer index of every layer run in execution order; run r owns cache / state r."""
        n = len(self.layer_specs)
        if not self.loop:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    @property
    def layers(self) -> int:
        return len(self.runs)

    @property
    def params(self) -> int:
        n = 2 * self.vocab * self.hidden + self.hidden
        for L in self.layer_specs:
            m, D = L.mixer, self.hidden
            if m.kind == "attention":
                n += D * (m.heads * m.dim + m.kv_heads * (m.dim + m.vdim)) + 2 * m.dim
            else:
                C = 2 * m.kv_heads * m.dim + m.heads * m.vdim
                n += D * (C + m.heads * m.vdim + 2 * m.heads) + C * m.taps + 2 * m.heads + m.vdim
            n += m.heads * m.vdim * D + D
            if L.mlp:
                n += L.mlp.experts * (3 * L.mlp.ff * D + D + 1) + D
        return n

    def kv_bytes_per_token(self, kv_elem_bytes: int = 2, tp: int = 1) -> int:
        return sum((m.dim + m.vdim) * m.kv_heads * kv_elem_bytes
                   for m in (self.layer_specs[i].mixer for i in self.runs) if m.kind == "attention")

    def state_bytes_per_seq(self, elem_bytes: int = 2) -> int:
        n = 0
        for m in (self.layer_specs[i].mixer for i in self.runs):
            if m.kind == "delta":
                n += m.heads * m.dim * m.vdim * 4 + (m.taps - 1) * (2 * m.kv_heads * m.dim + m.heads * m.vdim) * elem_bytes
        return n

    def activation_bytes(self, tokens: int, seqs: int, elem_bytes: int = 2) -> int:
        wide = max([self.hidden] + [2 * (2 * m.kv_heads * m.dim + 2 * m.heads * m.vdim + m.heads * m.dim)
                                    for m in (L.mixer for L in self.layer_specs)])
        moe = max([0] + [L.mlp.top * (L.mlp.ff * elem_bytes + self.hidden * 4) for L in self.layer_specs if L.mlp])
        return tokens * (max(self.streams, 1) * self.hidden * 4 + 6 * wide * 4 + 2 * moe) + seqs * self.vocab * 8 + (1 << 28)

    def build_model(self, device, **kw):
        return KofadraModel(self, device, **kw)


def config_from_dict(c: dict, name: str = ARCHITECTURE) -> KofadraConfig:
    """config.json -> KofadraConfig.  Keys: vocab, width, norm.eps, embedding.scale, streams, loop {start, stop, times},
    layers [{type, mixer {heads, kv_heads, dim, vdim, conv | mask.size, scale}, mlp null | {kind: moe, expert.ff,
    router {experts, top}}}]."""
    specs = []
    for L in c["layers"]:
        m = L["mixer"]
        kind = L["type"]
        if kind not in ("attention", "delta"):
            raise ValueError(f"unknown mixer type {kind!r}")
        heads = int(m["heads"])
        spec = MixerSpec(kind, heads, int(m.get("kv_heads", heads)), int(m["dim"]), int(m.get("vdim", m["dim"])))
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads {spec.heads} not a multiple of kv_heads {spec.kv_heads}")
        if kind == "delta":
            spec.taps = int(m.get("conv", 1))
        else:
            spec.chunk = int((m.get("mask") or {}).get("size", 0))
            spec.scale = float(m.get("scale", spec.dim ** -0.5))
        f = L.get("mlp")
        mlp = None
        if f:
            if f.get("kind", "moe") != "moe":
                raise ValueError(f"unknown feed-forward kind {f.get('kind')!r}")
            mlp = MoESpec(int(f["router"]["experts"]), int(f["router"]["top"]), int(f["expert"]["ff"]))
            if not 1 <= mlp.top <= mlp.experts:
                raise ValueError(f"router picks {mlp.top} of {mlp.experts} experts")
        specs.append(LayerSpec(spec, mlp))
    loop = c.get("loop")
    lp = None
    if loop:
        lp = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
        if not 0 <= lp[0] <= lp[1] <= len(specs) or lp[2] < 1:
            raise ValueError(f"bad loop {loop}")
    return KofadraConfig(name=name, vocab=int(c["vocab"]), hidden=int(c["width"]), layer_specs=specs,
                         eps=float((c.get("norm") or {}).get("eps", 1e-6)), streams=int(c.get("streams") or 0),
                         embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)), loop=lp)


def config_from_dir(path: Path) -> KofadraConfig:
    return config_from_dict(json.loads((Path(path) / "config.json").read_text()), name=Path(path).name)


def bench_config(hidden: int, layers: int, heads: int, kv_heads: int, head_dim: int, ff: int, experts: int, top: int,
                 vocab: int, chunk: int = 1024, streams: int = 2, taps: int = 4, name: str = "kofadra-bench") -> KofadraConfig:
    """A model-sized geometry for benchmarks: delta and attention layers alternate (delta first)."""
    specs = []
    for i in range(layers):
        if i % 2 == 0:
            m = MixerSpec("delta", heads, kv_heads, head_dim, head_dim, taps=taps)
        else:
            m = MixerSpec("attention", heads, kv_heads, head_dim, head_dim, chunk=chunk, scale=head_dim ** -0.5)
        specs.append(LayerSpec(m, MoESpec(experts, top, ff)))
    return KofadraConfig(name, vocab, hidden, specs, streams=streams, embed_scale=1.0)


class KofadraModel:
    """Weights + per-run caches and states + forward over one scheduled token batch.  One instance per GPU."""

    supports_fp32 = True

    def __init__(self, cfg: KofadraConfig, device: torch.device, num_blocks: int, block_size: int = 16, seed: int = 0,
                 weights_dir: Optional[Path] = None, max_position: Optional[int] = None,
                 kv_dtype: torch.dtype = torch.bfloat16, tp=None, dtype: torch.dtype = torch.bfloat16,
                 max_num_seqs: int = 1):
        if device.type != "cuda":
            raise ValueError("KofadraModel needs a CUDA device (b200attn has no CPU path)")
        if tp is not None and tp.size > 1:
            raise ValueError("Kofadra runs on one GPU per replica: tensor_parallel_size must be 1")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype}: bfloat16 or float32")
        if kv_dtype not in (torch.bfloat16, dtype):
            raise ValueError("Kofadra keeps its K/V pools in the activation type (no fp8 cache)")
        self.cfg, self.dev, self.bs, self.dtype = cfg, device, block_size, dtype
        self.tp, self.tp_size, self.tp_rank = None, 1, 0
        self.vocab_parallel = False
        self.Hq = self.Hkv = 0                      # no paged-decode schedule to plan
        self.S = max(cfg.streams, 1)
        self.max_position = max_position or cfg.max_position
        self.max_num_seqs = max_num_seqs
        self.w: Dict[str, torch.Tensor] = {}
        if weights_dir is not None and any(Path(weights_dir).glob("*.safetensors")):
            self._load(Path(weights_dir))
        else:
            self._random_init(seed)
        self._fuse()
        self.num_blocks = 0
        self.k_cache: Dict[int, torch.Tensor] = {}
        self.v_cache: Dict[int, torch.Tensor] = {}
        self.conv_state: Dict[int, torch.Tensor] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self.alloc_cache(num_blocks)
        self.alloc_state(max_num_seqs)
        self.capture: Optional[list] = None         # tests: set to a list to collect the summed streams after every run

    # ------------------------------------------------------------------ weights
    def _tensor_names(self) -> Dict[str, Tuple[int, ...]]:
        """Name -> shape of every tensor of a checkpoint of this configuration."""
        c, D = self.cfg, self.cfg.hidden
        out = {"embed": (c.vocab, D), "final.norm": (D,), "head": (c.vocab, D)}
        for i, L in enumerate(c.layer_specs):
            p, m = f"l{i}", L.mixer
            out[p + ".norm1"] = (D,)
            if m.kind == "attention":
                out.update({p + ".mix.q": (m.heads * m.dim, D), p + ".mix.k": (m.kv_heads * m.dim, D),
                            p + ".mix.v": (m.kv_heads * m.vdim, D), p + ".mix.q.norm": (m.dim,), p + ".mix.k.norm": (m.dim,)})
            else:
                out.update({p + ".mix.q": (m.kv_heads * m.dim, D), p + ".mix.k": (m.kv_heads * m.dim, D),
                            p + ".mix.v": (m.heads * m.vdim, D), p + ".mix.q.conv": (m.kv_heads * m.dim, m.taps),
                            p + ".mix.k.conv": (m.kv_heads * m.dim, m.taps), p + ".mix.v.conv": (m.heads * m.vdim, m.taps),
                            p + ".mix.b": (m.heads, D), p + ".mix.a": (m.heads, D), p + ".mix.A_log": (m.heads,),
                            p + ".mix.dt_bias": (m.heads,), p + ".mix.norm": (m.vdim,), p + ".mix.g": (m.heads * m.vdim, D)})
            out[p + ".mix.o"] = (D, m.heads * m.vdim)
            if L.mlp:
                out[p + ".norm2"] = (D,)
                for e in range(L.mlp.experts):
                    out.update({f"{p}.mlp.e{e}.gate": (L.mlp.ff, D), f"{p}.mlp.e{e}.up": (L.mlp.ff, D),
                                f"{p}.mlp.e{e}.down": (D, L.mlp.ff)})
                out.update({p + ".mlp.router": (L.mlp.experts, D), p + ".mlp.router.b": (L.mlp.experts,)})
            if c.streams:
                for q in (1, 2) if L.mlp else (1,):
                    out.update({f"{p}.hc{q}.in": (c.streams,), f"{p}.hc{q}.out": (c.streams,),
                                f"{p}.hc{q}.mix": (c.streams, c.streams)})
        return out

    def _random_init(self, seed: int) -> None:
        g = torch.Generator(device=self.dev).manual_seed(seed)
        raw = {}
        for name, shape in self._tensor_names().items():
            leaf = name.rsplit(".", 1)[-1]
            fan = shape[-1] if len(shape) > 1 else 1
            t = torch.randn(*shape, generator=g, device=self.dev, dtype=torch.float32)
            if name.endswith(".mix.q.norm") or name.endswith(".mix.k.norm") or leaf in ("norm", "norm1", "norm2") \
                    or name == "final.norm":
                t = 1.0 + 0.1 * t
            elif leaf == "mix" and ".hc" in name:
                t = torch.eye(shape[0], device=self.dev) + 0.1 * t
            elif leaf in ("in", "out") and ".hc" in name:
                t = (1.0 / shape[0] if leaf == "in" else 1.0) + 0.1 * t
            elif leaf == "A_log":
                t = 0.5 * t - 1.0
            elif leaf in ("dt_bias", "b") and len(shape) == 1:
                t = 0.5 * t
            elif leaf == "conv":
                t = t * shape[1] ** -0.5
            elif name == "embed":
                t = t / max(self.cfg.embed_scale, 1e-6)
            else:
                t = t * fan ** -0.5
            raw[name] = t.to(torch.bfloat16)
        self._ingest(raw)

    def _load(self, path: Path) -> None:
        from safetensors import safe_open
        raw: Dict[str, torch.Tensor] = {}
        for f in sorted(path.glob("*.safetensors")):
            with safe_open(str(f), framework="pt", device="cpu") as sf:
                for k in sf.keys():
                    raw[k] = sf.get_tensor(k)
        want = self._tensor_names()
        missing = [k for k in want if k not in raw]
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {missing[:3]}")
        for k, shape in want.items():
            if tuple(raw[k].shape) != tuple(shape):
                raise ValueError(f"{k}: shape {tuple(raw[k].shape)} in the checkpoint, {tuple(shape)} by config.json")
        self._ingest({k: raw[k].to(self.dev) for k in want})

    def _ingest(self, raw: Dict[str, torch.Tensor]) -> None:
        """Matrices in the activation type, parameter vectors (and the stream-mixing matrices) in fp32."""
        for k, t in raw.items():
            small = t.dim() == 1 or k.endswith(".conv") or ".hc" in k
            self.w[k] = t.to(torch.float32 if small else self.dtype).contiguous()

    def _fuse(self) -> None:
        """Per layer: one projection matrix for the mixer's inputs, stacked expert matrices."""
        w, c = self.w, self.cfg
        for i, L in enumerate(c.layer_specs):
            p, m = f"l{i}", L.mixer
            if m.kind == "attention":
                w[p + ".wqkv"] = torch.cat([w.pop(p + ".mix.q"), w.pop(p + ".mix.k"), w.pop(p + ".mix.v")]).contiguous()
            else:
                # columns: q | k | v | output gate | beta input | decay input
                w[p + ".wproj"] = torch.cat([w.pop(p + ".mix.q"), w.pop(p + ".mix.k"), w.pop(p + ".mix.v"),
                                             w.pop(p + ".mix.g"), w.pop(p + ".mix.b"), w.pop(p + ".mix.a")]).contiguous()
                w[p + ".conv"] = torch.cat([w.pop(p + ".mix.q.conv"), w.pop(p + ".mix.k.conv"),
                                            w.pop(p + ".mix.v.conv")]).contiguous()
            if L.mlp:
                # gate and up stacked per expert [E, 2F, D] (one grouped product for both); down [E, D, F]
                w[f"{p}.mlp.gate_up"] = torch.stack([torch.cat([w.pop(f"{p}.mlp.e{e}.gate"), w.pop(f"{p}.mlp.e{e}.up")])
                                                     for e in range(L.mlp.experts)]).contiguous()
                w[f"{p}.mlp.down"] = torch.stack([w.pop(f"{p}.mlp.e{e}.down") for e in range(L.mlp.experts)]).contiguous()
        self._ones = torch.ones(self.S, dtype=torch.float32, device=self.dev)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.w.values())

    # ------------------------------------------------------------------ caches and state
    def alloc_cache(self, num_blocks: int) -> None:
        """K/V pools of every attention run: [num_blocks, G, bs, dk] and [num_blocks, G, bs, dv]."""
        self.num_blocks = int(num_blocks)
        self.k_cache.clear(), self.v_cache.clear()
        for r, li in enumerate(self.cfg.runs):
            m = self.cfg.layer_specs[li].mixer
            if m.kind == "attention":
                self.k_cache[r] = torch.zeros(num_blocks, m.kv_heads, self.bs, m.dim, dtype=self.dtype, device=self.dev)
                self.v_cache[r] = torch.zeros(num_blocks, m.kv_heads, self.bs, m.vdim, dtype=self.dtype, device=self.dev)

    def alloc_state(self, max_num_seqs: int) -> None:
        """Recurrent state of every delta run, one slot per live sequence: the matrix state (fp32) and the convolution
        tail (activation type).  Slots are never cleared: a sequence that starts at position 0 ignores their contents."""
        self.max_num_seqs = int(max_num_seqs)
        self.conv_state.clear(), self.state.clear()
        for r, li in enumerate(self.cfg.runs):
            m = self.cfg.layer_specs[li].mixer
            if m.kind == "delta":
                C = 2 * m.kv_heads * m.dim + m.heads * m.vdim
                self.state[r] = torch.zeros(max_num_seqs, m.heads, m.dim, m.vdim, dtype=torch.float32, device=self.dev)
                if m.taps > 1:
                    self.conv_state[r] = torch.zeros(max_num_seqs, m.taps - 1, C, dtype=self.dtype, device=self.dev)

    def prepare_decode(self, max_batch: int, max_nb: int) -> None:
        """Static index tensors of the decode-only batch (one row per sequence)."""
        self._arange = torch.arange(max_batch + 1, dtype=torch.int32, device=self.dev)

    def decode_schedule(self, seq_lens_host) -> int:
        return 0

    launches_per_layer = 9

    # ------------------------------------------------------------------ forward
    def _batch(self, n_decode: int, dec_bt, dec_sl, dec_state, prefill) -> ops.SeqBatch:
        """[decode rows | prompt chunks] as one list of sequences."""
        npf = prefill.cu_q.shape[0] - 1 if prefill is not None and prefill.total_tokens else 0
        if n_decode and not hasattr(self, "_arange") or (n_decode and self._arange.shape[0] < n_decode + 1):
            self._arange = torch.arange(n_decode + 1, dtype=torch.int32, device=self.dev)
        if n_decode and dec_state is None:
            raise ValueError("decode rows need their state slots")
        if npf and prefill.state_slots is None:
            raise ValueError("prompt chunks need their state slots")
        return ops.step_batch(self._arange, n_decode, dec_bt, dec_sl, dec_state, prefill)

    def _hc(self, li: int, q: int):
        """(in, out, mix) of sublayer q of layer li; None = the plain residual's ones / identity."""
        if not self.cfg.streams:
            return None, None, None
        p = f"l{li}.hc{q}"
        return self.w[p + ".in"], self.w[p + ".out"], self.w[p + ".mix"]

    def _mixer(self, r: int, li: int, h: torch.Tensor, slots: torch.Tensor, batch: ops.SeqBatch) -> torch.Tensor:
        m, w, p = self.cfg.layer_specs[li].mixer, self.w, f"l{li}"
        H, G, dk, dv = m.heads, m.kv_heads, m.dim, m.vdim
        if m.kind == "attention":
            qkv = torch.nn.functional.linear(h, w[p + ".wqkv"])
            q = ops.qknorm_cache(qkv, H, G, dk, dv, w[p + ".mix.q.norm"], w[p + ".mix.k.norm"], self.cfg.eps, slots,
                                 self.k_cache[r], self.v_cache[r])
            # the sink: one more term exp(0) in the denominator, no value
            o = ops.chunk_attention(q, self.k_cache[r], self.v_cache[r], batch, m.scale, m.chunk, sink=1.0, sink_logit=0.0)
            o = o.view(h.shape[0], H * dv)
        else:
            proj = torch.nn.functional.linear(h, w[p + ".wproj"])
            C = 2 * G * dk + H * dv
            off_g, off_b, off_a = C, C + H * dv, C + H * dv + H
            qkv, beta, decay = ops.delta_prep(proj, off_b, off_a, H, G, dk, dv, m.taps, w[p + ".conv"], w[p + ".mix.A_log"],
                                              w[p + ".mix.dt_bias"], batch, self.conv_state.get(r))
            o32 = ops.delta_scan(qkv, beta, decay, H, G, dk, dv, batch, self.state[r])
            o = ops.delta_out(o32, proj, off_g, w[p + ".mix.norm"], self.cfg.eps)
        return torch.nn.functional.linear(o, w[p + ".mix.o"])

    def _mlp(self, li: int, h: torch.Tensor) -> torch.Tensor:
        f, w, p = self.cfg.layer_specs[li].mlp, self.w, f"l{li}.mlp"
        ids, wts = ops.moe_route(h, w[p + ".router"], w[p + ".router.b"], f.top)
        gu = w[p + ".gate_up"]
        return ops.moe_experts(h, ids, wts, gu[:, :f.ff], gu[:, f.ff:], w[p + ".down"], w_gate_up=gu)

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, n_decode: int,
                dec_block_tables: Optional[torch.Tensor], dec_seq_lens: Optional[torch.Tensor], prefill,
                sample_rows: Optional[torch.Tensor], num_splits: int = 0,
                dec_state_slots: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens int64 [T] (rows [0, n_decode) = one new token per running sequence, the rest = prompt chunks),
        slots int64 [T] (cache slot of every row), positions unused (nothing in this design depends on them beyond
        the causal order).  Returns logits [len(sample_rows) or T, vocab] in the model's dtype."""
        c, w = self.cfg, self.w
        batch = self._batch(n_decode, dec_block_tables, dec_seq_lens, dec_state_slots, prefill)
        x = ops.embed_streams(w["embed"], tokens, self.S, c.embed_scale)
        runs = c.runs
        hin, _, _ = self._hc(runs[0], 1)
        h = ops.hc_step(x, in_w=hin, norm_w=w[f"l{runs[0]}.norm1"], eps=c.eps, h_dtype=self.dtype)
        for r, li in enumerate(runs):
            y = self._mixer(r, li, h, slots, batch)
            _, out1, mix1 = self._hc(li, 1)
            if c.layer_specs[li].mlp:
                in2, out2, mix2 = self._hc(li, 2)
                h = ops.hc_step(x, y, mix1, out1, in2, w[f"l{li}.norm2"], c.eps, h_dtype=self.dtype)
                y = self._mlp(li, h)
                out1, mix1 = out2, mix2
            if r + 1 < len(runs):
                nin, _, _ = self._hc(runs[r + 1], 1)
                h = ops.hc_step(x, y, mix1, out1, nin, w[f"l{runs[r + 1]}.norm1"], c.eps, h_dtype=self.dtype)
            else:
                ops.hc_step(x, y, mix1, out1)
            if self.capture is not None:
                self.capture.append(x.sum(1))
        if sample_rows is not None:
            x = x.index_select(0, sample_rows).contiguous()
        h = ops.hc_step(x, in_w=self._ones, norm_w=w["final.norm"], eps=c.eps, h_dtype=self.dtype)
        return torch.nn.functional.linear(h, w["head"])
