"""Host-side parts of the Kofadra integration (no GPU): configuration reader, layer-run order, the scheduler's replay
mode with state slots, and sanity of the plain oracle the GPU tests compare against."""
import math

import numpy as np
import pytest
import torch

import kofadra_ref as R
import kofadra_util as U
from b200attn import Scheduler, _lib
from b200attn.kofadra import KofadraConfig, config_from_dict
from b200attn.model import ARCHITECTURES, resolve_config


# ------------------------------------------------------------------------------------------------ configuration
def test_config_reads_every_size_and_orders_runs():
    c = config_from_dict(U.cfg_a())
    assert (c.vocab, c.hidden, c.streams, c.eps, c.embed_scale) == (97, 64, 2, 1e-5, 4.0)
    assert c.runs == [0, 1, 2, 1, 2, 3] and c.layers == 6
    m = c.layer_specs[1].mixer
    assert (m.kind, m.heads, m.kv_heads, m.dim, m.vdim, m.chunk, m.scale) == ("attention", 4, 1, 24, 16, 8, 0.3)
    assert c.layer_specs[1].mlp is None and c.layer_specs[0].mlp.top == 2 and c.layer_specs[0].mixer.taps == 3
    assert R.layer_runs(U.cfg_a()) == c.runs


def test_config_defaults_and_errors():
    c = config_from_dict(U.cfg_b())
    assert c.streams == 0 and c.loop is None and c.runs == [0, 1, 2]
    assert c.layer_specs[2].mixer.chunk == 0                       # no mask: plain causal
    assert config_from_dict(U.cfg_d()).runs == [0, 1] * 3
    bad = U.cfg_b()
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError, match="mixer type"):
        config_from_dict(bad)
    bad = U.cfg_b()
    bad["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(ValueError, match="feed-forward"):
        config_from_dict(bad)
    bad = U.cfg_a()
    bad["loop"]["stop"] = 9
    with pytest.raises(ValueError, match="loop"):
        config_from_dict(bad)


def test_cache_and_state_sizes_follow_the_runs():
    c = config_from_dict(U.cfg_a())
    # attention runs: layer 1 twice (G=1, 24+16) and layer 2 twice (G=2, 16+16), 2 bytes each
    assert c.kv_bytes_per_token(2) == 2 * (40 * 1 * 2) + 2 * (32 * 2 * 2)
    # delta runs: layer 0 (4 heads 16x24 fp32 + 2 tail rows of 2*2*16+4*24 channels) and layer 3 (2 heads 32x16 + 1 row of 2*32+2*16)
    assert c.state_bytes_per_seq(2) == 4 * 16 * 24 * 4 + 2 * 160 * 2 + 2 * 32 * 16 * 4 + 1 * 96 * 2


def test_model_directory_selects_the_family(tmp_path):
    import json
    (tmp_path / "config.json").write_text(json.dumps(U.cfg_c()))
    cfg = resolve_config(str(tmp_path))
    assert isinstance(cfg, KofadraConfig) and cfg.runs == [0, 1] and "Kofadra" in ARCHITECTURES
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(ValueError, match="unknown architecture"):
        resolve_config(str(tmp_path))


# ------------------------------------------------------------------------------------------------ scheduler replay mode
def test_replay_rows_slots_and_reuse():
    s = Scheduler(num_blocks=8, block_size=4, max_num_seqs=3, max_model_len=32, max_num_batched_tokens=64)
    p = s.step_explicit([10, 11], [5, 1])                          # both new: two prompt chunks, slots 0 and 1
    assert list(p.prefill_ids) == [10, 11] and list(p.prefill_state_slots) == [0, 1] and len(p.decode_ids) == 0
    assert list(p.prefill_start) == [0, 0] and list(p.prefill_len) == [5, 1] and list(p.prefill_last) == [0, 0]
    assert s.num_free_blocks == 8 - 2 - 1
    p = s.step_explicit([11, 10, 12], [1, 2, 3])                   # 11 decodes, 10 continues its prompt, 12 arrives
    assert list(p.decode_ids) == [11] and list(p.decode_state_slots) == [1] and list(p.seq_lens) == [2]
    assert list(p.prefill_ids) == [10, 12] and list(p.prefill_start) == [5, 0] and list(p.prefill_state_slots) == [0, 2]
    assert list(p.slot_mapping) == [int(p.block_tables[0, 0]) * 4 + 1]
    with pytest.raises(_lib.B2Error, match="max_num_seqs"):
        s.step_explicit([13], [1])                                 # a fourth live sequence
    free = s.num_free_blocks
    s.finish(10)                                                   # 7 tokens = 2 blocks and slot 0 come back
    assert s.num_free_blocks == free + 2
    p = s.step_explicit([13], [4])
    assert list(p.prefill_state_slots) == [0]                      # the lowest free slot is handed out again
    s.finish(11), s.finish(12)
    p = s.step_explicit([14, 15], [1, 1])
    assert sorted(p.prefill_state_slots) == [1, 2] and list(p.prefill_start) == [0, 0]     # first tokens are chunks


def test_replay_refuses_a_step_that_does_not_fit_and_applies_nothing():
    s = Scheduler(num_blocks=3, block_size=4, max_num_seqs=2, max_model_len=12, max_num_batched_tokens=64)
    s.step_explicit([1], [6])
    with pytest.raises(_lib.B2Error, match="blocks"):
        s.step_explicit([1, 2], [2, 5])                            # 1 would stay in its block, 2 needs two: one is free
    assert s.num_free_blocks == 1 and s.num_running == 1
    p = s.step_explicit([1, 2], [2, 4])
    assert list(p.prefill_start) == [6, 0] and s.num_free_blocks == 0
    with pytest.raises(_lib.B2Error):
        s.step_explicit([1, 1], [1, 1])                            # one request twice in a step


def test_policy_steps_carry_state_slots():
    s = Scheduler(num_blocks=16, block_size=4, max_num_seqs=2, max_model_len=32, max_num_batched_tokens=64)
    s.add_request(1, 5, 3), s.add_request(2, 3, 2), s.add_request(3, 2, 2)
    p = s.step()
    assert list(p.prefill_ids) == [1, 2] and list(p.prefill_state_slots) == [0, 1]
    p = s.step()
    assert list(p.decode_ids) == [1, 2] and list(p.decode_state_slots) == [0, 1]
    p = s.step()                                                   # 2 finished by length: 3 takes its slot
    assert 2 in list(p.finished_ids) and list(p.prefill_ids) == [3] and list(p.prefill_state_slots) == [1]


# ------------------------------------------------------------------------------------------------ the oracle itself
def test_oracle_delta_rule_by_hand():
    q = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=torch.float64)
    k = torch.tensor([[1.0, 0.0], [1.0, 1.0]], dtype=torch.float64)
    v = torch.tensor([[2.0], [3.0]], dtype=torch.float64)
    beta, g = torch.tensor([0.5, 1.0], dtype=torch.float64), torch.tensor([1.0, 0.5], dtype=torch.float64)
    o, S = R.delta_rule(q, k, v, beta, g)
    # t0: S = k0 (0.5*2)^T = [[1],[0]], o0 = 1.   t1: S = [[.5],[0]]; u = 3 - .5 = 2.5; S = [[3],[2.5]]; o1 = 2.5
    assert torch.allclose(o, torch.tensor([[1.0], [2.5]], dtype=torch.float64))
    assert torch.allclose(S, torch.tensor([[3.0], [2.5]], dtype=torch.float64))


def test_oracle_sink_and_block_mask():
    T, d = 7, 4
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(T, d, generator=g, dtype=torch.float64) for _ in range(3))
    o = R.sink_attention(q, k, v, 0.5, 3)
    # position 3 opens a block: it sees itself only, with weight e^s / (1 + e^s)
    s = float(q[3] @ k[3]) * 0.5
    assert torch.allclose(o[3], v[3] * (math.exp(s) / (1 + math.exp(s))))
    # position 5 sees 3, 4, 5 and nothing of the first block
    sc = (k[3:6] @ q[5]) * 0.5
    w = torch.exp(sc) / (1 + torch.exp(sc).sum())
    assert torch.allclose(o[5], (w.unsqueeze(1) * v[3:6]).sum(0))
    full = R.sink_attention(q, k, v, 0.5, None)
    assert not torch.allclose(full[5], o[5]) and torch.allclose(full[2], o[2])


def test_oracle_conv_and_router():
    x = torch.arange(12, dtype=torch.float64).view(6, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)      # last column = current token
    y = R.causal_conv(x, w)
    assert y[0, 0] == 0 * 100 and y[2, 0] == 4 * 100 + 2 * 10 + 0 * 1 and torch.equal(y[:, 1], x[:, 1])
    W = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=torch.float64),
         "r.router.b": torch.tensor([0.0, 0.5, -3.0], dtype=torch.float64)}
    idx, wt = R.moe_route(torch.tensor([[2.0, 1.0]], dtype=torch.float64), W, "r", 2)
    assert idx.tolist() == [[0, 1]] and torch.allclose(wt, torch.softmax(torch.tensor([[2.0, 1.5]], dtype=torch.float64), -1))
