"""The Gatolix family through the engine: checkpoints written to disk and loaded by the model directory, schedules replayed
through the scheduler and the latent pools, compared with the plain oracle over whole sequences.  Covers prefill against
token-by-token decoding, portions down to two tokens, unequal batches against each request alone, pages that are freed
and used again, the first tokens of a sequence, windows crossed in prompts and in decoding, long decoding, other page
sizes, and greedy generation through LLMEngine.generate and the server."""
import json

import pytest
import torch

import gatolix_ref as R
import gatolix_util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, make in U.CONFIGS.items():
        cfg = make()
        W = R.random_weights(cfg, seed=len(name) + ord(name))
        out[name] = (cfg, W, U.save_checkpoint(tmp_path_factory.mktemp("gatolix_" + name), cfg, W))
    return out


_oracle_cache = {}


def _oracle(name, cfg, W, toks):
    key = (name, tuple(toks))
    if key not in _oracle_cache:
        _oracle_cache[key] = U.oracle_logits(cfg, W, toks)
    return _oracle_cache[key]


def _check(got, name, cfg, W, reqs, dtype, what=""):
    for rid, toks in reqs.items():
        err = U.rel_err(got[rid], _oracle(name, cfg, W, toks), dtype)
        assert err <= U.TOL[dtype], f"{what} request {rid}: error {err:.3e} above {U.TOL[dtype]:.1e} ({dtype})"


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_token_by_token(cuda, models, name, dtype):
    cfg, W, path = models[name]
    eng = U.make_engine(path, dtype)
    reqs = {"p": U.tokens(90, cfg["vocab"], 1), "q": U.tokens(1, cfg["vocab"], 2)}
    whole = U.replay(eng, reqs, [[("p", 90)], [("q", 1)]])
    _check(whole, name, cfg, W, reqs, dtype, "whole")
    single = U.replay(eng, {"p": reqs["p"]}, [[("p", 1)] for _ in range(90)])          # every token a step of its own
    _check(single, name, cfg, W, {"p": reqs["p"]}, dtype, "token by token")
    assert U.rel_err(single["p"], whole["p"], dtype) <= U.TOL[dtype]
    eng.close()


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_many_sizes(cuda, models, name, dtype):
    """Cuts inside pages (16) and inside every window of the configurations (1 .. 70), portions of 2 and 3."""
    cfg, W, path = models[name]
    eng = U.make_engine(path, dtype)
    toks = U.tokens(131, cfg["vocab"], 7)
    for cuts in ([2, 3, 11, 17, 31, 2, 33, 30, 2], [64, 2, 2, 63], [15, 1, 1, 16, 32, 1, 65]):
        assert sum(cuts) == 131
        got = U.replay(eng, {"r": toks}, [[("r", n)] for n in cuts])
        _check(got, name, cfg, W, {"r": toks}, dtype, f"cuts {cuts}")
    eng.close()


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "float32"), ("d", "float32"),
                                        ("e", "float32"), ("a", "bfloat16"), ("c", "bfloat16"), ("e", "bfloat16")])
def test_unequal_batches_with_reuse_of_pages(cuda, models, name, dtype):
    """Up to four live requests, prompt portions beside single tokens; requests leave and new ones take over their pages
    (a pool of 15 pages for ~320 tokens in total).  Every request equals the oracle over its own tokens, and equals
    itself run alone."""
    cfg, W, path = models[name]
    V = cfg["vocab"]
    reqs = {"a": U.tokens(90, V, 1), "b": U.tokens(33, V, 2), "c": U.tokens(1, V, 3), "d": U.tokens(47, V, 4),
            "e": U.tokens(60, V, 5), "f": U.tokens(52, V, 6), "g": U.tokens(40, V, 7)}
    sched = [[("a", 30), ("b", 31), ("c", 1)],                       # c lives for one step
             [("a", 1), ("b", 1), ("d", 17)],
             [("a", 1), ("b", 1), ("d", 2), ("e", 3)],               # b ends: its pages go back
             [("a", 28), ("d", 1), ("e", 1), ("f", 20)],             # f takes them
             [("a", 1), ("d", 27), ("e", 40), ("f", 1)],             # d ends
             [("a", 29), ("e", 16), ("f", 31), ("g", 2)],            # a, e, f end
             [("g", 1)], [("g", 1)], [("g", 36)]]
    eng = U.make_engine(path, dtype, max_tokens=15 * 16)
    got = U.replay(eng, reqs, sched)
    _check(got, name, cfg, W, reqs, dtype, "mixed")
    assert eng.sched.num_free_blocks == eng.num_blocks and eng.sched.num_running == 0
    alone = U.replay(eng, {"e": reqs["e"]}, [[("e", 60)]])
    assert U.rel_err(got["e"], alone["e"], dtype) <= U.TOL[dtype]
    eng.close()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_long_portions_rebuild_keys_per_head(cuda, tmp_path, monkeypatch, dtype):
    """Steps with 256 prompt rows and more take another attention path in bf16 (keys and values per head over gathered pool
    rows): a whole prompt, long portions with context before them (inside and beyond the windows), a long portion beside
    decode rows and a short one, and the same requests cut small -- all against the oracle."""
    cfg = U.cfg_f()
    W = R.random_weights(cfg, seed=17)
    path = U.save_checkpoint(tmp_path / "f", cfg, W)
    V = cfg["vocab"]
    reqs = {"p": U.tokens(620, V, 1), "q": U.tokens(300, V, 2), "r": U.tokens(40, V, 3)}
    sched = [[("p", 300), ("r", 3)],                       # whole start of p beside a short portion
             [("p", 1), ("r", 1), ("q", 280)],             # decode rows beside a long portion from position 0
             [("p", 299), ("r", 1), ("q", 1)],             # a long portion with 301 tokens before it
             [("q", 19), ("p", 20), ("r", 35)]]            # short portions again
    from b200attn import ops
    calls, real = [], ops.window_attention
    monkeypatch.setattr(ops, "window_attention", lambda *a, **k: (calls.append(a[0].shape[0]), real(*a, **k))[1])
    eng = U.make_engine(path, dtype, max_tokens=1024)
    got = U.replay(eng, reqs, sched)
    for rid, toks in reqs.items():
        err = U.rel_err(got[rid], U.oracle_logits(cfg, W, toks), dtype)
        assert err <= U.TOL[dtype], f"request {rid}: error {err:.3e} ({dtype})"
    layers = len(cfg["layers"])
    assert calls == ([303] * layers + [280] * layers + [299] * layers if dtype == "bfloat16" else [])
    small = U.replay(eng, {"q": reqs["q"]}, [[("q", 100)], [("q", 100)], [("q", 100)]])
    assert U.rel_err(small["q"], got["q"], dtype) <= U.TOL[dtype]
    eng.close()


@pytest.mark.parametrize("eager", [False, True])
def test_long_decoding_through_graph_and_eager_steps(cuda, models, eager):
    """A 20-token prompt then 230 single-token steps (the decode-only step is a CUDA graph unless eager), beside a second
    request that joins late: every window slides over decoded tokens many times."""
    cfg, W, path = models["a"]
    reqs = {"x": U.tokens(250, cfg["vocab"], 21), "y": U.tokens(120, cfg["vocab"], 22)}
    sched = [[("x", 20)]] + [[("x", 1)] for _ in range(110)] + [[("x", 1), ("y", 1)] for _ in range(120)]
    eng = U.make_engine(path, "float32", eager=eager)
    got = U.replay(eng, reqs, sched)
    _check(got, "a", cfg, W, reqs, "float32", "long decode")
    assert eng.stats.decode_steps >= 229 and (eager or len(eng._graphs) >= 2)
    eng.close()


def test_block_size_and_pool_do_not_change_the_logits(cuda, models):
    cfg, W, path = models["c"]
    toks = U.tokens(77, cfg["vocab"], 9)
    ref = None
    for bs in (8, 16, 32):
        eng = U.make_engine(path, "float32", max_tokens=96, block_size=bs)
        got = U.replay(eng, {"r": toks}, [[("r", 50)], [("r", 2)], [("r", 25)]])["r"]
        _check({"r": got}, "c", cfg, W, {"r": toks}, "float32", f"block size {bs}")
        ref = got if ref is None else ref
        assert U.rel_err(got, ref) <= 1e-5
        eng.close()


def test_residual_after_every_layer(cuda, models):
    """The fp32 residual after each layer against the oracle's, for a prompt fed in two portions."""
    cfg, W, path = models["a"]
    toks = U.tokens(40, cfg["vocab"], 3)
    want = []
    R.forward(cfg, W, toks, want)
    eng = U.make_engine(path, "float32")
    eng.model.capture = []
    eng.replay_step([("r", toks[:25], [])])
    eng.replay_step([("r", toks[25:], [])], ["r"])
    n = len(cfg["layers"])
    for i in range(n):
        got = torch.cat([eng.model.capture[i], eng.model.capture[n + i]]).cpu().double()
        assert float((got - want[i]).abs().max()) <= 2e-4 * float(want[i].abs().max()), f"layer {i}"
    eng.close()


@pytest.mark.parametrize("name", ["a", "c"])
def test_greedy_generation_through_the_engine(cuda, models, name):
    """LLMEngine.generate (scheduler policy, chunked prefill, CUDA-graph decode, b2_sample at temperature 0) continues
    three prompts exactly as the oracle's argmax does, with fewer sequence slots than requests."""
    from b200attn.engine import SamplingParams
    cfg, W, path = models[name]
    eng = U.make_engine(path, "float32", max_num_seqs=2)
    prompts = [U.tokens(n, cfg["vocab"], 30 + n) for n in (5, 29, 1)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    for p, out in zip(prompts, outs):
        seq = list(p)
        for k in range(12):
            lg = U.oracle_logits(cfg, W, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) < 1e-3 * float(lg.abs().max()):
                break                                               # a near tie: either continuation is right
            assert out[k] == int(lg.argmax()), f"token {k} of prompt of {len(p)}"
            seq.append(out[k])
    eng.close()


def test_random_init_and_checkpoint_shape_check(cuda, tmp_path, models):
    """Without weights in the directory the engine serves seeded random weights of the configuration; a checkpoint
    whose shapes contradict config.json, or that lacks a tensor, is refused."""
    cfg, W, _ = models["b"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    eng = U.make_engine(tmp_path, "bfloat16")
    lg = eng.replay_step([("r", U.tokens(9, cfg["vocab"], 1), [8])], ["r"])
    assert lg.shape == (1, cfg["vocab"]) and bool(torch.isfinite(lg).all())
    eng.close()
    bad = dict(W)
    bad["l1.mix.dkv.norm"] = torch.zeros(5, dtype=torch.bfloat16)
    U.save_checkpoint(tmp_path / "bad", cfg, bad)
    with pytest.raises(ValueError, match="dkv.norm"):
        U.make_engine(tmp_path / "bad", "bfloat16")
    lacking = {k: v for k, v in W.items() if k != "l2.norm2b.b"}
    U.save_checkpoint(tmp_path / "lacking", cfg, lacking)
    with pytest.raises(ValueError, match="lacks"):
        U.make_engine(tmp_path / "lacking", "bfloat16")


def test_server_serves_a_model_directory(cuda, models):
    """`python -m b200attn.server --model DIR --dtype float32`: the family comes from config.json, a completion is the
    oracle's greedy continuation of a token-id prompt."""
    import os
    import socket
    import subprocess
    import sys
    import time
    from pathlib import Path

    import requests
    cfg, W, path = models["a"]
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root / "vllm-backend-public_b200"))
    proc = subprocess.Popen([sys.executable, "-m", "b200attn.server", "--model", str(path), "--dtype", "float32", "--port", str(port),
                             "--host", "127.0.0.1", "--max-num-seqs", "4", "--max-model-len", "256",
                             "--num-gpu-blocks-override", "80", "--served-model-name", "gatolix-test"], env=env,
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    base = f"http://127.0.0.1:{port}"
    try:
        for _ in range(600):
            if proc.poll() is not None:
                raise RuntimeError("server exited: " + proc.stdout.read().decode()[-2000:])
            try:
                if requests.get(base + "/health", timeout=1).status_code == 200:
                    break
            except requests.RequestException:
                pass
            time.sleep(0.2)
        else:
            raise RuntimeError("server did not become healthy")
        prompt = U.tokens(13, cfg["vocab"], 78)
        r = requests.post(base + "/v1/completions", json={"model": "gatolix-test", "prompt": prompt, "max_tokens": 6,
                                                          "temperature": 0.0, "ignore_eos": True}, timeout=60)
        assert r.status_code == 200, r.text
        body = r.json()
        assert body["usage"]["prompt_tokens"] == 13 and body["usage"]["completion_tokens"] == 6
        seq = list(prompt)
        for _ in range(6):
            seq.append(int(U.oracle_logits(cfg, W, seq)[-1].argmax()))
        want = bytes(t % 256 for t in seq[13:]).decode("utf-8", errors="replace")      # the byte tokenizer's text
        assert body["choices"][0]["text"] == want
    finally:
        proc.terminate()
        try:
            proc.wait(20)
        except subprocess.TimeoutExpired:
            proc.kill()


def test_trace_runner_replays_a_schedule(cuda, tmp_path, models):
    """bin/trace_run on a model directory: steps from standard input, logits files and `done` lines out."""
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np
    cfg, W, path = models["d"]
    toks = U.tokens(40, cfg["vocab"], 11)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:31], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[31:], "want": [8]}, {"id": "y", "tokens": toks[:2], "want": [1]}],
              "end": ["x", "y"]}]
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    out.mkdir()
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(path), "--dtype", "float32", "--out",
                        str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                       capture_output=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = U.oracle_logits(cfg, W, toks)
    a = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    c = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1))
    assert not (out / "1.f32").exists()
    assert U.rel_err(a, want[[0, 29]]) <= U.TOL["float32"] and U.rel_err(c, want[[39, 1]]) <= U.TOL["float32"]
