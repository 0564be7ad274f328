"""Gatolix on the host (no GPU): the configuration reader and its refusals, and the plain oracle checked against cases
worked out by hand."""
import json
import math

import pytest
import torch

import gatolix_ref as R
import gatolix_util as U


def test_configuration_reader(tmp_path):
    from b200attn import gatolix
    from b200attn.model import resolve_config
    c = U.cfg_a()
    (tmp_path / "config.json").write_text(json.dumps(c))
    cfg = resolve_config(str(tmp_path))
    assert isinstance(cfg, gatolix.GatolixConfig) and cfg.family == "gatolix"
    assert (cfg.vocab, cfg.hidden, cfg.layers, cfg.eps, cfg.logit_softcap) == (97, 64, 4, 1e-5, 20.0)
    m0, m1, m2, m3 = (L.mixer for L in cfg.layer_specs)
    assert (m0.heads, m0.dim, m0.rot_dim, m0.vdim, m0.kv_rank, m0.window, m0.rot_dims) == (4, 16, 8, 24, 48, 8, 8)
    assert m0.rot_scaling == U.YARN and m0.kv_from is None and m1.kv_from == 0 and m3.kv_from == 2
    assert m2.window == 0 and m2.rot_dims == 8 and m2.rot_dim == 12 and m2.scale == 0.2 and m2.rot_base == 500.0
    assert isinstance(cfg.layer_specs[0].mlp, gatolix.DenseSpec) and cfg.layer_specs[1].mlp is None
    e = cfg.layer_specs[2].mlp
    assert (e.experts, e.top, e.ff, e.limit) == (5, 2, 40, 0.5)
    # two pools (layers 0 and 2), rows of 48 + 8 and 36 + 12 numbers
    assert cfg.kv_bytes_per_token(2) == 2 * (56 + 48) and cfg.state_bytes_per_seq() == 0
    assert cfg.params == sum(math.prod(s) for s in R.tensor_shapes(c).values())


@pytest.mark.parametrize("edit,match", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),            # itself
    (lambda c: c["layers"][1]["mixer"].update(kv_from=3), "kv_from"),            # a later layer
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),            # a layer without a pool of its own
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=40), "latent size"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(base=7.0), "rotation"),
    (lambda c: c["layers"][0].update(type="attention"), "mixer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "feed-forward kind"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=6), "router picks"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
])
def test_configuration_refusals(edit, match):
    from b200attn import gatolix
    c = U.cfg_a()
    edit(c)
    with pytest.raises(ValueError, match=match):
        gatolix.config_from_dict(c)


def test_oracle_rotary_frequencies_by_hand():
    f, mag = R.rotary_frequencies(8, 16.0, None)
    assert mag == 1.0 and f == pytest.approx([1.0, 0.5, 0.25, 0.125])
    # original 64: a pair turns t times within it when dims * ln(64 / (2 pi t)) / (2 ln base) is its index
    s = {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}
    lo = math.floor(8 * math.log(64 / (2 * math.pi * 4)) / (2 * math.log(16.0)))         # 1
    hi = math.ceil(8 * math.log(64 / (2 * math.pi * 1)) / (2 * math.log(16.0)))          # 4
    assert (lo, hi) == (1, 4)
    f2, mag2 = R.rotary_frequencies(8, 16.0, s)
    assert mag2 == pytest.approx(0.1 * math.log(4.0) + 1.0)
    ramps = [0.0, 0.0, 1 / 3, 2 / 3]
    assert f2 == pytest.approx([fi / 4.0 * r + fi * (1 - r) for fi, r in zip(f, ramps)])
    x = torch.tensor([1.0, 0.0, 0.0, 2.0, 5.0, 7.0], dtype=torch.float64)
    y = R.rotate(x, 3, [0.5, 0.25], 2.0, 4)
    assert y.tolist() == pytest.approx([2 * math.cos(1.5), 2 * math.sin(1.5), -4 * math.sin(0.75), 4 * math.cos(0.75), 5.0, 7.0])


def test_oracle_window_and_router_by_hand():
    # one head, keys that are zero: the output is the mean of the values in sight
    q = torch.ones(5, 1, 2, dtype=torch.float64)
    k = torch.zeros(5, 1, 2, dtype=torch.float64)
    v = torch.arange(5, dtype=torch.float64).view(5, 1, 1)
    assert R.windowed_attention(q, k, v, 1.0, 2)[:, 0, 0].tolist() == pytest.approx([0.0, 0.5, 1.5, 2.5, 3.5])
    assert R.windowed_attention(q, k, v, 1.0, 0)[:, 0, 0].tolist() == pytest.approx([0.0, 0.5, 1.0, 1.5, 2.0])
    assert R.windowed_attention(q[:2], k, v, 1.0, 3, first_pos=3)[:, 0, 0].tolist() == pytest.approx([2.0, 3.0])
    # router: equal logits -> equal scores 1/3; the correction alone decides, the weight stays 1/3
    w = {"l0.mlp.router": torch.zeros(3, 4), "l0.mlp.correction": torch.tensor([0.0, 0.2, 0.1])}
    ids, wts = R.route(torch.ones(1, 4, dtype=torch.float64), w, "l0", 2)
    assert ids.tolist() == [[1, 2]] and wts[0].tolist() == pytest.approx([1 / 3, 1 / 3])
    # the bounded gated unit: gate above the limit is cut, up is cut on both sides, and one is added to it
    w = {"l0.mlp.e0.gate": torch.tensor([[3.0], [-3.0]]), "l0.mlp.e0.up": torch.tensor([[5.0], [-5.0]]),
         "l0.mlp.e0.down": torch.eye(2)}
    y = R.expert(torch.ones(1, 1, dtype=torch.float64), w, "l0", 0, 2.0)
    assert y[0].tolist() == pytest.approx([2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0, -3.0 / (1 + math.exp(1.702 * 3.0)) * -1.0])


def test_oracle_prefix_property():
    """Logits at a position depend only on the tokens up to it (windows, shared pools and routing included)."""
    c = U.cfg_a()
    W = R.random_weights(c, 3)
    toks = U.tokens(30, c["vocab"], 5)
    full = R.forward(c, W, toks)
    part = R.forward(c, W, toks[:17])
    assert torch.allclose(full[:17], part, atol=1e-10)
