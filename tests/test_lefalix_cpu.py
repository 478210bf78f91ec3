"""Lefalix without a GPU: configuration parsing, the layer schedule, rotary frequencies, checkpoint names, the registry and the
oracle's own consistency (a prompt recomputed from a longer one, causal convolution and delta rule against closed forms)."""
from __future__ import annotations

import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import lefalix_oracle as O  # noqa: E402
from test_gpu_lefalix import CFG_ODD, CFG_WIDE, _write_checkpoint, checkpoint, tokens_for  # noqa: E402


def test_config_parses_every_branch():
    from lit_gpt_b200.config import DenseMLPSpec, GatedMoESpec, LefalixConfig

    c = LefalixConfig.from_dict(CFG_ODD)
    assert (c.vocab_size, c.n_embd, c.n_layer) == (83, 40, 4) and (c.loop_start, c.loop_stop, c.loop_times) == (1, 3, 3)
    left = c.layers[1].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.conv, left.window, left.scale) == (4, 2, 10, 6, 2, 7, 0.9)
    assert left.rot.factor == 3.0 and c.layers[2].mixer.left.rot.factor is None
    assert c.layers[0].mixer.channel and not c.layers[1].mixer.right.channel
    assert isinstance(c.layers[0].mlp, DenseMLPSpec) and c.layers[2].mlp is None
    m = c.layers[3].mlp
    assert isinstance(m, GatedMoESpec) and (m.experts, m.top, m.groups, m.keep) == (5, 3, 1, 1)      # no groups entry: one group
    runs = c.schedule()
    assert [r[0] for r in runs] == [0, 1, 2, 1, 2, 1, 2, 3] and [r[2] for r in runs] == [False, False, False, True, False, True, False, False]
    assert [r[1] for r in runs] == list(range(8))                                                  # a state per run
    w = LefalixConfig.from_dict(CFG_WIDE)                                                          # no loop entry at all
    assert [r[0] for r in w.schedule()] == [0, 1, 2] and not any(r[2] for r in w.schedule())
    assert [(i, r) for i, r in O.layer_runs(CFG_ODD)] == [(r[0], r[2]) for r in runs]


def test_bad_configurations_are_refused():
    import copy

    from lit_gpt_b200.config import LefalixConfig

    bad = copy.deepcopy(CFG_ODD)
    bad["layers"][1]["type"] = "something"
    with pytest.raises(ValueError, match="unknown mixer type"):
        LefalixConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_ODD)
    bad["loop"]["stop"] = 9
    with pytest.raises(ValueError, match="loop"):
        LefalixConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_ODD)
    bad["layers"][1]["mlp"]["router"]["groups"]["keep"] = 0
    with pytest.raises(ValueError, match="groups"):
        LefalixConfig.from_dict(bad)


@pytest.mark.parametrize("rot", [dict(base=100.0, dims=6, scaling=dict(factor=3.0, original=16, fast=4.0, slow=1.0)), dict(base=1e4, dims=24),
                                 dict(base=5e5, dims=64, scaling=dict(factor=16.0, original=4096, fast=32.0, slow=1.0))])
def test_rotary_frequencies(rot):
    from lit_gpt_b200.config import RotarySpec

    sc = rot.get("scaling")
    spec = RotarySpec(dims=rot["dims"], base=rot["base"]) if sc is None else RotarySpec(rot["dims"], rot["base"], sc["factor"], sc["original"],
                                                                                       sc["fast"], sc["slow"])
    got, want = torch.tensor(spec.frequencies(), dtype=torch.float64), O.rotary_frequencies(rot)
    assert torch.allclose(got, want, rtol=1e-12, atol=0)
    assert spec.magnitude == (1.0 if sc is None else 0.1 * math.log(sc["factor"]) + 1.0)
    if sc is not None:   # fast-turning pairs keep their frequency, the slowest are divided by the factor
        plain = torch.tensor(RotarySpec(rot["dims"], rot["base"]).frequencies(), dtype=torch.float64)
        assert got[0] == plain[0] and abs(float(got[-1] / plain[-1]) - 1.0 / sc["factor"]) < 1e-12


def test_registry_and_loader_on_cpu(tmp_path):
    from lit_gpt_b200.checkpoint import load_registered
    from lit_gpt_b200.config import LefalixConfig, load_config, model_class
    from lit_gpt_b200.lefalix import Lefalix

    w = checkpoint(CFG_ODD, 3)
    _write_checkpoint(tmp_path, CFG_ODD, w)
    cfg = load_config(tmp_path)
    assert isinstance(cfg, LefalixConfig) and model_class(cfg) is Lefalix
    model = load_registered(tmp_path, dtype=torch.float32, device="cpu")
    assert model.blocks[0].mixer.spec.decay_rank == 5 and model.blocks[0].mixer.spec.gate_rank == 7      # read from the weights' shapes
    mx = model.blocks[1].mixer
    assert torch.equal(mx.left.w_qkv[: 4 * 10], w["l1.mix.left.q"].float()) and torch.equal(mx.left.b_qkv[4 * 10 : 6 * 10], w["l1.mix.left.k.b"].float())
    assert torch.equal(mx.right.w_in[-3:], w["l1.mix.right.b"].float()) and torch.equal(mx.right_out, w["l1.mix.right.out"].float())
    ex = model.blocks[1].mlp
    assert torch.equal(ex.w_up[4, :14], w["l1.mlp.e4.gate"].float()) and torch.equal(ex.w_up[4, 14:], w["l1.mlp.e4.up"].float())
    assert model.blocks[2].mlp is None and model.blocks[2].norm_2 is None
    del w["l3.mix.a2"]
    _write_checkpoint(tmp_path, CFG_ODD, w)
    with pytest.raises(KeyError, match="l3.mix.a2"):
        load_registered(tmp_path, dtype=torch.float32, device="cpu")
    w = checkpoint(CFG_ODD, 3)
    w["l0.mix.extra"] = torch.zeros(2, dtype=torch.bfloat16)
    _write_checkpoint(tmp_path, CFG_ODD, w)
    with pytest.raises(KeyError, match="unexpected"):
        load_registered(tmp_path, dtype=torch.float32, device="cpu")


def test_oracle_is_causal_and_its_mechanisms_match_closed_forms():
    w = checkpoint(CFG_ODD, 7)
    toks = tokens_for(CFG_ODD, 30, 7)
    whole = O.forward(CFG_ODD, w, toks)
    assert torch.allclose(O.forward(CFG_ODD, w, toks[:17]), whole[:17], rtol=1e-9, atol=1e-9)
    # convolution: the last tap multiplies the current input, nothing reaches back past the first position
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    y = O.causal_conv(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    # delta rule with beta = 1, no decay, orthonormal keys: a look-up table; rewriting a key replaces its value
    k = torch.eye(3, dtype=torch.float64)[[0, 1, 0]]
    v = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=torch.float64)
    o = O.delta_scan(k, k, v, torch.ones(3, dtype=torch.float64), torch.ones(3, dtype=torch.float64))
    assert torch.equal(o, v)
    q = torch.eye(3, dtype=torch.float64)[[2, 0, 1]]
    o = O.delta_scan(q, k, v, torch.full((3,), 0.5, dtype=torch.float64), torch.ones(3, dtype=torch.float64))
    assert o[0].tolist() == [0.0, 0.0] and o[1].tolist() == [0.5, 1.0] and o[2].tolist() == [1.5, 2.0]      # decayed before the write and the read
    # sink: a lone key with score 0 weighs 1 / (1 + e^sink)
    m = dict(heads=1, kv_heads=1, dim=2, vdim=2, mask=dict(size=4), scale=1.0, rot=None)
    W = {"p.q": torch.zeros(2, 3), "p.k": torch.zeros(2, 3), "p.v": torch.zeros(2, 3), "p.q.b": torch.zeros(2), "p.k.b": torch.zeros(2),
         "p.v.b": torch.ones(2), "p.q.conv": torch.ones(2, 1), "p.k.conv": torch.ones(2, 1), "p.v.conv": torch.ones(2, 1),
         "p.sink": torch.tensor([1.0]), "p.o": torch.eye(2), "p.o.b": torch.zeros(2)}
    W = {k_: v_.double() for k_, v_ in W.items()}
    out = O.window_attention(torch.zeros(1, 3, dtype=torch.float64), W, "p.", m, 1e-5)
    assert torch.allclose(out, torch.full((1, 2), 1.0 / (1.0 + math.e), dtype=torch.float64))
