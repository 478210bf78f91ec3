"""Host-side parts of the Pomipel integration: configuration reader and registry, slot allocator, safetensors reader, the
session's bookkeeping (against a stand-in model) and the plain restatement's own consistency."""
from __future__ import annotations

import json
import os
import struct
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import pomipel_oracle as O  # noqa: E402
from test_gpu_pomipel import CFG_ODD, checkpoint, tokens_for  # noqa: E402

from lit_gpt_b200.config import Config, PomipelConfig, load_config, model_class  # noqa: E402


def test_config_reader_and_registry(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG_ODD))
    cfg = load_config(tmp_path)
    assert isinstance(cfg, PomipelConfig) and cfg.n_layer == 5 and cfg.n_embd == 72 and cfg.block_size == 640
    assert cfg.layers[1].mixer.kv_from == 0 and cfg.layers[1].mlp is None and cfg.layers[1].mixer.scale == 0.3
    assert cfg.layers[3].mlp.groups == 4 and cfg.layers[3].mlp.keep == 2 and cfg.layers[3].mlp.top == 4
    assert cfg.embedding_scale == 3.0 and cfg.logit_scale == 0.7
    assert model_class(cfg).__name__ == "Pomipel" and model_class(Config.from_name("pythia-14m")).__name__ == "GPT"
    bad = json.loads(json.dumps(CFG_ODD))
    bad["architecture"] = "Nonesuch"
    (tmp_path / "config.json").write_text(json.dumps(bad))
    with pytest.raises(ValueError, match="unknown architecture"):
        load_config(tmp_path)


@pytest.mark.parametrize("edit,msg", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=1), "earlier layer"),          # layer 1 borrows its latents itself
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=40), "kv_rank differs"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "do not fit"),
    (lambda c: c["layers"][0].update(type="convolution"), "unknown mixer"),
])
def test_config_validation(edit, msg):
    cfg = json.loads(json.dumps(CFG_ODD))
    edit(cfg)
    with pytest.raises(ValueError, match=msg):
        PomipelConfig.from_dict(cfg)


def test_slot_allocator():
    from lit_gpt_b200.pomipel import SlotAllocator

    a = SlotAllocator(3)
    assert [a.acquire(), a.acquire(), a.acquire()] == [0, 1, 2] and a.in_use == 3
    with pytest.raises(RuntimeError):
        a.acquire()
    a.release(1)
    a.release(0)
    assert a.acquire() == 0 and a.in_use == 2
    with pytest.raises(ValueError):
        a.release(1)


def test_safetensors_reader(tmp_path):
    from lit_gpt_b200.checkpoint import read_safetensors

    a = torch.randn(3, 5).to(torch.bfloat16)
    b = torch.arange(7, dtype=torch.int32)
    blob = a.view(torch.int16).numpy().tobytes() + b.numpy().tobytes()
    header = json.dumps({"__metadata__": {"k": "v"}, "a.b": {"dtype": "BF16", "shape": [3, 5], "data_offsets": [0, 30]},
                         "t": {"dtype": "I32", "shape": [7], "data_offsets": [30, 58]}}).encode()
    path = tmp_path / "m.safetensors"
    path.write_bytes(struct.pack("<Q", len(header)) + header + blob)
    got = read_safetensors(path)
    assert set(got) == {"a.b", "t"} and torch.equal(got["a.b"], a) and torch.equal(got["t"], b)
    path.write_bytes(struct.pack("<Q", len(header)) + header + blob[:-4])
    with pytest.raises(Exception, match="inconsistent"):
        read_safetensors(path)


def test_weights_fill_every_parameter_and_reject_strays():
    from lit_gpt_b200.pomipel import Pomipel

    w = checkpoint(CFG_ODD, 3)
    model = Pomipel(PomipelConfig.from_dict(CFG_ODD))
    for p in model.parameters():
        p.data.fill_(float("nan"))
    model.load_tensors(w)
    assert all(torch.isfinite(p).all() for p in model.parameters())
    mx = model.blocks[0].mixer
    assert torch.equal(mx.w_down[:18], w["l0.mix.dq"].float()) and torch.equal(mx.w_down[18:], w["l0.mix.dkv"].float())
    assert torch.equal(mx.w_uv, w["l0.mix.uv"].float()) and model.blocks[1].mixer.source is mx and model.blocks[1].mixer.kv_norm is None
    assert torch.equal(model.blocks[3].mlp.w_down[5], w["l3.mlp.e5.down"].float())
    with pytest.raises(KeyError, match="unexpected"):
        model.load_tensors(dict(w, **{"l1.mix.dkv": w["l0.mix.dkv"]}))
    del w["l2.mlp.e0.up"]
    with pytest.raises(KeyError, match="l2.mlp.e0.up"):
        model.load_tensors(w)


def test_session_bookkeeping_with_a_stand_in_model():
    from lit_gpt_b200.generate.serve import Session
    from lit_gpt_b200.pomipel import SlotAllocator

    calls = []

    class Fake:
        max_seq_length = 50
        marks = None

        def set_kv_cache(self, batch_size):
            self.slots = SlotAllocator(batch_size)
            self.marks = torch.zeros(batch_size, 2)

        def state_tensors(self):
            return [self.marks]

        def step(self, tokens, seqs, want):
            calls.append((list(tokens), list(seqs), list(want)))
            return torch.zeros(len(want), 4)

    s = Session(Fake(), slots=1)
    s.model.marks[0] = 5.0
    out = s.step([("a", [1, 2, 3], [2]), ("b", [4], [])])          # b forces the cache to grow: what slot 0 held moves along
    assert s.model.marks.tolist() == [[5.0, 5.0], [0.0, 0.0]]
    assert out.shape == (1, 4) and calls[-1] == ([1, 2, 3, 4], [(0, 0, 3), (1, 0, 1)], [2])
    assert s.step([("a", [5], []), ("b", [6], [])], end=["a"]) is None      # nothing wanted: nothing returned, the step still runs
    assert calls[-1][1] == [(0, 3, 1), (1, 1, 1)]
    s.step([("c", [7, 8], None)])                                           # a's slot again; None asks for every row
    assert calls[-1] == ([7, 8], [(0, 0, 2)], [0, 1]) and s.model.slots.in_use == 2


def test_oracle_bf16_stays_near_its_own_fp64():
    w = checkpoint(CFG_ODD, 7)
    toks = tokens_for(CFG_ODD, 24, 7)
    hi = O.forward(CFG_ODD, w, toks, torch.float64)
    assert float((O.forward(CFG_ODD, w, toks, torch.float32).double() - hi).norm() / hi.norm()) < 1e-5
    assert float((O.forward(CFG_ODD, w, toks, torch.bfloat16).double() - hi).norm() / hi.norm()) < 6e-2
