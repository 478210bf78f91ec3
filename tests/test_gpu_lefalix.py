"""Lefalix on the GPU against the plain restatement in ``lefalix_oracle.py``: every mechanism alone, then whole models of several
shapes through prefill, decoding, portions, ragged batches, reused slots and the generation entry points."""
from __future__ import annotations

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import lefalix_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def K():
    from lit_gpt_b200 import kernels

    return kernels


# ---------------------------------------------------------------------------------------------------------
# configurations and random checkpoints
# ---------------------------------------------------------------------------------------------------------
def delta(heads, kv_heads, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


def window(heads, kv_heads, dim, vdim, conv, size, rot_dims, base=100.0, scaling=None, scale=None):
    rot = dict(base=base, dims=rot_dims)
    if scaling is not None:
        rot["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, mask=dict(size=size), rot=rot,
                scale=scale if scale is not None else dim ** -0.5)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, groups=None, keep=None):
    router = dict(experts=experts, top=top)
    if groups is not None:
        router["groups"] = dict(count=groups, keep=keep)
    return dict(kind="moe", expert=dict(ff=ff), router=router)


def channel_layer(mixer, mlp):
    return dict(type="channel_delta", mixer=mixer, mlp=mlp)


def parallel_layer(left, right, mlp):
    return dict(type="parallel", mixer=dict(left=left, right=right), mlp=mlp)


def config(width, vocab, layers, loop=None, eps=1e-5):
    cfg = dict(architecture="Lefalix", layers=layers, norm=dict(eps=eps), vocab=vocab, width=width)
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


# odd sizes on purpose: grouped heads on both sides, key size != value size, different taps per mixer (one mixer without a
# convolution), a window shorter than the taps of its neighbour, a layer without feed-forward, a router without groups, the middle
# two layers repeated three times
CFG_ODD = config(width=40, vocab=83, loop=(1, 3, 3), layers=[
    channel_layer(delta(4, 2, 12, 10, 4), dense(50)),
    parallel_layer(window(4, 2, 10, 6, 2, size=7, rot_dims=6, scaling=(3.0, 16, 4.0, 1.0), scale=0.9), delta(3, 3, 8, 12, 3), moe(6, 2, 14, 3, 2)),
    parallel_layer(window(2, 1, 16, 12, 1, size=3, rot_dims=16, base=50.0), delta(2, 1, 6, 6, 2), None),
    channel_layer(delta(1, 1, 20, 9, 1), moe(5, 3, 11)),
])
# heads wider than one warp pass of the recurrence (key size > 64) and than one value chunk of the attention tile (> 128), a
# window of one position, one expert per token, no repeated layers (no "loop" entry at all), rotation of a part of the head
CFG_WIDE = config(width=64, vocab=120, eps=1e-3, layers=[
    parallel_layer(window(2, 2, 72, 136, 3, size=1, rot_dims=20, scaling=(8.0, 32, 16.0, 2.0)), delta(2, 2, 72, 40, 4), dense(96)),
    channel_layer(delta(2, 1, 136, 24, 3), moe(4, 1, 40, 2, 1)),
    parallel_layer(window(3, 1, 24, 24, 4, size=33, rot_dims=24, base=1e4, scale=0.35), delta(4, 2, 16, 16, 3), moe(8, 4, 24, 4, 3)),
])

# head sizes the tensor-core prompt kernel takes in bf16 (64 and 128, grouped), a window that ends inside a key tile, a key size
# that spreads a state column over 32 lanes for prompts and 8 for single tokens, a repeated run that starts at the first layer
CFG_TILES = config(width=96, vocab=140, loop=(0, 2, 2), layers=[
    parallel_layer(window(4, 2, 64, 64, 3, size=40, rot_dims=32, base=1e5, scaling=(4.0, 64, 8.0, 1.0)), delta(2, 1, 64, 32, 3), moe(8, 2, 48, 4, 2)),
    channel_layer(delta(2, 2, 128, 48, 4), dense(200)),
    parallel_layer(window(2, 1, 128, 128, 2, size=100, rot_dims=64, base=1e4, scale=0.2), delta(2, 2, 48, 64, 4), dense(160)),
])


def checkpoint(cfg, seed, sharp=1.0):
    """Random bf16 weights of a size that keeps every mechanism alive; `sharp` multiplies the attention scale's effect by scaling
    the sinks down and is used with configurations whose score scale is large."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    d = cfg["width"]
    w = {"embed": rnd(cfg["vocab"], d), "final.norm": rnd(d, std=0.2, mean=1.0), "head": rnd(cfg["vocab"], d, std=d ** -0.5)}

    def put_delta(p, m, channel):
        H, G, dk, dv, n = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        for name, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
            w[p + name] = rnd(rows, d, std=d ** -0.5)
            w[p + name + ".conv"] = rnd(rows, n, std=0.7)
        w[p + "b"] = rnd(H, d, std=d ** -0.5)
        w[p + "A_log"] = rnd(H, std=0.7)
        w[p + "norm"] = rnd(dv, std=0.2, mean=1.0)
        w[p + "o"] = rnd(d, H * dv, std=(H * dv) ** -0.5)
        if channel:
            ra, rg = 5, 7
            w[p + "a1"], w[p + "a2"] = rnd(ra, d, std=d ** -0.5), rnd(H * dk, ra, std=1.5 * ra ** -0.5)
            w[p + "g1"], w[p + "g2"] = rnd(rg, d, std=d ** -0.5), rnd(H * dv, rg, std=1.5 * rg ** -0.5)
            w[p + "dt_bias"] = rnd(H * dk, std=0.7)
        else:
            w[p + "a"], w[p + "g"] = rnd(H, d, std=1.5 * d ** -0.5), rnd(H * dv, d, std=d ** -0.5)
            w[p + "dt_bias"] = rnd(H, std=0.7)

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        for nm in ("norm1", "norm1b", "norm2", "norm2b"):
            w[p + nm] = rnd(d, std=0.2, mean=1.0)
        if layer["type"] == "parallel":
            m, q = layer["mixer"]["left"], p + "mix.left."
            H, G, dk, dv, n = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for name, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                w[q + name] = rnd(rows, d, std=d ** -0.5)
                w[q + name + ".b"] = rnd(rows, std=0.3)
                w[q + name + ".conv"] = rnd(rows, n, std=0.7)
            w[q + "sink"] = rnd(H, std=1.0, mean=0.5 / sharp)
            w[q + "o"], w[q + "o.b"] = rnd(d, H * dv, std=(H * dv) ** -0.5), rnd(d, std=0.2)
            put_delta(p + "mix.right.", layer["mixer"]["right"], False)
            w[p + "mix.left.out"], w[p + "mix.right.out"] = rnd(d, std=0.2, mean=1.0), rnd(d, std=0.2, mean=1.0)
        else:
            put_delta(p + "mix.", layer["mixer"], True)
        f = layer["mlp"]
        if f is None:
            del w[p + "norm2"], w[p + "norm2b"]
        elif f["kind"] == "dense":
            w[p + "mlp.up"], w[p + "mlp.down"] = rnd(f["ff"], d, std=d ** -0.5), rnd(d, f["ff"], std=f["ff"] ** -0.5)
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            w[p + "mlp.router"] = rnd(E, d, std=2.0 * d ** -0.5)
            for e in range(E):
                w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"] = rnd(ff, d, std=d ** -0.5), rnd(ff, d, std=d ** -0.5)
                w[f"{p}mlp.e{e}.down"] = rnd(d, ff, std=ff ** -0.5)
    return w


def build(cfg, weights, dtype, slots=2):
    from lit_gpt_b200.config import LefalixConfig
    from lit_gpt_b200.lefalix import Lefalix

    config_ = LefalixConfig.from_dict(cfg)
    Lefalix.complete_config(config_, {k: tuple(v.shape) for k, v in weights.items()})
    model = Lefalix(config_).to("cuda").to(dtype)
    model.load_tensors(weights)
    model.set_kv_cache(batch_size=slots)
    return model.eval()


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def rel_err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


TOL = {torch.float32: 3e-5}


def assert_close(got, want, dtype, what=""):
    """fp32: the whole block within rounding.  bf16: a rounding difference ahead of a router can move a token to another expert
    (in exact arithmetic on bf16-rounded inputs just as well), so the typical row and four rows in five must be within bf16
    rounding (these models are a few dozen channels wide, so one moved token is a large share of a row); the fp32 runs of the same tests are the sharp ones."""
    if dtype == torch.float32:
        assert rel_err(got, want) < TOL[dtype], (what, rel_err(got, want))
        return
    got, want = got.double().cpu(), want.double().cpu()
    rows = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-30)
    assert float(rows.median()) < 6e-2 and float((rows < 0.12).double().mean()) >= 0.8, (what, rows)


# ---------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------
def _one_layer(layer, width, dtype, seed, slots=3, sharp=1.0):
    """A one-layer model whose mixer is driven directly with a given input."""
    cfg = config(width=width, vocab=11, layers=[layer])
    w = checkpoint(cfg, seed, sharp)
    return cfg, w, build(cfg, w, dtype, slots=slots)


def _drive(mixer, state, h, cuts, slot, dtype):
    """Feed the rows of h to `mixer` in steps of the given sizes for one sequence in `slot`; returns all output rows."""
    from lit_gpt_b200.ragged import state_batch

    out, at = [], 0
    for n in cuts:
        batch, _ = state_batch([(slot, at, n)], torch.device("cuda"))
        out.append(mixer(h[at : at + n].to(dtype).cuda().contiguous(), batch, state).float().cpu())
        at += n
    assert at == h.shape[0]
    return torch.cat(out)


def _poison(state):
    for t in state.tensors():
        t.fill_(7.0 if t.dtype != torch.float32 else 3.0e3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cuts", [[37], [1] * 37, [2, 2, 3, 1, 17, 2, 8, 2], [36, 1]])
def test_window_attention_alone(dtype, cuts):
    """Projection biases, convolution tail, rotation with blended frequencies, weightless norm, window edge, sink, grouped heads and
    the ring, in prompts, portions down to two tokens and single tokens.  The score scale is large, so the softmax is nearly
    one-hot and a key that is one position off moves the output far beyond rounding."""
    layer = parallel_layer(window(4, 2, 10, 6, 3, size=7, rot_dims=6, scaling=(3.0, 16, 4.0, 1.0), scale=2.5), delta(1, 1, 4, 4, 2), None)
    cfg, w, model = _one_layer(layer, 24, dtype, seed=3, sharp=4.0)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(37, 24, generator=g).to(torch.bfloat16).double()
    W = {k: v.double() for k, v in w.items()}
    want = O.window_attention(h, W, "l0.mix.left.", layer["mixer"]["left"], cfg["norm"]["eps"])
    state = model.states[0].left
    _poison(state)      # a slot that another sequence used: nothing of it may be read
    got = _drive(model.blocks[0].mixer.left, state, h, cuts, slot=1, dtype=dtype)
    assert rel_err(got, want) < (2e-5 if dtype == torch.float32 else 4e-2), rel_err(got, want)


def test_window_edge_is_exact_in_prompt_and_decoding():
    """One key is made loud (its projected row scaled up), queries likewise: a query `size - 1` positions later must still see
    it, the next one must not, in a prompt, in a later portion and in single-token steps, through the tiled and the single-row kernel."""
    k = K()
    H, G, dk, dv, size = 2, 1, 8, 5, 6
    g = torch.Generator().manual_seed(9)
    n = 30
    q = torch.randn(n, H * dk, generator=g)
    kk = torch.randn(n, G * dk, generator=g) * 0.1
    v = torch.randn(n, G * dv, generator=g)
    loud = 11
    kk[loud] = q[loud + size - 1, :dk] * 3.0         # aligned with the query of the last position that may see it
    q[loud + size] = q[loud + size - 1]              # the next query looks for the same key, which has left its window
    sink = torch.tensor([-30.0, -30.0])

    def reference():
        out = torch.zeros(n, H, dv, dtype=torch.float64)
        for i in range(n):
            lo = max(0, i - size + 1)
            for hh in range(H):
                s = kk[lo : i + 1].double() @ q[i, hh * dk : (hh + 1) * dk].double()
                e = torch.exp(s - s.max())
                out[i, hh] = (e / (e.sum() + torch.exp(sink[hh].double() - s.max()))) @ v[lo : i + 1].double()
        return out.reshape(n, H * dv)

    want = reference()
    assert (want[loud + size - 1, :dv] - v[loud].double()).abs().max() < 1e-3      # the loud key owns that row ...
    assert (want[loud + size, :dv] - v[loud].double()).abs().max() > 1e-2          # ... and is gone one position later
    from lit_gpt_b200.ragged import state_batch

    for cuts in ([n], [loud + 2, n - loud - 2], [loud + size - 1, 1, 1, n - loud - size - 1], [1] * n):
        for tiled in (False, True):
            old = k.window_attn_tune(force_tiled_kernel=tiled)
            try:
                k_ring, v_ring = torch.full((2, size, G * dk), 9.0, device="cuda"), torch.full((2, size, G * dv), 9.0, device="cuda")
                got, at = [], 0
                for c in cuts:
                    batch, _ = state_batch([(1, at, c)], torch.device("cuda"))
                    got.append(k.window_attn(q[at : at + c].cuda(), kk[at : at + c].cuda(), v[at : at + c].cuda(), k_ring, v_ring, sink.cuda(),
                                             batch.seq_state, batch.row_seq, c, H, G, dk, dv, size, 1.0).cpu())
                    at += c
            finally:
                k.window_attn_tune(force_tiled_kernel=old)
            assert rel_err(torch.cat(got), want) < 1e-5, (cuts, tiled)


def _windowed_softmax(q, kk, v, sink, H, G, dk, dv, size, scale):
    """float64 attention of one sequence from position 0: q (n, H dk), kk (n, G dk), v (n, G dv)."""
    n = q.shape[0]
    q, kk, v = q.double().view(n, H, dk), kk.double().view(n, G, dk), v.double().view(n, G, dv)
    out = torch.zeros(n, H, dv, dtype=torch.float64)
    for i in range(n):
        lo = max(0, i - size + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (kk[lo : i + 1, g] @ q[i, hh]) * scale
            e = torch.exp(s - s.max())
            out[i, hh] = (e / (e.sum() + torch.exp(sink[hh].double() - s.max()))) @ v[lo : i + 1, g]
    return out.reshape(n, H * dv)


@pytest.mark.parametrize("hs,size", [(64, 100), (64, 64), (128, 1), (128, 150), (64, 1000)])
def test_window_prefill_on_the_tensor_cores(hs, size):
    """bf16 prompts with 64- / 128-wide heads take the tensor-core tiles: windows that end inside a key tile, at its edge, of one
    position and longer than the prompt; grouped heads; three sequences of unequal length in one launch (one shorter than a
    query tile, one spanning several).  Compared with exact attention on the same bf16 operands and with the any-size kernel."""
    k = K()
    from lit_gpt_b200.ragged import state_batch

    H, G = 4, 2
    g = torch.Generator().manual_seed(hs + size)
    lens = [200, 37, 300]
    n = sum(lens)
    q = torch.randn(n, H * hs, generator=g).to(torch.bfloat16)
    kk = torch.randn(n, G * hs, generator=g).to(torch.bfloat16)
    v = torch.randn(n, G * hs, generator=g).to(torch.bfloat16)
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0]).to(torch.bfloat16)
    scale = 2.0 * hs ** -0.5           # sharp: the few largest scores carry the row
    want, at = [], 0
    for ln in lens:
        want.append(_windowed_softmax(q[at : at + ln], kk[at : at + ln], v[at : at + ln], sink.float(), H, G, hs, hs, size, scale))
        at += ln
    want = torch.cat(want)
    batch, _ = state_batch([(0, 0, lens[0]), (2, 0, lens[1]), (1, 0, lens[2])], torch.device("cuda"))
    assert batch.identity_ctx
    ring = min(size, 400)
    outs = {}
    for mma in (True, False):
        k.WINDOW_PREFILL_MMA = mma
        try:
            k_ring, v_ring = torch.zeros(3, ring, G * hs, dtype=torch.bfloat16, device="cuda"), torch.zeros(3, ring, G * hs, dtype=torch.bfloat16, device="cuda")
            launches = k.launch_count()
            outs[mma] = k.window_attn(q.cuda(), kk.cuda(), v.cuda(), k_ring, v_ring, sink.cuda(), batch.seq_state, batch.row_seq, max(lens), H, G, hs, hs,
                                      min(size, ring), scale, from_start=True).float().cpu()
            assert k.launch_count() - launches == 2
        finally:
            k.WINDOW_PREFILL_MMA = True
        # the rings hold every sequence's last positions whichever kernel ran
        last = lens[2] - 1
        assert torch.equal(k_ring[1, last % ring].cpu(), kk[lens[0] + lens[1] + last]) and torch.equal(v_ring[2, (lens[1] - 1) % ring].cpu(), v[lens[0] + lens[1] - 1])
    assert rel_err(outs[False], want) < 6e-3 and rel_err(outs[True], want) < 1.2e-2, (rel_err(outs[False], want), rel_err(outs[True], want))


def test_sink_takes_probability_once_and_unscaled():
    k = K()
    from lit_gpt_b200.ragged import state_batch

    H, dk, dv = 3, 4, 4
    q = torch.zeros(1, H * dk)
    kk, v = torch.zeros(1, H * dk), torch.ones(1, H * dv)
    sink = torch.tensor([0.0, 2.0, -2.0])
    batch, _ = state_batch([(0, 0, 1)], torch.device("cuda"))
    ring = torch.zeros(1, 4, H * dk, device="cuda")
    for scale in (1.0, 17.0):    # the score is 0 whatever the scale: the only key weighs 1 / (1 + e^sink)
        out = k.window_attn(q.cuda(), kk.cuda(), v.cuda(), ring, ring.clone(), sink.cuda(), batch.seq_state, batch.row_seq, 1, H, H, dk, dv, 4, scale)
        assert torch.allclose(out.cpu().view(H, dv)[:, 0], 1.0 / (1.0 + torch.exp(sink)), atol=1e-6)
    out = k.window_attn(q.cuda(), kk.cuda(), v.cuda(), ring, ring.clone(), None, batch.seq_state, batch.row_seq, 1, H, H, dk, dv, 4, 1.0)
    assert torch.allclose(out.cpu(), torch.ones(1, H * dv), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channel", [False, True])
@pytest.mark.parametrize("cuts,dim,taps", [([41], 12, 4), ([1] * 41, 12, 4), ([2, 2, 1, 20, 2, 3, 9, 2], 12, 4), ([40, 1], 12, 4), ([30, 1, 10], 40, 4),
                                           ([3, 37, 1], 72, 4), ([2, 3, 1, 1, 30, 4], 12, 7), ([41], 12, 9)])
def test_delta_rule_alone(dtype, channel, cuts, dim, taps):
    """Grouped heads, convolution tail with its activation, unit vectors, decay per head or per channel, write-then-read order,
    gated norm -- with the state carried over every cut (prompts and single tokens spread a state column over different numbers
    of lanes for the larger key sizes: both read the same stored state)."""
    m = delta(4, 2, dim, 10, taps)      # more taps than the unrolled cases, and portions shorter than the taps
    layer = channel_layer(m, None) if channel else parallel_layer(window(1, 1, 4, 4, 1, size=2, rot_dims=4), m, None)
    cfg, w, model = _one_layer(layer, 24, dtype, seed=13)
    g = torch.Generator().manual_seed(15)
    h = torch.randn(41, 24, generator=g).to(torch.bfloat16).double()
    W = {k: v.double() for k, v in w.items()}
    want = O.delta_mixer(h, W, "l0.mix." if channel else "l0.mix.right.", m, cfg["norm"]["eps"], channel)
    mixer = model.blocks[0].mixer if channel else model.blocks[0].mixer.right
    state = model.states[0] if channel else model.states[0].right
    _poison(state)
    got = _drive(mixer, state, h, cuts, slot=2, dtype=dtype)
    assert rel_err(got, want) < (2e-5 if dtype == torch.float32 else 4e-2), rel_err(got, want)


def test_delta_rule_remembers_a_far_write():
    """With decay ~ 1 and orthogonal keys a value written at the first position is read back exactly 300 positions later; with a
    strong decay on one head it is gone.  Kernel alone, prompt then single steps."""
    k = K()
    from lit_gpt_b200.ragged import state_batch

    H, dk, dv, n = 2, 16, 6, 301
    kk = torch.zeros(n, dk)
    kk[0, 3] = 1.0
    for t in range(1, n - 1):
        kk[t, 4 + t % 12] = 1.0          # later writes never touch channel 3
    q = torch.zeros(n, dk)
    q[n - 1, 3] = 1.0
    v = torch.zeros(n, H * dv)
    v[0] = torch.arange(1, H * dv + 1).float()
    beta_in = torch.full((n, H), 30.0)                    # sigmoid -> 1
    decay_in = torch.stack([torch.full((n,), -40.0), torch.full((n,), 2.0)], dim=1)    # head 0 keeps everything, head 1 forgets
    a_log, dt_bias = torch.zeros(H), torch.zeros(H)
    state = torch.full((2, H * k.delta_rule_state_floats(dk, dv)), 5.0, device="cuda")
    outs = []
    for at, c in ((0, 200), (200, 100), (300, 1)):
        batch, _ = state_batch([(1, at, c)], torch.device("cuda"))
        s = slice(at, at + c)
        outs.append(k.delta_rule(q[s].cuda(), kk[s].cuda(), v[s].cuda(), beta_in[s].cuda(), decay_in[s].cuda(), a_log.cuda(), dt_bias.cuda(), state,
                                 batch.seq_state, H, 1, dk, dv, False, max_rows=c).cpu())
    last = outs[-1][0]
    assert torch.allclose(last[:dv], v[0, :dv], rtol=1e-5) and float(last[dv:].abs().max()) < 1e-6


@pytest.mark.parametrize("experts,top,groups,keep", [(18, 5, 2, 1), (12, 4, 4, 2), (6, 1, 1, 1), (8, 2, 8, 3), (9, 3, 3, 3), (8, 4, 4, 3)])
def test_softmax_router(experts, top, groups, keep):
    k = K()
    g = torch.Generator().manual_seed(experts * 100 + top)
    n, d = 40, 52
    x = torch.randn(n, d, generator=g)
    w = {"r.router": torch.randn(experts, d, generator=g) * 0.3}
    ids, wts = k.moe_route(x.cuda(), w["r.router"].cuda(), None, top, groups, keep, softmax=True, group_max=True)
    want_ids, want_w = O.route(x.double(), {"r.router": w["r.router"].double()}, "r.", dict(experts=experts, top=top, groups=dict(count=groups, keep=keep)))
    assert torch.equal(ids.cpu().long(), want_ids)
    assert rel_err(wts, want_w) < 1e-6
    assert float(wts.sum(dim=-1).max()) <= 1.0 + 1e-6      # scores of a softmax over ALL experts, not renormalised over the chosen


def test_group_rank_is_the_largest_score_not_a_sum():
    k = K()
    # group 0 holds the single best expert, group 1 two good ones whose sum is larger: with keep = 1 group 0 wins
    z = torch.tensor([[4.0, -9.0, 3.5, 3.4]])
    x = torch.eye(4)[:1] * 0 + torch.tensor([[1.0, 0.0, 0.0, 0.0]])
    wr = z.t().contiguous() @ torch.tensor([[1.0, 0.0, 0.0, 0.0]])     # logits = z for this x
    ids, _ = k.moe_route(x.cuda(), wr.cuda(), None, 1, 2, 1, softmax=True, group_max=True)
    assert ids.cpu().tolist() == [[0]]
    ids, _ = k.moe_route(x.cuda(), wr.cuda(), None, 2, 2, 1, softmax=True, group_max=True)
    assert ids.cpu().tolist() == [[0, 1]]                                # the second choice stays inside the kept group


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 5, 150])   # GEMV path (few pairs) and grouped path, with experts that get no token
def test_gated_experts(dtype, n):
    from lit_gpt_b200.config import GatedMoESpec
    from lit_gpt_b200.moe import GatedSparseExperts

    d, E, ff = 40, 6, 14
    f = moe(E, 2, ff, 3, 2)
    g = torch.Generator().manual_seed(n)
    w = {"m.router": (torch.randn(E, d, generator=g) * 0.5).to(torch.bfloat16)}
    for e in range(E):
        for nm, shape in (("gate", (ff, d)), ("up", (ff, d)), ("down", (d, ff))):
            w[f"m.e{e}.{nm}"] = (torch.randn(*shape, generator=g) * shape[1] ** -0.5).to(torch.bfloat16)
    mod = GatedSparseExperts(d, GatedMoESpec(E, 2, ff, 3, 2)).to("cuda").to(dtype)
    mod.router.weight.data.copy_(w["m.router"])
    mod.w_up.data.copy_(torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(E)]))
    mod.w_down.data.copy_(torch.stack([w[f"m.e{e}.down"] for e in range(E)]))
    x = torch.randn(n, d, generator=g).to(torch.bfloat16)
    want = O.feed_forward(x.double(), {k_: v.double() for k_, v in w.items()}, "m.", f)
    got = mod(x.to(dtype).cuda())
    assert rel_err(got, want) < (2e-5 if dtype == torch.float32 else 3e-2), rel_err(got, want)


def test_gated_experts_vendor_grouped_path_agrees_with_own_kernels():
    import lit_gpt_b200.moe as M
    from lit_gpt_b200.config import GatedMoESpec

    d, E, ff, n = 64, 8, 48, 300
    mod = M.GatedSparseExperts(d, GatedMoESpec(E, 3, ff, 4, 2)).to("cuda").to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(4)
    for p in mod.parameters():
        p.data.copy_(torch.randn(p.shape, generator=g, device="cuda") * 0.15)
    x = torch.randn(n, d, generator=g, device="cuda").to(torch.bfloat16)
    a = mod(x)
    M.VENDOR_GROUPED_GEMM = False
    try:
        b = mod(x)
    finally:
        M.VENDOR_GROUPED_GEMM = True
    assert rel_err(a, b) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [40, 70, 1024])
def test_sandwich_residual_and_activations(dtype, d):
    k = K()
    g = torch.Generator().manual_seed(d)
    n, eps = 9, 1e-3
    x = torch.randn(n, d, generator=g)
    y0, y1 = (torch.randn(n, d, generator=g) * 4).to(dtype), (torch.randn(n, d, generator=g) * 0.2).to(dtype)
    w0, w1, post, pre = [(1 + 0.3 * torch.randn(d, generator=g)).to(dtype) for _ in range(4)]
    tol = 1e-6 if dtype == torch.float32 else 6e-3
    # two branches joined, post-norm, residual sum, next pre-norm
    xs, act = x.clone().cuda(), torch.empty(n, d, dtype=dtype, device="cuda")
    k.sandwich_residual(xs, y0.cuda(), post.cuda(), eps, w0=w0.cuda(), y1=y1.cuda(), w1=w1.cuda(), pre_w=pre.cuda(), act=act)
    y = 0.5 * (O.norm(y0.double(), w0.double(), eps) + O.norm(y1.double(), w1.double(), eps))
    want = x.double() + O.norm(y, post.double(), eps)
    assert rel_err(xs, want) < 1e-6 and xs.dtype == torch.float32
    assert rel_err(act, O.norm(want, pre.double(), eps)) < tol
    # one branch, no following norm; then a plain addition with a pre-norm (the embedding re-entering)
    xs = x.clone().cuda()
    k.sandwich_residual(xs, y0.cuda(), post.cuda(), eps)
    assert rel_err(xs, x.double() + O.norm(y0.double(), post.double(), eps)) < 1e-6
    xs = x.clone().cuda()
    k.sandwich_residual(xs, y1.cuda(), None, eps, pre_w=pre.cuda(), act=act)
    assert rel_err(xs, x.double() + y1.double()) < 1e-6 and rel_err(act, O.norm(x.double() + y1.double(), pre.double(), eps)) < tol
    # activations
    z = (torch.randn(n, d, generator=g) * 3).to(dtype)
    assert rel_err(k.activation_(z.clone().cuda(), k.ACT_GELU), torch.nn.functional.gelu(z.double())) < tol
    assert rel_err(k.activation_(z.clone().cuda(), k.ACT_GELU_TANH), torch.nn.functional.gelu(z.double(), approximate="tanh")) < tol
    zz = torch.cat([z, y0], dim=1).contiguous()
    assert rel_err(k.glu(zz.cuda(), k.ACT_SILU), torch.nn.functional.silu(z.double()) * y0.double()) < tol


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cfg,seed", [(CFG_ODD, 11), (CFG_WIDE, 12), (CFG_TILES, 13)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_matches_oracle(cfg, seed, dtype):
    w = checkpoint(cfg, seed)
    model = build(cfg, w, dtype)
    toks = tokens_for(cfg, 150 if cfg is CFG_TILES else 90, seed)
    got = model.step(toks, [(1, 0, len(toks))])
    assert got.dtype == torch.float32
    assert_close(got, O.forward(cfg, w, toks), dtype)


def test_layers_follow_the_oracle_one_by_one():
    cfg = CFG_ODD
    w = checkpoint(cfg, 21)
    model = build(cfg, w, torch.float32)
    toks = tokens_for(cfg, 19, 21)
    model.trace = []
    model.step(toks, [(0, 0, len(toks))])
    seen, model.trace = model.trace, None
    _, layers = O.forward(cfg, w, toks, return_layers=True)
    assert len(seen) == len(layers) == 1 + 2 * 3 + 1          # the two repeated layers count every time
    for i, x in enumerate(seen):
        assert rel_err(x, layers[i]) < 1e-5, f"residual stream after layer run {i}"


@pytest.mark.parametrize("cfg", [CFG_ODD, CFG_WIDE, CFG_TILES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decoding_token_by_token_equals_prefill(dtype, cfg):
    w = checkpoint(cfg, 31)
    model = build(cfg, w, dtype)
    toks = tokens_for(cfg, 60, 31)
    whole = model.step(toks, [(0, 0, len(toks))])
    rows = [model.step([t], [(1, p, 1)]) for p, t in enumerate(toks)]      # the very first token too is a decode step
    assert_close(torch.cat(rows), whole, dtype)
    assert_close(torch.cat(rows), O.forward(cfg, w, toks), dtype)


@pytest.mark.parametrize("portions", [[2, 2, 2, 30, 3, 34, 1, 35, 2], [109, 2], [1, 110], [5] * 22 + [1]])
@pytest.mark.parametrize("cfg", [CFG_ODD, CFG_WIDE])
def test_prompt_in_portions(portions, cfg):
    """Portions shorter than the convolutions' taps and than the windows, and portions that span several windows."""
    w = checkpoint(cfg, 41)
    model = build(cfg, w, torch.float32)
    toks = tokens_for(cfg, sum(portions), 41)
    whole = model.step(toks, [(0, 0, len(toks))])
    got, at = [], 0
    for n in portions:
        got.append(model.step(toks[at : at + n], [(1, at, n)]))
        at += n
    assert rel_err(torch.cat(got), whole) < 2e-5
    assert rel_err(whole, O.forward(cfg, w, toks)) < 3e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_batch_equals_each_alone(dtype):
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_ODD
    w = checkpoint(cfg, 51)
    model = build(cfg, w, dtype)
    session = Session(model, slots=2)     # grows to 4 when the third request arrives
    lens = {"a": 1, "b": 67, "c": 100, "d": 9}
    prompts = {r: tokens_for(cfg, n + 12, 60 + i) for i, (r, n) in enumerate(lens.items())}
    alone = {r: O.forward(cfg, w, t) for r, t in prompts.items()}
    out = session.step([(r, prompts[r][: lens[r]], None) for r in lens])
    at = 0
    for r in lens:
        assert_close(out[at : at + lens[r]], alone[r][: lens[r]], dtype, r)
        at += lens[r]
    decoded = {r: [] for r in lens}
    live = list(lens)
    for stepno in range(12):
        ending = ["a"] if stepno == 3 else (["c"] if stepno == 7 else [])    # shorter requests leave the batch
        out = session.step([(r, [prompts[r][lens[r] + stepno]], [0]) for r in live], end=ending)
        for j, r in enumerate(live):
            decoded[r].append(out[j : j + 1])
        live = [r for r in live if r not in ending]
    for r, rows in decoded.items():
        assert_close(torch.cat(rows), alone[r][lens[r] : lens[r] + len(rows)], dtype, r)
    assert model.slots.capacity == 4 and model.slots.in_use == 2


def test_growing_the_session_keeps_live_states():
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_ODD
    w = checkpoint(cfg, 55)
    model = build(cfg, w, torch.float32, slots=1)
    session = Session(model, slots=1)
    a, b = tokens_for(cfg, 40, 56), tokens_for(cfg, 30, 57)
    session.step([("a", a[:25], [])])
    session.step([("b", b[:20], [])])                    # no free slot: the states move to a larger allocation
    out = session.step([("a", a[25:], None), ("b", b[20:], None)])
    assert rel_err(out[:15], O.forward(cfg, w, a)[25:]) < 3e-5 and rel_err(out[15:], O.forward(cfg, w, b)[20:]) < 3e-5


def test_freed_slots_are_reused_without_leftovers():
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_ODD
    w = checkpoint(cfg, 71)
    model = build(cfg, w, torch.float32)
    session = Session(model, slots=2)
    long, short = tokens_for(cfg, 90, 72), tokens_for(cfg, 20, 73)
    session.step([("x", long, [0]), ("y", short, [0])], end=["x"])
    assert model.slots.in_use == 1
    # the new request takes x's slot, which still holds x's rings, tails and state matrices; it must see only its own
    fresh = tokens_for(cfg, 33, 74)
    want = O.forward(cfg, w, fresh)
    out = session.step([("z", fresh[:2], None)])          # fewer tokens than any convolution has taps
    assert session.live["z"][0] == 0
    assert rel_err(out, want[:2]) < 3e-5
    out = session.step([("z", fresh[2:30], None)])
    assert rel_err(out, want[2:30]) < 3e-5
    for p in range(30, 33):
        out = session.step([("z", [fresh[p]], [0]), ("y", [short[0]], [])])
        assert rel_err(out, want[p : p + 1]) < 3e-5


def test_long_decoding_wraps_the_rings_many_times():
    """250 single-token steps after a short prompt: every ring position is overwritten dozens of times and the fp32 states run
    through hundreds of updates; compared with the oracle's recomputation of the whole sequence."""
    cfg = CFG_ODD
    w = checkpoint(cfg, 81)
    model = build(cfg, w, torch.float32)
    toks = tokens_for(cfg, 260, 81)
    want = O.forward(cfg, w, toks)
    got = [model.step(toks[:10], [(1, 0, 10)])]
    got += [model.step([toks[p]], [(1, p, 1)]) for p in range(10, 260)]
    assert rel_err(torch.cat(got), want) < 5e-5
    assert rel_err(got[-1], want[-1:]) < 5e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_generate_entry_points(dtype):
    """Greedy generation through generate() (captured decode graph) and through the batch scheduler give the oracle's tokens."""
    from lit_gpt_b200.generate.base import generate
    from lit_gpt_b200.generate.serve import generate_batch

    cfg = CFG_ODD
    w = checkpoint(cfg, 91)
    prompt = tokens_for(cfg, 9, 91)
    seq = list(prompt)
    for _ in range(14):   # the oracle's own greedy continuation (recomputing the whole sequence every time)
        seq.append(int(O.forward(cfg, w, seq)[-1].argmax()))
    model = build(cfg, w, dtype, slots=1)
    model.max_seq_length = 64
    y = generate(model, torch.tensor(prompt, device="cuda"), len(seq), temperature=0.0)
    if dtype == torch.float32:
        assert y.tolist() == seq
    other = tokens_for(cfg, 4, 92)
    model.set_kv_cache(batch_size=2)
    ys = generate_batch(model, [prompt, other], 14)
    assert ys[0] == y.tolist() and len(ys[1]) == 4 + 14 and model.slots.in_use == 0
    seq2 = list(other)
    for _ in range(14):
        seq2.append(int(O.forward(cfg, w, seq2)[-1].argmax()))
    if dtype == torch.float32:
        assert ys[1] == seq2


def test_forward_signature_of_the_other_models():
    """forward(idx, input_pos) with batch rows = slots and shared positions, as GPT.forward: a prompt, then single tokens."""
    cfg = CFG_WIDE
    w = checkpoint(cfg, 95)
    model = build(cfg, w, torch.float32, slots=2)
    a, b = tokens_for(cfg, 12, 96), tokens_for(cfg, 12, 97)
    idx = torch.tensor([a, b], device="cuda")
    out = model(idx[:, :10], torch.arange(10, device="cuda"))
    for p in (10, 11):
        out = torch.cat([out, model(idx[:, p : p + 1], torch.tensor([p], device="cuda"))], dim=1)
    assert out.shape == (2, 12, cfg["vocab"])
    assert rel_err(out[0], O.forward(cfg, w, a)) < 3e-5 and rel_err(out[1], O.forward(cfg, w, b)) < 3e-5


def _write_checkpoint(folder, cfg, weights):
    import json
    import struct

    header, blob = {}, b""
    for name, t in weights.items():
        raw = t.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    hj = json.dumps(header).encode()
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob)
    (folder / "config.json").write_text(json.dumps(cfg))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_end_to_end(tmp_path, dtype):
    """The command-line replayer on a checkpoint directory written here: a ragged first step, decoding together, a request that
    ends, a new one in its slot, steps without anything wanted -- the files it writes against the oracle."""
    import json
    import subprocess

    import numpy as np

    cfg = CFG_ODD
    w = checkpoint(cfg, 101)
    _write_checkpoint(tmp_path, cfg, w)
    a, b, c = tokens_for(cfg, 40, 102), tokens_for(cfg, 9, 103), tokens_for(cfg, 70, 104)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:37], "want": [0, 36]}, {"id": "b", "tokens": b[:6], "want": [5]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [a[37]], "want": []}, {"id": "b", "tokens": [b[6]], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": [a[38]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": [a[39]], "want": [0]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": c, "want": [0, 1, 63, 64, 69]}], "end": ["c"]},
    ]
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", dtype, "--out", str(out), "--max-tokens", "120"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
    assert sorted(os.listdir(out)) == ["0.f32", "2.f32", "3.f32", "4.f32"]        # step 1 wanted nothing
    full = {k: O.forward(cfg, w, t) for k, t in (("a", a), ("b", b), ("c", c))}
    want = {0: torch.stack([full["a"][0], full["a"][36], full["b"][5]]), 2: torch.stack([full["a"][38], full["b"][7]]),
            3: full["a"][39:40], 4: full["c"][[0, 1, 63, 64, 69]]}
    for step, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        assert got.shape == ref.shape
        if dtype == "float32":
            assert rel_err(got, ref) < 3e-5, f"step {step}"
    if dtype == "bfloat16":
        got = torch.cat([torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, cfg["vocab"])) for step in want])
        assert_close(got, torch.cat(list(want.values())), torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompts_on_the_tensor_cores_then_decoding_over_their_rings(dtype):
    """Two unequal prompts in one step (bf16: the tensor-core tiles for both attention layers), each longer than one window and
    shorter than the other, then 45 single-token steps that slide both windows over the prompt's ring rows, and a third request
    that arrives in portions while the others decode."""
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_TILES
    w = checkpoint(cfg, 61)
    model = build(cfg, w, dtype)
    session = Session(model, slots=2)
    a, b, c = tokens_for(cfg, 115, 62), tokens_for(cfg, 95, 63), tokens_for(cfg, 60, 64)
    want = {r: O.forward(cfg, w, t) for r, t in (("a", a), ("b", b), ("c", c))}
    out = session.step([("a", a[:70], [0, 39, 40, 69]), ("b", b[:50], [49])])
    assert_close(out, torch.cat([want["a"][[0, 39, 40, 69]], want["b"][49:50]]), dtype, "prompts")
    got = {"a": [], "b": [], "c": []}
    for i in range(45):
        entries = [("a", [a[70 + i]], [0]), ("b", [b[50 + i]], [0])]
        if i % 15 == 5:                       # c's portions of 20 tokens ride along with the single-token steps
            j = (i // 15) * 20
            entries.append(("c", c[j : j + 20], None))
        out = session.step(entries)
        got["a"].append(out[0:1]); got["b"].append(out[1:2])
        if len(entries) == 3:
            got["c"].append(out[2:])
    assert_close(torch.cat(got["a"]), want["a"][70:115], dtype, "a")
    assert_close(torch.cat(got["b"]), want["b"][50:95], dtype, "b")
    assert_close(torch.cat(got["c"]), want["c"], dtype, "c")
