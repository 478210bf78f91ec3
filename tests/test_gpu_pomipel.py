"""Pomipel on the GPU against the plain restatement in ``pomipel_oracle.py``: every mechanism alone, then whole models of several
shapes through prefill, decoding, portions, ragged batches, reused slots and the generation entry points."""
from __future__ import annotations

import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import pomipel_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def K():
    from lit_gpt_b200 import kernels

    return kernels


# ---------------------------------------------------------------------------------------------------------
# configurations and random checkpoints
# ---------------------------------------------------------------------------------------------------------
def mixer(heads, dim, vdim, kv_rank, q_rank, scale=None, kv_from=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale if scale is not None else dim ** -0.5)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, groups, keep):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, groups=dict(count=groups, keep=keep)))


def config(width, vocab, layers, max_positions=640, emb_scale=3.0, logit_scale=0.7, eps=1e-5):
    return dict(architecture="Pomipel", embedding=dict(scale=emb_scale), layers=[dict(type="latent_attention", mixer=m, mlp=f) for m, f in layers],
                logit_scale=logit_scale, max_positions=max_positions, norm=dict(eps=eps), vocab=vocab, width=width)


# odd sizes on purpose: nothing a multiple of 8, value size != key size, ranks differ, two owners of latents, a layer without
# feed-forward, one expert per token in one layer and several kept groups in another
CFG_ODD = config(width=72, vocab=150, layers=[
    (mixer(3, 20, 12, 28, 18), moe(6, 2, 36, 3, 2)),
    (mixer(5, 12, 20, 28, 22, scale=0.3, kv_from=0), None),
    (mixer(2, 36, 28, 44, 30), moe(8, 1, 20, 1, 1)),
    (mixer(4, 16, 16, 44, 26, kv_from=2), moe(12, 4, 24, 4, 2)),
    (mixer(1, 40, 24, 28, 20, kv_from=0), moe(4, 3, 30, 2, 2)),
])
# round sizes with a wide value head (two column chunks in the prefill kernel) and a big latent
CFG_WIDE = config(width=128, vocab=200, layers=[
    (mixer(2, 64, 160, 192, 48), moe(8, 2, 64, 2, 1)),
    (mixer(4, 32, 32, 192, 64, kv_from=0), moe(8, 3, 48, 4, 3)),
], max_positions=1100)


# nothing divisible by four, not even the width: every kernel on its element-by-element path, odd leading dimensions in the GEMMs
CFG_RAGGED_SIZES = config(width=70, vocab=97, layers=[
    (mixer(2, 10, 6, 14, 9), moe(5, 2, 11, 1, 1)),
    (mixer(3, 6, 10, 14, 7, scale=0.5, kv_from=0), moe(6, 3, 9, 3, 2)),
    (mixer(1, 7, 7, 22, 5), None),
], max_positions=130, emb_scale=1.7, logit_scale=1.3, eps=1e-3)


def checkpoint(cfg, seed, gain=1.0):
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    d = cfg["width"]
    w = {"embed": rnd(cfg["vocab"], d, std=0.5), "pos": rnd(cfg["max_positions"], d, std=0.5), "final.norm": rnd(d, std=0.2),
         "head": rnd(cfg["vocab"], d, std=d ** -0.5)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H = m["heads"]
        w[p + "norm1"] = rnd(d, std=0.2)
        w[p + "mix.dq"] = rnd(m["q_rank"], d, std=d ** -0.5)
        w[p + "mix.dq.norm"] = 1 + rnd(m["q_rank"], std=0.2)
        w[p + "mix.uq"] = rnd(H * m["dim"], m["q_rank"], std=gain * m["q_rank"] ** -0.5)
        if "kv_from" not in m:
            w[p + "mix.dkv"] = rnd(m["kv_rank"], d, std=d ** -0.5)
            w[p + "mix.dkv.norm"] = 1 + rnd(m["kv_rank"], std=0.2)
        w[p + "mix.uk"] = rnd(H * m["dim"], m["kv_rank"], std=gain * m["kv_rank"] ** -0.5)
        w[p + "mix.uv"] = rnd(H * m["vdim"], m["kv_rank"], std=m["kv_rank"] ** -0.5)
        w[p + "mix.o"] = rnd(d, H * m["vdim"], std=(H * m["vdim"]) ** -0.5)
        f = layer["mlp"]
        if f is not None:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            w[p + "norm2"] = rnd(d, std=0.2)
            w[p + "mlp.router"] = rnd(E, d, std=2.0 * d ** -0.5)
            w[p + "mlp.correction"] = rnd(E, std=0.3)
            for e in range(E):
                w[f"{p}mlp.e{e}.up"] = rnd(ff, d, std=d ** -0.5)
                w[f"{p}mlp.e{e}.down"] = rnd(d, ff, std=ff ** -0.5)
    return w


def build(cfg, weights, dtype, slots=2, max_seq=None):
    from lit_gpt_b200.config import PomipelConfig
    from lit_gpt_b200.pomipel import Pomipel

    model = Pomipel(PomipelConfig.from_dict(cfg)).to("cuda").to(dtype)
    model.load_tensors(weights)
    if max_seq is not None:
        model.max_seq_length = max_seq
    model.set_kv_cache(batch_size=slots)
    return model.eval()


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def rel_err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


TOL = {torch.float32: 2e-5, torch.bfloat16: 6e-2}


def assert_close(got, want, dtype, what=""):
    """fp32: the whole block within rounding.  bf16: a rounding difference ahead of a router can move a token to another expert
    (in the restatement just as well), so the typical row and nine rows in ten must be within bf16 rounding; the fp32 runs of the same tests are the sharp ones."""
    if dtype == torch.float32:
        assert rel_err(got, want) < TOL[dtype], what
        return
    got, want = got.double().cpu(), want.double().cpu()
    rows = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-30)
    assert float(rows.median()) < 3e-2 and float((rows < TOL[dtype]).double().mean()) >= 0.9, (what, rows)


# ---------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_kernels(dtype):
    k = K()
    g = torch.Generator().manual_seed(1)
    n, d1, d2 = 7, 50, 37
    both = torch.randn(n, d1 + d2, generator=g).to(dtype).cuda()
    w1, w2 = (1 + 0.3 * torch.randn(d1, generator=g)).to(dtype).cuda(), (0.3 * torch.randn(d2, generator=g)).to(dtype).cuda()
    out1 = torch.zeros(n, d1, dtype=dtype, device="cuda")
    table = torch.zeros(20, d2, dtype=dtype, device="cuda")
    where = torch.tensor([3, 19, 0, 7, -1, 12, 5], device="cuda")
    k.rms_rows(n, 1e-3, k.rms_seg(both[:, :d1], w1, out1, d1, False), k.rms_seg(both[:, d1:], w2, table, d2, True, out_rows=where),
               in_dtype=dtype, out_dtype=dtype, device=both.device)
    assert rel_err(out1, O.norm_plain(both[:, :d1].cpu(), w1.cpu(), 1e-3, torch.float64)) < (1e-6 if dtype == torch.float32 else 6e-3)
    want2 = O.norm_zero_centred(both[:, d1:].cpu(), w2.cpu(), 1e-3, torch.float64)
    keep = [i for i in range(n) if int(where[i]) >= 0]
    assert rel_err(table[where[keep]], want2[keep]) < (1e-6 if dtype == torch.float32 else 6e-3)
    untouched = sorted(set(range(20)) - {int(where[i]) for i in keep})
    assert float(table[untouched].abs().max()) == 0.0   # the skipped row wrote nothing

    # residual update: fp32 stream, working copy in the model's dtype
    x = torch.randn(n, d1, generator=g).cuda()
    y = torch.randn(n, d1, generator=g).to(dtype).cuda() * 5
    x0, act = x.clone(), torch.empty(n, d1, dtype=dtype, device="cuda")
    wz = (0.3 * torch.randn(d1, generator=g)).to(dtype).cuda()
    k.residual_norm_add(y, wz, 1e-3, x, act)
    want = x0.double().cpu() + O.norm_zero_centred(y.cpu(), wz.cpu(), 1e-3, torch.float64)
    assert rel_err(x, want) < 1e-6 and x.dtype == torch.float32
    assert torch.equal(act, x.to(dtype))

    # final norm reads chosen rows of the fp32 stream
    pick = torch.tensor([6, 0, 3], device="cuda")
    xn = torch.empty(3, d1, dtype=dtype, device="cuda")
    k.rms_rows(3, 1e-3, k.rms_seg(x, wz, xn, d1, True, in_rows=pick), in_dtype=torch.float32, out_dtype=dtype, device=x.device)
    assert rel_err(xn, O.norm_zero_centred(x[pick].cpu(), wz.cpu(), 1e-3, torch.float64)) < (1e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_positions(dtype):
    k = K()
    g = torch.Generator().manual_seed(2)
    emb, pos = torch.randn(30, 44, generator=g).to(dtype), torch.randn(16, 44, generator=g).to(dtype)
    toks, where = [4, 29, 0, 4], [0, 15, 7, 1]
    x, act = k.embed_pos(torch.tensor(toks, dtype=torch.int32, device="cuda"), torch.tensor(where, dtype=torch.int32, device="cuda"), emb.cuda(),
                         pos.cuda(), 2.5)
    want = emb.double()[toks] * 2.5 + pos.double()[where]
    assert rel_err(x, want) < 1e-6 and torch.equal(act, x.to(dtype))


@pytest.mark.parametrize("experts,top,groups,keep", [(18, 5, 2, 1), (12, 4, 4, 2), (6, 1, 1, 1), (8, 2, 8, 3), (9, 3, 3, 3)])
def test_router(experts, top, groups, keep):
    k = K()
    g = torch.Generator().manual_seed(experts * 100 + top)
    n, d = 40, 52
    x = torch.randn(n, d, generator=g)
    w = {"r.router": torch.randn(experts, d, generator=g) * 0.3, "r.correction": torch.randn(experts, generator=g) * 0.4}
    ids, wts = k.moe_route(x.cuda(), w["r.router"].cuda(), w["r.correction"].cuda(), top, groups, keep)
    want_ids, want_w = O.route(x, w, "r.", dict(experts=experts, top=top, groups=dict(count=groups, keep=keep)), torch.float64)
    assert torch.equal(ids.cpu().long(), want_ids)          # same experts in the same (descending) order
    assert rel_err(wts, want_w) < 1e-6


def test_router_negative_choice_scores_and_excluded_groups():
    """With strongly negative corrections every choice score is below zero: an excluded group must count as minus infinity, not 0,
    and the weights stay the uncorrected sigmoid scores."""
    k = K()
    g = torch.Generator().manual_seed(5)
    n, d, E = 25, 24, 8
    x = torch.randn(n, d, generator=g)
    w = {"r.router": torch.randn(E, d, generator=g) * 0.2, "r.correction": -3.0 + 0.5 * torch.randn(E, generator=g)}
    ids, wts = k.moe_route(x.cuda(), w["r.router"].cuda(), w["r.correction"].cuda(), 2, 4, 1)
    want_ids, want_w = O.route(x, w, "r.", dict(experts=E, top=2, groups=dict(count=4, keep=1)), torch.float64)
    assert torch.equal(ids.cpu().long(), want_ids)
    assert (ids.cpu() // 2)[:, 0].eq((ids.cpu() // 2)[:, 1]).all()     # both picks from the one kept group
    assert rel_err(wts, want_w) < 1e-6 and float(wts.min()) > 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 5, 150])   # GEMV path (few pairs) and grouped path, with experts that get no token
def test_experts(dtype, n):
    k = K()
    g = torch.Generator().manual_seed(n)
    d, ff, E, top = 44, 27, 7, 3
    x = torch.randn(n, d, generator=g).to(dtype)
    w = {"m.router": torch.randn(E, d, generator=g) * 0.3, "m.correction": torch.randn(E, generator=g) * 0.4}
    w["m.correction"][2] = -50.0   # never chosen
    for e in range(E):
        w[f"m.e{e}.up"] = (torch.randn(ff, d, generator=g) * d ** -0.5).to(dtype)
        w[f"m.e{e}.down"] = (torch.randn(d, ff, generator=g) * ff ** -0.5).to(dtype)
    spec = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=E, top=top, groups=dict(count=1, keep=1)))
    hi = torch.float64 if dtype == torch.float32 else torch.bfloat16
    want = O.moe(x, {a: b.to(hi) if b.is_floating_point() else b for a, b in w.items()}, "m.", spec, hi)
    ids, wts = k.moe_route(x.cuda(), w["m.router"].to(dtype).cuda(), w["m.correction"].to(dtype).cuda(), top, 1, 1)
    up = torch.stack([w[f"m.e{e}.up"] for e in range(E)]).cuda()
    down = torch.stack([w[f"m.e{e}.down"] for e in range(E)]).cuda()
    got = k.moe_experts(x.cuda(), ids, wts, up, down)
    assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 1.5e-2)
    if n == 5:   # the two paths agree: force the grouped one
        old, k.MOE_GEMV_MAX_PAIRS = k.MOE_GEMV_MAX_PAIRS, 0
        try:
            again = k.moe_experts(x.cuda(), ids, wts, up, down)
        finally:
            k.MOE_GEMV_MAX_PAIRS = old
        assert rel_err(again, got) < (1e-6 if dtype == torch.float32 else 1e-2)


def test_expert_module_vendor_grouped_path_agrees_with_own_kernels():
    import lit_gpt_b200.moe as M
    from lit_gpt_b200.config import MoESpec

    g = torch.Generator().manual_seed(3)
    layer = M.SparseExperts(64, MoESpec(experts=8, top=3, ff=40, groups=4, keep=2)).cuda().to(torch.bfloat16)
    for p in layer.parameters():
        p.data.copy_(torch.randn(p.shape, generator=g) * (0.4 if p.dim() == 1 else p.shape[-1] ** -0.5))
    layer.router.correction.data[5] = -40.0   # an expert without tokens in the middle of the sorted rows
    x = torch.randn(300, 64, generator=g).to(torch.bfloat16).cuda()
    vendor = layer(x)
    M.VENDOR_GROUPED_GEMM = False
    try:
        own = layer(x)
    finally:
        M.VENDOR_GROUPED_GEMM = True
    assert rel_err(vendor, own) < 1e-2
    few = layer(x[:4])     # GEMV path on the first rows
    assert rel_err(few, own[:4]) < 1e-2


def _attention_reference(q, kk, v, scale, start):
    """q (T, H, dk) at positions start .., kk (start + T, H, dk), v (.., H, dv), all float64"""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=torch.float64)
    for i in range(T):
        for h in range(H):
            s = (kk[: start + i + 1, h] @ q[i, h]) * scale
            out[i, h] = torch.softmax(s, 0) @ v[: start + i + 1, h]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dv", [(20, 12), (64, 160), (36, 64), (64, 64), (128, 128)])   # the last two: tensor-core kernel in bf16
def test_prefill_attention_ragged(dtype, dk, dv):
    """Three sequences of unequal length in one launch, one of them continuing at a later position, lengths around the 64-row and
    64-key tile edges."""
    k = K()
    g = torch.Generator().manual_seed(dk)
    H, scale = 3, 0.21
    shapes = [(0, 65), (70, 59), (0, 1), (63, 2)]   # (first position, new rows)
    qs, ks, vs, meta, want = [], [], [], [], []
    qrow = krow = 0
    for start, T in shapes:
        q = torch.randn(T, H, dk, generator=g).to(dtype)
        kk = torch.randn(start + T, H, dk, generator=g).to(dtype)
        v = torch.randn(start + T, H, dv, generator=g).to(dtype)
        want.append(_attention_reference(q.double(), kk.double(), v.double(), scale, start).reshape(T, H * dv))
        qs.append(q.reshape(T, -1)); ks.append(kk.reshape(start + T, -1)); vs.append(v.reshape(start + T, -1))
        meta.append((qrow, T, start, krow))
        qrow += T; krow += start + T
    kv = torch.cat([torch.cat(ks), torch.cat(vs)], dim=1).cuda()      # keys and values as column slices of one buffer
    got = k.latent_prefill(torch.cat(qs).cuda(), kv[:, : H * dk], kv[:, H * dk :], torch.tensor(meta, dtype=torch.int32, device="cuda"),
                           max(t for _, t in shapes), H, dk, dv, scale)
    assert rel_err(got, torch.cat(want)) < (2e-6 if dtype == torch.float32 else 8e-3)
    if dtype == torch.bfloat16 and dk == dv:   # the any-size kernel on the same operands
        k.LATENT_PREFILL_MMA = False
        try:
            plain = k.latent_prefill(torch.cat(qs).cuda(), kv[:, : H * dk], kv[:, H * dk :], torch.tensor(meta, dtype=torch.int32, device="cuda"),
                                     max(t for _, t in shapes), H, dk, dv, scale)
        finally:
            k.LATENT_PREFILL_MMA = True
        assert rel_err(plain, torch.cat(want)) < 8e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_attention_finds_one_far_key(dtype):
    """Among hundreds of cached latents one (far back, or right at a tile / split edge) is made to match the query: the output
    must be that position's value.  Run for contexts around the 32-key tile and the per-split ranges, in a slot that is not 0."""
    k = K()
    g = torch.Generator().manual_seed(9)
    H, dk, dv, r, max_seq = 2, 24, 20, 40, 700
    w_uk = (torch.randn(H * dk, r, generator=g) * r ** -0.5).to(dtype)
    w_uv = (torch.randn(H * dv, r, generator=g) * r ** -0.5).to(dtype)
    for ctx, hot in [(1, 0), (32, 0), (33, 32), (257, 255), (513, 256), (600, 3), (600, 599), (700, 511)]:
        cache = torch.randn(3, max_seq, r, generator=g).to(dtype)
        cache[2, hot] *= 3.0
        q = torch.zeros(1, H * dk)
        for h in range(H):   # the query of head h points at the hot position's key
            q[0, h * dk : (h + 1) * dk] = 2.5 * (w_uk[h * dk : (h + 1) * dk].float() @ cache[2, hot].float())
        q = q.to(dtype)
        got = k.latent_decode(q.cuda(), w_uk.cuda(), w_uv.cuda(), cache.cuda(), torch.tensor([2], dtype=torch.int32, device="cuda"),
                              torch.tensor([ctx - 1], dtype=torch.int32, device="cuda"), H, dk, dv, 1.0, 4)
        kk = (cache[2, :ctx].double() @ w_uk.double().t()).view(ctx, H, dk)
        v = (cache[2, :ctx].double() @ w_uv.double().t()).view(ctx, H, dv)
        want = _attention_reference(q.double().view(1, H, dk), kk, v, 1.0, ctx - 1).reshape(1, -1)
        assert rel_err(got, want) < (2e-5 if dtype == torch.float32 else 2e-2), (ctx, hot)
        if ctx > 1:   # the hot key really decides the output
            assert rel_err(got, v[hot].reshape(1, -1)) < 0.05, (ctx, hot)
        # the position just past the context must not be seen, however loud it is
        cache2 = cache.clone()
        if ctx < max_seq:
            cache2[2, ctx] = cache[2, hot] * 50
            again = k.latent_decode(q.cuda(), w_uk.cuda(), w_uv.cuda(), cache2.cuda(), torch.tensor([2], dtype=torch.int32, device="cuda"),
                                    torch.tensor([ctx - 1], dtype=torch.int32, device="cuda"), H, dk, dv, 1.0, 4)
            assert torch.equal(again, got)


@pytest.mark.parametrize("H,r", [(16, 512), (5, 96), (20, 64), (1, 32)])
def test_decode_attention_tensor_core_kernel(H, r):
    """bf16 with a latent size that is a multiple of 32: sixteen heads per CTA on the tensor cores.  Ragged contexts in slots that
    are out of order, head counts that do not fill the last tile of sixteen, against fp64 and against the any-size kernel."""
    k = K()
    g = torch.Generator().manual_seed(H * r)
    dk, dv, max_seq = 24, 16, 300
    ctxs, slots = [1, 33, 64, 65, 300, 129], [4, 0, 5, 2, 1, 3]
    B = len(ctxs)
    w_uk = (torch.randn(H * dk, r, generator=g) * r ** -0.5).to(torch.bfloat16)
    w_uv = (torch.randn(H * dv, r, generator=g) * r ** -0.5).to(torch.bfloat16)
    cache = torch.randn(6, max_seq, r, generator=g).to(torch.bfloat16)
    q = (torch.randn(B, H * dk, generator=g) * 2).to(torch.bfloat16)
    args = (q.cuda(), w_uk.cuda(), w_uv.cuda(), cache.cuda(), torch.tensor(slots, dtype=torch.int32, device="cuda"),
            torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device="cuda"), H, dk, dv, 0.3)
    for splits in (1, 5):
        got = k.latent_decode(*args, splits)
        old = k.latent_decode_tune(True)
        try:
            plain = k.latent_decode(*args, splits)
        finally:
            k.latent_decode_tune(old)
        for b, (ctx, slot) in enumerate(zip(ctxs, slots)):
            kk = (cache[slot, :ctx].double() @ w_uk.double().t()).view(ctx, H, dk)
            v = (cache[slot, :ctx].double() @ w_uv.double().t()).view(ctx, H, dv)
            want = _attention_reference(q[b].double().view(1, H, dk), kk, v, 0.3, ctx - 1).reshape(1, -1)
            assert rel_err(got[b : b + 1], want) < 2e-2, (b, splits)
            assert rel_err(plain[b : b + 1], want) < 2e-2, (b, splits)


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cfg,seed", [(CFG_ODD, 11), (CFG_WIDE, 12), (CFG_RAGGED_SIZES, 13)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_matches_oracle(cfg, seed, dtype):
    w = checkpoint(cfg, seed)
    model = build(cfg, w, dtype)
    toks = tokens_for(cfg, 70, seed)
    got = model.step(toks, [(1, 0, len(toks))])
    want = O.forward(cfg, w, toks, torch.float64)
    assert got.dtype == torch.float32
    assert_close(got, want, dtype)
    if dtype == torch.bfloat16:   # and typically no further from the truth than the plain bf16 restatement is
        mine = ((got.double().cpu() - want).norm(dim=-1) / want.norm(dim=-1)).median()
        plain = ((O.forward(cfg, w, toks, torch.bfloat16).double() - want).norm(dim=-1) / want.norm(dim=-1)).median()
        assert float(mine) < 2.0 * float(plain) + 1e-3


def test_layers_follow_the_oracle_one_by_one():
    cfg = CFG_ODD
    w = checkpoint(cfg, 21)
    model = build(cfg, w, torch.float32)
    toks = tokens_for(cfg, 19, 21)
    seen = []
    hooks = [b.register_forward_hook(lambda m, a, o: seen.append(a[0].clone())) for b in model.blocks]
    model.step(toks, [(0, 0, len(toks))])
    for h in hooks:
        h.remove()
    _, layers = O.forward(cfg, w, toks, torch.float64, return_layers=True)
    for i, x in enumerate(seen):
        assert rel_err(x, layers[i]) < 1e-5, f"residual stream after layer {i}"


@pytest.mark.parametrize("cfg", [CFG_ODD, CFG_RAGGED_SIZES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decoding_token_by_token_equals_prefill(dtype, cfg):
    w = checkpoint(cfg, 31)
    model = build(cfg, w, dtype)
    toks = tokens_for(cfg, 45, 31)
    whole = model.step(toks, [(0, 0, len(toks))])
    rows = [model.step([t], [(1, p, 1)]) for p, t in enumerate(toks)]      # the very first token too is a decode step
    assert_close(torch.cat(rows), whole, dtype)
    assert_close(torch.cat(rows), O.forward(cfg, w, toks, torch.float64), dtype)


@pytest.mark.parametrize("portions", [[2, 2, 2, 60, 3, 64, 1, 65, 2], [199, 2], [1, 200]])
def test_prompt_in_portions(portions):
    cfg = CFG_WIDE
    w = checkpoint(cfg, 41)
    model = build(cfg, w, torch.float32)
    toks = tokens_for(cfg, sum(portions), 41)
    whole = model.step(toks, [(0, 0, len(toks))])
    got, at = [], 0
    for n in portions:
        got.append(model.step(toks[at : at + n], [(1, at, n)]))
        at += n
    assert rel_err(torch.cat(got), whole) < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_batch_equals_each_alone(dtype):
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_ODD
    w = checkpoint(cfg, 51)
    model = build(cfg, w, dtype)
    session = Session(model, slots=2)     # grows to 4 when the third request arrives
    lens = {"a": 1, "b": 67, "c": 130, "d": 9}
    prompts = {r: tokens_for(cfg, n + 12, 60 + i) for i, (r, n) in enumerate(lens.items())}
    alone = {r: O.forward(cfg, w, t, torch.float64) for r, t in prompts.items()}
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


def test_freed_slots_are_reused_without_leftovers():
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_ODD
    w = checkpoint(cfg, 71)
    model = build(cfg, w, torch.float32)
    session = Session(model, slots=2)
    long, short = tokens_for(cfg, 90, 72), tokens_for(cfg, 20, 73)
    session.step([("x", long, [0]), ("y", short, [0])], end=["x"])
    assert model.slots.in_use == 1
    # the new request takes x's slot, which still holds x's 90 latents; it must see only its own
    fresh = tokens_for(cfg, 33, 74)
    out = session.step([("z", fresh[:30], None)])
    assert session.live["z"][0] == 0
    assert rel_err(out, O.forward(cfg, w, fresh, torch.float64)[:30]) < 2e-5
    for p in range(30, 33):
        out = session.step([("z", [fresh[p]], [0]), ("y", [short[0]], [])])
        assert rel_err(out, O.forward(cfg, w, fresh, torch.float64)[p : p + 1]) < 2e-5


def test_one_loud_key_far_back_in_a_whole_model():
    """The first layer's query and key maps are scaled up so that its attention is nearly one-hot: a wrong, missing or shifted key
    anywhere in a long context would move the logits far beyond rounding.  Checked in a prompt and in decoding across 300 steps
    (several decode splits and many 32-key tiles)."""
    cfg = CFG_WIDE
    w = checkpoint(cfg, 81, gain=6.0)
    model = build(cfg, w, torch.float32)
    toks = tokens_for(cfg, 1000, 81)
    want = O.forward(cfg, w, toks, torch.float64)
    got = model.step(toks[:700], [(0, 0, 700)], want=list(range(0, 700, 7)))
    assert rel_err(got, want[0:700:7]) < 1e-4
    tail = [model.step([toks[p]], [(0, p, 1)]) for p in range(700, 1000)]
    assert rel_err(torch.cat(tail), want[700:]) < 1e-4


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
        seq.append(int(O.forward(cfg, w, seq, torch.float64)[-1].argmax()))
    model = build(cfg, w, dtype, slots=1, max_seq=64)
    y = generate(model, torch.tensor(prompt, device="cuda"), len(seq), temperature=0.0)
    if dtype == torch.float32:
        assert y.tolist() == seq
    other = tokens_for(cfg, 4, 92)
    model.set_kv_cache(batch_size=2)
    ys = generate_batch(model, [prompt, other], 14)
    assert ys[0] == y.tolist() and len(ys[1]) == 4 + 14 and model.slots.in_use == 0
    seq2 = list(other)
    for _ in range(14):
        seq2.append(int(O.forward(cfg, w, seq2, torch.float64)[-1].argmax()))
    if dtype == torch.float32:
        assert ys[1] == seq2


def test_forward_signature_of_the_other_models():
    """forward(idx, input_pos) with batch rows = slots and shared positions, as GPT.forward: a prompt, then single tokens."""
    cfg = CFG_ODD
    w = checkpoint(cfg, 95)
    model = build(cfg, w, torch.float32, slots=2)
    a, b = tokens_for(cfg, 12, 96), tokens_for(cfg, 12, 97)
    idx = torch.tensor([a, b], device="cuda")
    out = model(idx[:, :10], torch.arange(10, device="cuda"))
    for p in (10, 11):
        out = torch.cat([out, model(idx[:, p : p + 1], torch.tensor([p], device="cuda"))], dim=1)
    assert out.shape == (2, 12, cfg["vocab"])
    assert rel_err(out[0], O.forward(cfg, w, a, torch.float64)) < 2e-5 and rel_err(out[1], O.forward(cfg, w, b, torch.float64)) < 2e-5


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
    full = {k: O.forward(cfg, w, t, torch.float64) for k, t in (("a", a), ("b", b), ("c", c))}
    want = {0: torch.stack([full["a"][0], full["a"][36], full["b"][5]]), 2: torch.stack([full["a"][38], full["b"][7]]),
            3: full["a"][39:40], 4: full["c"][[0, 1, 63, 64, 69]]}
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    for step, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        assert got.shape == ref.shape
        assert_close(got, ref, dt, f"step {step}") if dt == torch.float32 else assert_close(torch.cat([got] * 4), torch.cat([ref] * 4), dt, f"step {step}")
