"""Lefalix: a decoder-only model of sandwich-normed blocks over an fp32 residual stream, without a position table.

    x = embed[token]                                                                      (fp32)
    per layer run:  x += norm_1b(mixer(norm_1(x)));  x += norm_2b(ff(norm_2(x)))          norm(y) = y / sqrt(mean(y^2) + eps) * w
    logits = head(final_norm(x))

Mixers: ``channel_delta`` -- a gated delta rule with one decay per head and key channel (``delta.GatedDeltaRule``);
``parallel`` -- sliding-window attention with a sink (``window.WindowAttention``) and a gated delta rule with one decay per
head side by side on the same input, joined as (norm(left) * w_left + norm(right) * w_right) / 2.  Feed-forwards: dense
with the exact gelu, or softmax-routed gated experts (``moe``), or none.  A run of consecutive layers may repeat with the same
weights; every repetition keeps states of its own, and the embedding is added to the stream again before each repetition
but the first.

The residual stream, norms, softmax, router, decays and recurrent states are fp32 whatever the matrix-product dtype is; the
products go to the vendor GEMM, everything else is this library's kernels: ``K.sandwich_residual`` does a sublayer's
post-norm, the residual sum and the next sublayer's pre-norm in one launch.

Sequences live in slots: per layer run and slot a constant-size state (convolution tails, key / value rings of one window,
delta-rule matrices), so a sequence can be any length.  The model plugs into the entry points ``Pomipel`` uses:
``forward(idx, input_pos)`` for ``generate.base`` (single-token steps are CUDA-graph capturable), and ``step`` over ragged
batches for ``generate.serve.Session``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kernels as K
from .config import DenseMLPSpec, GatedMoESpec, LefalixConfig, LefalixLayerSpec
from .delta import GatedDeltaRule
from .moe import DenseMLP, GatedSparseExperts
from .ragged import RaggedBatch, SlotAllocator, SlotServed, state_batch
from .window import WindowAttention


class ParallelState(nn.Module):
    def __init__(self, left: nn.Module, right: nn.Module) -> None:
        super().__init__()
        self.left, self.right = left, right

    def tensors(self) -> List[torch.Tensor]:
        return self.left.tensors() + self.right.tensors()


class ParallelMixer(nn.Module):
    """Two mixers reading the same input; their outputs are joined by the block's residual kernel."""

    def __init__(self, width: int, spec: Any, eps: float) -> None:
        super().__init__()
        self.left = WindowAttention(width, spec.left, eps)
        self.right = GatedDeltaRule(width, spec.right, eps)
        self.left_out = nn.Parameter(torch.ones(width), requires_grad=False)
        self.right_out = nn.Parameter(torch.ones(width), requires_grad=False)

    def build_state(self, slots: int, device=None, dtype=None) -> ParallelState:
        return ParallelState(self.left.build_state(slots, device, dtype), self.right.build_state(slots, device, dtype))


class LefalixBlock(nn.Module):
    def __init__(self, config: LefalixConfig, spec: LefalixLayerSpec) -> None:
        super().__init__()
        d, self.eps = config.n_embd, config.norm_eps
        self.parallel = spec.type == "parallel"
        self.mixer = ParallelMixer(d, spec.mixer, self.eps) if self.parallel else GatedDeltaRule(d, spec.mixer, self.eps)
        self.norm_1 = nn.Parameter(torch.ones(d), requires_grad=False)
        self.norm_1b = nn.Parameter(torch.ones(d), requires_grad=False)
        if isinstance(spec.mlp, DenseMLPSpec):
            self.mlp: Optional[nn.Module] = DenseMLP(d, spec.mlp.ff)
        elif isinstance(spec.mlp, GatedMoESpec):
            self.mlp = GatedSparseExperts(d, spec.mlp)
        else:
            self.mlp = None
        self.norm_2 = nn.Parameter(torch.ones(d), requires_grad=False) if self.mlp is not None else None
        self.norm_2b = nn.Parameter(torch.ones(d), requires_grad=False) if self.mlp is not None else None

    def forward(self, x: torch.Tensor, act: torch.Tensor, batch: RaggedBatch, state: nn.Module, next_norm: Optional[torch.Tensor]) -> None:
        """x fp32 (n, d) residual, updated in place; act (n, d) = norm_1(x) in the matrix-product dtype on entry, on exit the
        stream normed with `next_norm` (the pre-norm of whatever reads the stream next; None: left as it is)."""
        after_mixer = self.norm_2 if self.mlp is not None else next_norm
        if self.parallel:
            yl = self.mixer.left(act, batch, state.left)
            yr = self.mixer.right(act, batch, state.right)
            K.sandwich_residual(x, yl, self.norm_1b, self.eps, w0=self.mixer.left_out, y1=yr, w1=self.mixer.right_out, pre_w=after_mixer, act=act)
        else:
            K.sandwich_residual(x, self.mixer(act, batch, state), self.norm_1b, self.eps, pre_w=after_mixer, act=act)
        if self.mlp is not None:
            K.sandwich_residual(x, self.mlp(act), self.norm_2b, self.eps, pre_w=next_norm, act=act)


class Lefalix(SlotServed, nn.Module):
    repeatable_steps = False   # a step advances recurrent states and convolution tails: repeating it is not idempotent

    def __init__(self, config: LefalixConfig) -> None:
        super().__init__()
        self.config = config
        d = config.n_embd
        self.embed = nn.Parameter(torch.empty(config.vocab_size, d), requires_grad=False)
        self.blocks = nn.ModuleList(LefalixBlock(config, spec) for spec in config.layers)
        self.final_norm = nn.Parameter(torch.ones(d), requires_grad=False)
        self.head = nn.Parameter(torch.empty(config.vocab_size, d), requires_grad=False)
        self.runs = config.schedule()                       # (layer, state index, the embedding re-enters before this run)
        self._max_seq_length = config.block_size
        self.slots: Optional[SlotAllocator] = None
        self.states: Optional[nn.ModuleList] = None         # one state per layer RUN: a repeated layer has one per repetition
        self.trace: Optional[List[torch.Tensor]] = None     # debugging: set to a list to receive the stream after every layer run

    # ---- the surface generate() uses (with ``SlotServed``) --------------------------------------------------------
    def set_kv_cache(self, batch_size: int, rope_cache_length: Optional[int] = None, device: Optional[torch.device] = None,
                     dtype: Optional[torch.dtype] = None) -> None:
        """`batch_size` state slots for every layer run.  A state is constant in size: nothing depends on `max_seq_length`."""
        device = device if device is not None else self.device
        dtype = dtype if dtype is not None else self.dtype
        self.states = nn.ModuleList(self.blocks[layer].mixer.build_state(batch_size, device, dtype) for layer, _, _ in self.runs)
        self.slots = SlotAllocator(batch_size)
        self._drop_graphs()

    def clear_kv_cache(self) -> None:
        self.states = None
        self.slots = None
        self._drop_graphs()

    def reset_caches(self) -> None:
        for t in self.state_tensors():
            t.zero_()

    def state_tensors(self) -> List[torch.Tensor]:
        return [t for st in (self.states or []) for t in st.tensors()]

    def _apply(self, fn, recurse: bool = True):
        self._drop_graphs()
        states, self.states = self.states, None     # states keep their own dtypes (fp32 matrices): a cast of the model skips them
        try:
            return super()._apply(fn, recurse)
        finally:
            self.states = states

    # ---- weights ----------------------------------------------------------------------------------------------------
    def reset_parameters(self, seed: int = 1234, std: float = 0.02) -> None:
        """Random weights for benchmarks and smoke runs: N(0, std) matrices, convolution taps N(0, 0.5), unit norms, zero biases,
        sinks, decay parameters."""
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for name, p in self.named_parameters():
            leaf = name.rsplit(".", 1)[-1]
            if leaf.startswith("norm") or leaf in ("final_norm", "left_out", "right_out"):
                p.data.fill_(1.0)
            elif p.dim() == 1:
                p.data.zero_()
            else:
                p.data.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, 0.5 if leaf == "conv" else std, generator=gen))

    @staticmethod
    def complete_config(config: LefalixConfig, shapes: Dict[str, Tuple[int, ...]]) -> None:
        """Sizes the configuration file leaves to the weights: the inner sizes of the low-rank decay and gate projections."""
        for i, layer in enumerate(config.layers):
            if layer.type == "channel_delta":
                layer.mixer.decay_rank = int(shapes[f"l{i}.mix.a1"][0])
                layer.mixer.gate_rank = int(shapes[f"l{i}.mix.g1"][0])

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Fill the parameters from the checkpoint's tensors: ``embed``, ``final.norm``, ``head`` and per layer i
        ``l<i>.norm1|norm1b|norm2|norm2b``, the mixer under ``l<i>.mix.`` (``q|k|v`` with ``.conv``, ``b``, ``A_log``, ``dt_bias``, ``norm``,
        ``o`` and ``a1|a2|g1|g2`` or ``a|g`` for a delta rule; under ``left.`` also ``.b`` biases and ``sink``; ``left.out`` /
        ``right.out``) and the feed-forward under ``l<i>.mlp.`` (``up|down`` or ``router`` and ``e<j>.gate|up|down``).  Projections that
        read the same input are stored fused, expert weights stacked."""
        used = set()

        def take(name: str) -> torch.Tensor:
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            return tensors[name]

        def put(param: nn.Parameter, value: torch.Tensor) -> None:
            if tuple(param.shape) != tuple(value.shape):
                raise ValueError(f"shape mismatch: parameter {tuple(param.shape)} vs checkpoint {tuple(value.shape)}")
            param.data.copy_(value)

        def put_delta(mx: GatedDeltaRule, p: str) -> None:
            if mx.spec.channel:
                rows = [take(p + "q"), take(p + "k"), take(p + "v"), take(p + "g1"), take(p + "a1"), take(p + "b")]
                put(mx.w_gate2, take(p + "g2"))
                put(mx.w_decay2, take(p + "a2"))
            else:
                rows = [take(p + "q"), take(p + "k"), take(p + "v"), take(p + "g"), take(p + "a"), take(p + "b")]
            put(mx.w_in, torch.cat(rows, dim=0))
            put(mx.conv, torch.cat([take(p + "q.conv"), take(p + "k.conv"), take(p + "v.conv")], dim=0))
            put(mx.a_log, take(p + "A_log"))
            put(mx.dt_bias, take(p + "dt_bias"))
            put(mx.norm, take(p + "norm"))
            put(mx.w_o, take(p + "o"))

        put(self.embed, take("embed"))
        put(self.final_norm, take("final.norm"))
        put(self.head, take("head"))
        for i, block in enumerate(self.blocks):
            p = f"l{i}."
            put(block.norm_1, take(p + "norm1"))
            put(block.norm_1b, take(p + "norm1b"))
            if block.parallel:
                lf, q = block.mixer.left, p + "mix.left."
                put(lf.w_qkv, torch.cat([take(q + "q"), take(q + "k"), take(q + "v")], dim=0))
                put(lf.b_qkv, torch.cat([take(q + "q.b"), take(q + "k.b"), take(q + "v.b")], dim=0))
                put(lf.conv, torch.cat([take(q + "q.conv"), take(q + "k.conv"), take(q + "v.conv")], dim=0))
                put(lf.sink, take(q + "sink"))
                put(lf.w_o, take(q + "o"))
                put(lf.b_o, take(q + "o.b"))
                put_delta(block.mixer.right, p + "mix.right.")
                put(block.mixer.left_out, take(p + "mix.left.out"))
                put(block.mixer.right_out, take(p + "mix.right.out"))
            else:
                put_delta(block.mixer, p + "mix.")
            if block.mlp is None:
                used.update(n for n in (p + "norm2", p + "norm2b") if n in tensors)   # a layer without feed-forward has no use for them
                continue
            put(block.norm_2, take(p + "norm2"))
            put(block.norm_2b, take(p + "norm2b"))
            if isinstance(block.mlp, DenseMLP):
                put(block.mlp.w_up, take(p + "mlp.up"))
                put(block.mlp.w_down, take(p + "mlp.down"))
            else:
                E = block.mlp.spec.experts
                put(block.mlp.router.weight, take(p + "mlp.router"))
                put(block.mlp.w_up, torch.stack([torch.cat([take(f"{p}mlp.e{j}.gate"), take(f"{p}mlp.e{j}.up")], dim=0) for j in range(E)]))
                put(block.mlp.w_down, torch.stack([take(f"{p}mlp.e{j}.down") for j in range(E)]))
        extra = sorted(set(tensors) - used)
        if extra:
            raise KeyError(f"unexpected tensors in the checkpoint: {extra[:6]}")

    # ---- one step ---------------------------------------------------------------------------------------------------
    def _run(self, tokens: torch.Tensor, batch: RaggedBatch, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """tokens int32 (n,) -> fp32 logits (rows wanted or n, vocab)"""
        c, eps = self.config, self.config.norm_eps
        n, d = tokens.numel(), c.n_embd
        with self._true_fp32():
            x, emb = K.embed_pos(tokens, None, self.embed, None, 1.0)
            act = torch.empty_like(emb)
            first = self.blocks[self.runs[0][0]].norm_1 if self.runs else self.final_norm
            K.rms_rows(n, eps, K.rms_seg(x, first, act, d, False), in_dtype=torch.float32, out_dtype=self.dtype, device=x.device)
            for r, (layer, state, reenter) in enumerate(self.runs):
                block = self.blocks[layer]
                if reenter:   # the embedding joins the stream again; the run's pre-norm is taken anew
                    K.sandwich_residual(x, emb, None, eps, pre_w=block.norm_1, act=act)
                nxt = None
                if r + 1 < len(self.runs) and not self.runs[r + 1][2]:
                    nxt = self.blocks[self.runs[r + 1][0]].norm_1
                block(x, act, batch, self.states[state], nxt)
                if self.trace is not None:
                    self.trace.append(x.clone())
            rows = n if want_rows is None else want_rows.numel()
            xn = torch.empty((rows, d), dtype=self.dtype, device=x.device)
            K.rms_rows(rows, eps, K.rms_seg(x, self.final_norm, xn, d, False, in_rows=want_rows), in_dtype=torch.float32, out_dtype=self.dtype,
                       device=x.device)
            return K.scale_f32(F.linear(xn, self.head), 1.0)

    @torch.inference_mode()
    def step(self, tokens: Sequence[int], seqs: Sequence[Tuple[int, int, int]], want: Optional[Sequence[int]] = None) -> torch.Tensor:
        """One step over a ragged batch.  `tokens`: the new tokens of all sequences, sequence after sequence; `seqs`: per
        sequence (state slot, position of its first new token, number of new tokens); `want`: indices into `tokens` of the rows
        whose logits are returned (default: all).  Returns fp32 (rows, vocab).  A sequence at position 0 starts from an empty
        state whatever its slot held; otherwise its slot must hold the state its earlier tokens left."""
        if self.slots is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        dev = self.device
        n = len(tokens)
        if n == 0 or n != sum(s[2] for s in seqs):
            raise ValueError("step: the sequence lengths must add up to the number of tokens (> 0)")
        for slot, start, length in seqs:
            if not 0 <= slot < self.slots.capacity or length <= 0 or start < 0 or start + length > self.max_seq_length:
                raise ValueError(f"step: sequence (slot {slot}, start {start}, length {length}) does not fit {self.slots.capacity} slots")
        batch, toks = state_batch(seqs, dev, tokens)
        want_rows = None if want is None else torch.tensor(list(want), dtype=torch.int64).to(dev, non_blocking=True)
        return self._run(toks, batch, want_rows)

    def forward(self, idx: torch.Tensor, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """idx (B, T) token ids, batch row b = state slot b, all rows at the positions `input_pos` (T,), as ``GPT.forward``.
        Returns fp32 logits (B, T, vocab).  T = 1 runs without any host synchronisation (CUDA-graph capturable)."""
        B, T = idx.shape
        if input_pos is None:
            raise TypeError("Lefalix runs over its states: pass input_pos")
        if self.slots is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        if B > self.slots.capacity:
            raise ValueError(f"batch of {B} rows, but only {self.slots.capacity} state slots")
        dev = idx.device
        const = self.__dict__.get("_const")
        if const is None or const[0].numel() < B or const[0].device != dev:
            slots = torch.arange(max(B, self.slots.capacity), dtype=torch.int32, device=dev)
            const = self.__dict__["_const"] = (slots, torch.ones_like(slots))
        ar = const[0][:B]
        if T == 1:
            seq_state = torch.stack([ar, const[1][:B], input_pos.to(torch.int32).expand(B), ar], dim=1).contiguous()
            batch = RaggedBatch(row_pos=None, row_slot=None, cache_rows=None, decode=True, context_hint=self.max_seq_length, seq_state=seq_state,
                                row_seq=ar)
            return self._run(idx.reshape(B).to(torch.int32), batch, None).view(B, 1, -1)
        start = int(input_pos[0])   # host read: the prompt's rows are laid out on the host
        if start + T > self.max_seq_length:
            raise ValueError(f"Cannot forward sequence of length {start + T}, max seq length is only {self.max_seq_length}.")
        seq_state = torch.tensor([(b * T, T, start, b) for b in range(B)], dtype=torch.int32).to(dev)
        batch = RaggedBatch(row_pos=None, row_slot=None, cache_rows=None, decode=False, context_hint=start + T, max_q_len=T, seq_state=seq_state,
                            identity_ctx=start == 0, row_seq=ar.repeat_interleave(T))
        return self._run(idx.reshape(B * T).to(torch.int32), batch, None).view(B, T, -1)
