"""Pomipel: a decoder-only model of post-normed blocks -- latent attention (``latent.py``) and sparse experts (``moe.py``) --
over an fp32 residual stream.

    x  = embed[token] * embedding_scale + pos[position]                                  (fp32)
    x += zero_centred_norm_1(mixer(x));  x += zero_centred_norm_2(experts(x))            per block; branches read x itself
    logits = head(zero_centred_norm(x)) * logit_scale

with zero_centred_norm(y) = y / sqrt(mean(y^2) + eps) * (1 + w).  The residual stream, every norm, the softmax and the router
are fp32 whatever the matrix-product dtype (bfloat16 or float32) of weights and activations is; the matrix products go to the
vendor GEMM, everything else is this library's kernels.

The model plugs into the same entry points as ``GPT``: ``forward(idx, input_pos)`` over batch rows = cache slots,
``set_kv_cache`` / ``clear_kv_cache`` / ``max_seq_length``, and the CUDA-graph decode loop of ``generate.base``.  Serving several
sequences of different lengths goes through ``step``, which takes a ragged batch (tokens of several cache slots, each
continuing at its own position) and returns logits for the requested rows only.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kernels as K
from .config import PomipelConfig
from .latent import LatentAttention
from .moe import SparseExperts
from .ragged import RaggedBatch, SlotAllocator, SlotServed


class PomipelBlock(nn.Module):
    def __init__(self, config: PomipelConfig, index: int, source: Optional[LatentAttention]) -> None:
        super().__init__()
        spec = config.layers[index]
        self.eps = config.norm_eps
        self.mixer = LatentAttention(config.n_embd, spec.mixer, config.norm_eps, source)
        self.norm_1 = nn.Parameter(torch.zeros(config.n_embd), requires_grad=False)      # stored around zero: gain = 1 + w
        self.mlp = SparseExperts(config.n_embd, spec.mlp) if spec.mlp is not None else None
        self.norm_2 = nn.Parameter(torch.zeros(config.n_embd), requires_grad=False) if spec.mlp is not None else None

    def forward(self, x: torch.Tensor, act: torch.Tensor, batch: RaggedBatch, shared: Dict[int, torch.Tensor]) -> None:
        """x fp32 (n, d) residual and act = its copy in the matrix-product dtype, both updated in place."""
        K.residual_norm_add(self.mixer(act, batch, shared), self.norm_1, self.eps, x, act)
        if self.mlp is not None:
            K.residual_norm_add(self.mlp(act), self.norm_2, self.eps, x, act)


class Pomipel(SlotServed, nn.Module):

    def __init__(self, config: PomipelConfig) -> None:
        super().__init__()
        self.config = config
        d = config.n_embd
        self.embed = nn.Parameter(torch.empty(config.vocab_size, d), requires_grad=False)
        self.pos = nn.Parameter(torch.empty(config.block_size, d), requires_grad=False)
        blocks: List[PomipelBlock] = []
        for i, layer in enumerate(config.layers):
            src = None if layer.mixer.kv_from is None else blocks[layer.mixer.kv_from].mixer
            blocks.append(PomipelBlock(config, i, src))
        self.blocks = nn.ModuleList(blocks)
        self.final_norm = nn.Parameter(torch.zeros(d), requires_grad=False)
        self.head = nn.Parameter(torch.empty(config.vocab_size, d), requires_grad=False)
        self._max_seq_length = config.block_size
        self.slots: Optional[SlotAllocator] = None

    # ---- the surface generate() uses (with ``SlotServed``) --------------------------------------------------------
    def set_kv_cache(self, batch_size: int, rope_cache_length: Optional[int] = None, device: Optional[torch.device] = None,
                     dtype: Optional[torch.dtype] = None) -> None:
        """`batch_size` cache slots of `max_seq_length` positions for every layer that projects its own latents."""
        device = device if device is not None else self.device
        dtype = dtype if dtype is not None else self.dtype
        for block in self.blocks:
            block.mixer.cache = block.mixer.build_cache(batch_size, self.max_seq_length, device, dtype)
        self.slots = SlotAllocator(batch_size)
        self._drop_graphs()

    def clear_kv_cache(self) -> None:
        for block in self.blocks:
            block.mixer.cache = None
        self.slots = None
        self._drop_graphs()

    def reset_caches(self) -> None:
        for block in self.blocks:
            if block.mixer.cache is not None:
                block.mixer.cache.reset_parameters()

    def _apply(self, fn, recurse: bool = True):
        self._drop_graphs()
        return super()._apply(fn, recurse)

    def state_tensors(self) -> List[torch.Tensor]:
        return [b.mixer.cache.latents for b in self.blocks if b.mixer.cache is not None]

    # ---- weights ----------------------------------------------------------------------------------------------------
    def reset_parameters(self, seed: int = 1234, std: float = 0.02) -> None:
        """Random weights for benchmarks and smoke runs: N(0, std) matrices, unit plain norms, zero-centred norms and selection
        biases at zero."""
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith(("q_norm", "kv_norm")):
                p.data.fill_(1.0)
            elif p.dim() == 1:
                p.data.zero_()
            else:
                p.data.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=gen))

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Fill the parameters from the checkpoint's tensors: ``embed``, ``pos``, ``final.norm``, ``head`` and per layer i
        ``l<i>.norm1|norm2``, ``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|o``, ``l<i>.mlp.router|correction|e<j>.up|e<j>.down``.
        Projections that feed one matrix product are stored fused (dq + dkv, uk + uv), expert weights stacked."""
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

        put(self.embed, take("embed"))
        put(self.pos, take("pos"))
        put(self.final_norm, take("final.norm"))
        put(self.head, take("head"))
        for i, block in enumerate(self.blocks):
            p, mx = f"l{i}.", block.mixer
            put(block.norm_1, take(p + "norm1"))
            down = [take(p + "mix.dq")] + ([take(p + "mix.dkv")] if mx.owns_latent else [])
            put(mx.w_down, torch.cat(down, dim=0))
            put(mx.q_norm, take(p + "mix.dq.norm"))
            if mx.owns_latent:
                put(mx.kv_norm, take(p + "mix.dkv.norm"))
            put(mx.w_uq, take(p + "mix.uq"))
            put(mx.w_ukv, torch.cat([take(p + "mix.uk"), take(p + "mix.uv")], dim=0))
            put(mx.w_o, take(p + "mix.o"))
            if block.mlp is not None:
                put(block.norm_2, take(p + "norm2"))
                put(block.mlp.router.weight, take(p + "mlp.router"))
                put(block.mlp.router.correction, take(p + "mlp.correction"))
                E = block.mlp.spec.experts
                put(block.mlp.w_up, torch.stack([take(f"{p}mlp.e{j}.up") for j in range(E)]))
                put(block.mlp.w_down, torch.stack([take(f"{p}mlp.e{j}.down") for j in range(E)]))
        extra = sorted(set(tensors) - used)
        if extra:
            raise KeyError(f"unexpected tensors in the checkpoint: {extra[:6]}")

    # ---- one step ---------------------------------------------------------------------------------------------------
    def _run(self, tokens: torch.Tensor, batch: RaggedBatch, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """tokens int32 (n,) -> fp32 logits (rows wanted or n, vocab)"""
        c = self.config
        with self._true_fp32():
            x, act = K.embed_pos(tokens, batch.row_pos, self.embed, self.pos, c.embedding_scale)
            shared: Dict[int, torch.Tensor] = {}
            for block in self.blocks:
                block(x, act, batch, shared)
            rows = x.shape[0] if want_rows is None else want_rows.numel()
            xn = torch.empty((rows, c.n_embd), dtype=self.dtype, device=x.device)
            K.rms_rows(rows, c.norm_eps, K.rms_seg(x, self.final_norm, xn, c.n_embd, True, in_rows=want_rows),
                       in_dtype=torch.float32, out_dtype=self.dtype, device=x.device)
            return K.scale_f32(F.linear(xn, self.head), c.logit_scale)

    @torch.inference_mode()
    def step(self, tokens: Sequence[int], seqs: Sequence[Tuple[int, int, int]], want: Optional[Sequence[int]] = None) -> torch.Tensor:
        """One step over a ragged batch.  `tokens`: the new tokens of all sequences, sequence after sequence; `seqs`: per
        sequence (cache slot, position of its first new token, number of new tokens); `want`: indices into `tokens` of the rows
        whose logits are returned (default: all).  Returns fp32 (rows, vocab).  Every sequence's earlier positions must be in
        its slot already; all of a step's sequences are computed together."""
        if self.slots is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        dev, L = self.device, self.max_seq_length
        n = len(tokens)
        if n == 0 or n != sum(s[2] for s in seqs):
            raise ValueError("step: the sequence lengths must add up to the number of tokens (> 0)")
        row_pos, row_slot, seq_meta, ctx_rows = [], [], [], []
        first = 0
        for slot, start, length in seqs:
            if not 0 <= slot < self.slots.capacity or length <= 0 or start < 0 or start + length > L:
                raise ValueError(f"step: sequence (slot {slot}, start {start}, length {length}) does not fit {self.slots.capacity} slots of {L}")
            row_pos.extend(range(start, start + length))
            row_slot.extend([slot] * length)
            seq_meta.append((first, length, start, len(ctx_rows)))
            ctx_rows.extend(range(slot * L, slot * L + start + length))
            first += length
        decode = all(s[2] == 1 for s in seqs)
        i32 = torch.tensor([list(tokens), row_pos, row_slot], dtype=torch.int32).to(dev, non_blocking=True)
        cache_rows = [s * L + p for s, p in zip(row_slot, row_pos)]
        i64 = torch.tensor(cache_rows + (list(want) if want is not None else []) + ([] if decode else ctx_rows), dtype=torch.int64).to(dev, non_blocking=True)
        nw = 0 if want is None else len(want)
        batch = RaggedBatch(row_pos=i32[1], row_slot=i32[2], cache_rows=i64[:n], decode=decode, context_hint=max(row_pos) + 1,
                            max_q_len=max(s[2] for s in seqs))
        if not decode:
            batch.seqs = torch.tensor(seq_meta, dtype=torch.int32).to(dev, non_blocking=True)
            batch.ctx_rows = i64[n + nw :]
        return self._run(i32[0], batch, i64[n : n + nw] if want is not None else None)

    def forward(self, idx: torch.Tensor, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """idx (B, T) token ids, batch row b = cache slot b, all rows at the positions `input_pos` (T,), as ``GPT.forward``.
        Returns fp32 logits (B, T, vocab).  T = 1 runs without any host synchronisation (CUDA-graph capturable)."""
        B, T = idx.shape
        if input_pos is None:
            raise TypeError("Pomipel runs over its cache: pass input_pos")
        if self.slots is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        if B > self.slots.capacity:
            raise ValueError(f"batch of {B} rows, but only {self.slots.capacity} cache slots")
        dev, L = idx.device, self.max_seq_length
        const = self.__dict__.get("_const")
        if const is None or const[0].numel() < B or const[0].device != dev:
            slots = torch.arange(max(B, self.slots.capacity), dtype=torch.int32, device=dev)
            const = self.__dict__["_const"] = (slots, slots.to(torch.int64) * L)
        if T == 1:
            pos32 = input_pos.to(torch.int32).expand(B).contiguous()
            batch = RaggedBatch(row_pos=pos32, row_slot=const[0][:B], cache_rows=const[1][:B] + input_pos.to(torch.int64), decode=True,
                                context_hint=L)
            return self._run(idx.reshape(B).to(torch.int32), batch, None).view(B, 1, -1)
        start = int(input_pos[0])   # host read: sizes the context of the prompt's attention
        if start + T > L:
            raise ValueError(f"Cannot forward sequence of length {start + T}, max seq length is only {L}.")
        pos32 = input_pos.to(torch.int32)
        ctx = start + T
        batch = RaggedBatch(
            row_pos=pos32.repeat(B), row_slot=const[0][:B].repeat_interleave(T),
            cache_rows=(const[1][:B, None] + input_pos.to(torch.int64)[None, :]).reshape(-1), decode=False, context_hint=ctx,
            seqs=torch.tensor([(b * T, T, start, b * ctx) for b in range(B)], dtype=torch.int32).to(dev),
            ctx_rows=(const[1][:B, None] + torch.arange(ctx, device=dev)[None, :]).reshape(-1), max_q_len=T)
        return self._run(idx.reshape(B * T).to(torch.int32), batch, None).view(B, T, -1)


def load_pomipel(checkpoint_dir: Any, dtype: torch.dtype = torch.bfloat16, device: Any = "cuda") -> Pomipel:
    """Build the Pomipel model of a checkpoint directory (``config.json`` + ``model.safetensors``) on `device` in `dtype`."""
    from .checkpoint import load_registered

    model = load_registered(checkpoint_dir, dtype=dtype, device=device)
    if not isinstance(model, Pomipel):
        raise TypeError(f"{str(checkpoint_dir)!r} does not hold a Pomipel model")
    return model
