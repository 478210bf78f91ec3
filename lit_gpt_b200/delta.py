"""Gated delta rule: a recurrent mixer whose state is one dim x vdim matrix per head, kept in fp32.

    q, k = silu(conv(W_q h)), silu(conv(W_k h))   per query / key head, then unit vectors (q also times dim^-1/2);
    v    = silu(conv(W_v h))                      per value head (value head j reads query / key head j / (heads / kv_heads));
    beta = sigmoid(W_b h);   g = exp(-exp(A_log) * softplus(a + dt_bias))
           with a = W_a h, one decay per head -- or (channel) a = W_a2 (W_a1 h), one per head and key channel;
    per token:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
    out  = W_o concat_h( o / sqrt(mean(o^2) + eps) * w_norm * gate ),   gate = silu(W_g h)  or (channel) sigmoid(W_g2 (W_g1 h)).

All projections that read h run as ONE matrix product (rows q | k | v | gate or gate-in | beta | decay or decay-in); the
convolution with its activation and unit norm is one kernel writing fp32, the recurrence (decay, softplus, sigmoid and state
in fp32) a second, the gated norm a third.  What a sequence keeps between steps (``DeltaState``): the last conv - 1 projected
rows of q | k | v and the state matrices, laid out as the recurrence kernel reads them.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kernels as K
from .config import DeltaMixerSpec
from .ragged import RaggedBatch


class DeltaState(nn.Module):
    """Per slot: conv tail (conv - 1, columns of q | k | v) in the model dtype and the fp32 state matrices of all heads."""

    def __init__(self, slots: int, spec: DeltaMixerSpec, device=None, dtype=None) -> None:
        super().__init__()
        cols = 2 * spec.kv_heads * spec.dim + spec.heads * spec.vdim
        floats = spec.heads * K.delta_rule_state_floats(spec.dim, spec.vdim)
        self.register_buffer("tail", torch.zeros((slots, max(spec.conv - 1, 1), cols), device=device, dtype=dtype), persistent=False)
        self.register_buffer("matrices", torch.zeros((slots, floats), device=device, dtype=torch.float32), persistent=False)

    def tensors(self):
        return [self.tail, self.matrices]


class GatedDeltaRule(nn.Module):
    def __init__(self, width: int, spec: DeltaMixerSpec, eps: float) -> None:
        super().__init__()
        self.spec, self.eps, self.width = spec, eps, width
        H, G, dk, dv = spec.heads, spec.kv_heads, spec.dim, spec.vdim
        self.conv_cols = 2 * G * dk + H * dv
        if spec.channel:
            if spec.decay_rank <= 0 or spec.gate_rank <= 0:
                raise ValueError("a per-channel delta rule needs the inner sizes of its low-rank decay and gate projections")
            # q | k | v | gate-in (gate_rank) | decay-in (decay_rank) | beta (H)
            self.off_gate, self.off_decay = self.conv_cols, self.conv_cols + spec.gate_rank
            self.off_beta = self.off_decay + spec.decay_rank
            self.w_gate2 = nn.Parameter(torch.empty(H * dv, spec.gate_rank), requires_grad=False)
            self.w_decay2 = nn.Parameter(torch.empty(H * dk, spec.decay_rank), requires_grad=False)
            self.dt_bias = nn.Parameter(torch.zeros(H * dk), requires_grad=False)
        else:
            # q | k | v | gate (H dv) | decay (H) | beta (H)
            self.off_gate, self.off_decay = self.conv_cols, self.conv_cols + H * dv
            self.off_beta = self.off_decay + H
            self.dt_bias = nn.Parameter(torch.zeros(H), requires_grad=False)
        self.w_in = nn.Parameter(torch.empty(self.off_beta + H, width), requires_grad=False)
        self.conv = nn.Parameter(torch.empty(self.conv_cols, spec.conv), requires_grad=False)
        self.a_log = nn.Parameter(torch.zeros(H), requires_grad=False)
        self.norm = nn.Parameter(torch.ones(dv), requires_grad=False)
        self.w_o = nn.Parameter(torch.empty(width, H * dv), requires_grad=False)

    def build_state(self, slots: int, device=None, dtype=None) -> DeltaState:
        return DeltaState(slots, self.spec, device, dtype)

    def forward(self, h: torch.Tensor, batch: RaggedBatch, state: DeltaState) -> torch.Tensor:
        """h (n, width) in the matrix-product dtype -> (n, width)"""
        s, n = self.spec, h.shape[0]
        H, G, dk, dv = s.heads, s.kv_heads, s.dim, s.vdim
        proj = F.linear(h, self.w_in)
        qkv = torch.empty((n, self.conv_cols), dtype=torch.float32, device=h.device)
        q, k, v = qkv[:, : G * dk], qkv[:, G * dk : 2 * G * dk], qkv[:, 2 * G * dk :]
        cw = self.conv
        groups = [
            K.conv_group(cw[: G * dk], q, 0, G, dk, act=1, post=2, post_scale=dk ** -0.5, eps=1e-6),
            K.conv_group(cw[G * dk : 2 * G * dk], k, G * dk, G, dk, act=1, post=2, eps=1e-6),
            K.conv_group(cw[2 * G * dk :], v, 2 * G * dk, H, dv, act=1),
        ]
        K.short_conv(proj, groups, s.conv, state.tail, batch.seq_state, batch.row_seq)
        beta_in = proj[:, self.off_beta :]
        if s.channel:
            decay_in = F.linear(proj[:, self.off_decay : self.off_beta], self.w_decay2)
            gate_in = F.linear(proj[:, self.off_gate : self.off_decay], self.w_gate2)
        else:
            decay_in = proj[:, self.off_decay : self.off_beta]
            gate_in = proj[:, self.off_gate : self.off_decay]
        o = K.delta_rule(q, k, v, beta_in, decay_in, self.a_log, self.dt_bias, state.matrices, batch.seq_state, H, G, dk, dv, s.channel,
                         max_rows=batch.max_q_len)
        y = K.gated_rms_heads(o, gate_in, self.norm, H, dv, K.GATE_SIGMOID if s.channel else K.GATE_SILU, self.eps)
        return F.linear(y, self.w_o)
