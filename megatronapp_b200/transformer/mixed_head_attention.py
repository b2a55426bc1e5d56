"""Grouped-query softmax attention whose weights are mixed across heads, with a short convolution on q / k / v, one RMS norm
across all heads' channels of q (and one of k), partial interleaved rotary positions and a sigmoid output gate.

Per token, from the mixer input ``h``::

    q, k, v = conv(W_q h + b_q), conv(W_k h + b_k), conv(W_v h + b_v)      causal depth-wise convolution over time, no activation
    q, k    = rms_norm(q) * w_q, rms_norm(k) * w_k                          over all heads of the projection at once
    q, k    = rotate the first rot_dims dimensions of every head            pair (2i, 2i + 1), angle position * f_i
    P_g     = softmax_j(q_g . k_kv(g)(j) * scale), j <= i
    M_h     = sum_g talk[h, g] P_g                                          head mixing, after the softmax
    o_h     = sum_j M_h(j) v_kv(h)(j);   y = W_o (concat(o) * sigmoid(W_g h))

Head mixing after the softmax: Shazeer et al., "Talking-Heads Attention".

The module follows the framework's recurrent mixers in shape: one fused input projection with the row segments
``[q | k | v | g]``, one convolution over the ``[q | k | v]`` channels whose window (the last ``taps - 1`` projected rows of
a sequence) lives in the inference context's per-request state, keys (normed, rotated) and values (convolved) in the
paged cache, and a row-parallel output projection.  Angles, norm statistics, scores, weights and the mixture are fp32.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..models.common.embeddings import llama3_scaled_frequencies
from ..ops import seqmix
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ..ssm.gated_delta import packed_tokens, unpacked_tokens
from .module import MegatronModule


def dense_pages(seq_len: int, batch: int, device):
    """Page table, sequence index and visible length of every token for ``batch`` whole sequences stored one after
    another (each sequence is one page of ``seq_len`` slots): lets the paged kernels run without a cache manager."""
    table = torch.arange(batch, dtype=torch.int32, device=device).view(batch, 1)
    tok_req = torch.arange(batch, dtype=torch.int32, device=device).repeat_interleave(seq_len)
    tok_len = torch.arange(1, seq_len + 1, dtype=torch.int32, device=device).repeat(batch)
    return table, tok_req, tok_len


class MixedHeadAttention(MegatronModule):
    def __init__(self, config, layer_number: int, num_heads: int, num_kv_heads: int, qk_dim: int, v_dim: int,
                 softmax_scale: float, conv_taps: int = 1, rot_dims: int = 0, rot_base: float = 10000.0,
                 rot_scaling: Optional[dict] = None, head_mixing: bool = True, eps: Optional[float] = None):
        super().__init__(config)
        if num_heads % num_kv_heads:
            raise ValueError("mixed-head attention: heads must be a multiple of kv_heads")
        if rot_dims % 2 or rot_dims > qk_dim:
            raise ValueError("mixed-head attention: rot_dims must be even and at most the head dimension")
        self.layer_number = layer_number
        self.nh, self.nkv, self.d, self.dv, self.taps = num_heads, num_kv_heads, qk_dim, v_dim, max(1, int(conv_taps))
        self.rot_dims, self.softmax_scale = int(rot_dims), float(softmax_scale)
        self.eps = config.layernorm_epsilon if eps is None else eps
        self.q_ch, self.k_ch, self.v_ch, self.o_ch = num_heads * qk_dim, num_kv_heads * qk_dim, num_kv_heads * v_dim, num_heads * v_dim
        self.conv_ch = self.q_ch + self.k_ch + self.v_ch
        self.in_proj = ColumnParallelLinear(config.hidden_size, self.conv_ch + self.o_ch, config=config, init_method=config.init_method,
                                            bias=True, skip_bias_add=False, gather_output=False)
        dev, dt_ = self.in_proj.weight.device, config.params_dtype
        self.conv_weight = nn.Parameter(torch.randn(self.conv_ch, self.taps, device=dev).mul_(self.taps ** -0.5).to(dt_))
        self.q_norm_weight = nn.Parameter(torch.ones(self.q_ch, device=dev, dtype=dt_))
        self.k_norm_weight = nn.Parameter(torch.ones(self.k_ch, device=dev, dtype=dt_))
        self.talk = nn.Parameter(torch.eye(num_heads, device=dev, dtype=dt_)) if head_mixing else None
        self.register_buffer("inv_freq", llama3_scaled_frequencies(self.rot_dims, rot_base, rot_scaling).to(dev)
                             if self.rot_dims else torch.zeros(0, device=dev), persistent=False)
        self.out_proj = RowParallelLinear(self.o_ch, config.hidden_size, config=config, init_method=config.output_layer_init_method,
                                          bias=False, input_is_parallel=True, skip_bias_add=True)

    def segments(self):
        """Row counts of the ``[q | k | v | g]`` segments of ``in_proj``."""
        return [("q", self.q_ch), ("k", self.k_ch), ("v", self.v_ch), ("g", self.o_ch)]

    def forward(self, hidden_states, inference_context=None, cache_index=None, **_):
        s, b = hidden_states.shape[0], hidden_states.shape[1]
        key = self.layer_number if cache_index is None else cache_index
        proj, _ = self.in_proj(hidden_states)
        proj = packed_tokens(proj)                                                     # [T, q | k | v | g]
        T = proj.shape[0]
        qkv, gate = proj[:, :self.conv_ch], proj[:, self.conv_ch:]
        ctx = inference_context
        if ctx is not None:
            if ctx.is_static_batching():
                raise NotImplementedError("mixed-head attention serves through the dynamic (paged) engine")
            pb, positions = ctx.packed, ctx.positions
            window = ctx.recurrent_state(("mixattn.conv", key), (self.taps - 1, self.conv_ch), proj.dtype)
        else:
            pb = seqmix.PackedBatch.dense(s, b, proj.device)
            positions = torch.arange(s, device=proj.device).repeat(b)
            window = proj.new_zeros(b, self.taps - 1, self.conv_ch)
        y = seqmix.causal_conv(qkv, self.conv_weight, pb, window)
        q, k = seqmix.norm_rope(y[:, :self.q_ch], y[:, self.q_ch:self.q_ch + self.k_ch], self.q_norm_weight, self.k_norm_weight,
                                positions, self.inv_freq, self.d, self.rot_dims, self.eps)
        q, k = q.view(T, self.nh, self.d), k.view(T, self.nkv, self.d)
        v = y[:, self.q_ch + self.k_ch:].reshape(T, self.nkv, self.dv)
        talk = None if self.talk is None else self.talk.float()
        if ctx is not None:
            o = ctx.attend_mixed(key, q, k, v, self.softmax_scale, talk, gate)
        else:
            table, tok_req, tok_len = dense_pages(s, b, proj.device)
            o = seqmix.mixed_attention_paged(q, k.contiguous(), v.contiguous(), table, tok_req, tok_len, s, self.softmax_scale,
                                             talk, gate, s)
        return self.out_proj(unpacked_tokens(o, s, b))
