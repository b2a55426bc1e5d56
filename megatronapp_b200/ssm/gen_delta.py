"""Generalized delta-rule mixer: a matrix memory with one decay and one removal rate per head and key channel.

Per head a memory ``S [d, dv]`` is carried from token to token; with the unit key ``u = k / sqrt(sum k^2 + unit_eps)``::

    w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 h) + w_0))        decay per key channel, in (exp(-decay_scale), 1)
    a = sigmoid(W_a h + b_a)                                         removal rate per key channel
    S <- diag(w) S - (a * u) (u^T S) + k v^T                         decay and removal both act on the previous S
    o = S^T r

The read-out is RMS-normalised head by head, scaled by one weight vector over all heads' channels, gated by
``sigmoid(W_g h)`` and projected out.  Formulation: Peng et al., "RWKV-7 'Goose' with Expressive Dynamic State Evolution".

Shape as the framework's other recurrent mixers (``ssm/gated_delta.py``): one fused input projection with the row
segments ``[r | k | v | g | a | w1]``, the low-rank decay up-projection, fp32 state in the inference context, row-parallel
output projection.  Decays, rates, unit keys and the state are fp32 (made inside the scan kernel from the projections).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import seqmix
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ..transformer.module import MegatronModule
from .gated_delta import packed_tokens, unpacked_tokens


class GeneralizedDeltaMixer(MegatronModule):
    def __init__(self, config, layer_number: int, num_heads: int, qk_dim: int, v_dim: int, decay_rank: int,
                 decay_scale: float = math.exp(-0.5), eps: float = None, unit_eps: float = 1e-6):
        super().__init__(config)
        self.layer_number = layer_number
        self.nh, self.d, self.dv, self.decay_rank = num_heads, qk_dim, v_dim, decay_rank
        self.decay_scale, self.unit_eps = float(decay_scale), float(unit_eps)
        self.eps = config.layernorm_epsilon if eps is None else eps
        self.k_ch, self.v_ch = num_heads * qk_dim, num_heads * v_dim
        col = dict(config=config, init_method=config.init_method, skip_bias_add=False, gather_output=False)
        self.in_proj = ColumnParallelLinear(config.hidden_size, 3 * self.k_ch + 2 * self.v_ch + decay_rank, bias=True, **col)
        self.decay_up = ColumnParallelLinear(decay_rank, self.k_ch, bias=False, **col)
        dev, dt_ = self.in_proj.weight.device, config.params_dtype
        self.decay_bias = nn.Parameter(torch.zeros(self.k_ch, device=dev, dtype=dt_))
        self.norm_weight = nn.Parameter(torch.ones(self.v_ch, device=dev, dtype=dt_))
        self.out_proj = RowParallelLinear(self.v_ch, config.hidden_size, config=config, init_method=config.output_layer_init_method,
                                          bias=False, input_is_parallel=True, skip_bias_add=True)
        self.decay_bias._no_weight_decay = True

    def segments(self):
        """Row counts of the ``[r | k | v | g | a | w1]`` segments of ``in_proj``."""
        return [("r", self.k_ch), ("k", self.k_ch), ("v", self.v_ch), ("g", self.v_ch), ("a", self.k_ch), ("w1", self.decay_rank)]

    def forward(self, hidden_states, inference_context=None, cache_index=None, **_):
        s, b = hidden_states.shape[0], hidden_states.shape[1]
        key = self.layer_number if cache_index is None else cache_index
        proj, _ = self.in_proj(hidden_states)
        proj = packed_tokens(proj)
        T = proj.shape[0]
        r, k, v, gate, a_pre, w1 = torch.split(proj, [n for _, n in self.segments()], dim=-1)
        if inference_context is not None:
            if inference_context.is_static_batching():
                raise NotImplementedError("recurrent mixers serve through the dynamic engine")
            pb = inference_context.packed
            state = inference_context.recurrent_state(("gdelta.S", key), (self.nh, self.d, self.dv), torch.float32)
        else:
            pb = seqmix.PackedBatch.dense(s, b, proj.device)
            state = torch.zeros(b, self.nh, self.d, self.dv, dtype=torch.float32, device=proj.device)
        w_pre, _ = self.decay_up(torch.tanh(w1))
        o = seqmix.gen_delta_scan(r.reshape(T, self.nh, self.d), k.reshape(T, self.nh, self.d), v.reshape(T, self.nh, self.dv),
                                  w_pre, a_pre, self.decay_bias, pb, state, self.decay_scale, self.unit_eps)
        y = seqmix.gated_head_rms_norm(o, self.norm_weight, gate, self.eps, proj.dtype)
        return self.out_proj(unpacked_tokens(y, s, b))
