"""mLSTM mixer: a matrix memory with exponential input gate and sigmoid forget gate, kept stable by a running maximum.

Per head, with log gates ``i = cap * tanh((W_i h + b_i) / cap)`` and ``f = logsigmoid(cap * tanh((W_f h + b_f) / cap))``::

    m' = max(f + m, i)
    S <- e^(f + m - m') S + e^(i - m') k v^T          n <- e^(f + m - m') n + e^(i - m') k
    o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)        (q carries the d^-1/2 factor)

All three parts of the state are zero before a sequence's first token (the maximum too: it is not minus infinity).
The read-out is RMS-normalised head by head, the concatenated heads are scaled by one weight vector over all their
channels and gated by ``sigmoid(W_g h)``, then projected out.  As in the framework's
other recurrent mixers one fused input projection produces the segments ``[q | k | v | g | i | f]``, the state lives in
the inference context, and gates, maxima and the memory are fp32.

Matrix-memory formulation: Beck et al., "xLSTM: Extended Long Short-Term Memory".
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import seqmix
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ..transformer.module import MegatronModule
from .gated_delta import packed_tokens, unpacked_tokens


class MLSTMMixer(MegatronModule):
    def __init__(self, config, layer_number: int, num_heads: int, qk_dim: int, v_dim: int, gate_cap: float,
                 eps: float = None, denom_eps: float = 1e-6):
        super().__init__(config)
        self.layer_number = layer_number
        self.nh, self.d, self.dv, self.gate_cap = num_heads, qk_dim, v_dim, float(gate_cap)
        self.eps = config.layernorm_epsilon if eps is None else eps
        self.denom_eps = denom_eps
        self.qk_ch, self.v_ch = num_heads * qk_dim, num_heads * v_dim
        self.in_proj = ColumnParallelLinear(config.hidden_size, 2 * self.qk_ch + 2 * self.v_ch + 2 * num_heads, config=config,
                                            init_method=config.init_method, bias=False, skip_bias_add=False,
                                            gather_output=False)
        dev, dt_ = self.in_proj.weight.device, config.params_dtype
        self.igate_bias = nn.Parameter(torch.zeros(num_heads, device=dev, dtype=dt_))
        self.fgate_bias = nn.Parameter(torch.full((num_heads,), 3.0, device=dev, dtype=dt_))
        self.norm_weight = nn.Parameter(torch.ones(self.v_ch, device=dev, dtype=dt_))
        self.out_proj = RowParallelLinear(self.v_ch, config.hidden_size, config=config,
                                          init_method=config.output_layer_init_method, bias=False, input_is_parallel=True,
                                          skip_bias_add=True)
        for p in (self.igate_bias, self.fgate_bias):
            p._no_weight_decay = True

    def segments(self):
        """Row counts of the ``[q | k | v | g | i | f]`` segments of ``in_proj``."""
        return [("q", self.qk_ch), ("k", self.qk_ch), ("v", self.v_ch), ("g", self.v_ch), ("i", self.nh), ("f", self.nh)]

    def forward(self, hidden_states, inference_context=None, **_):
        s, b = hidden_states.shape[0], hidden_states.shape[1]
        proj, _ = self.in_proj(hidden_states)
        proj = packed_tokens(proj)
        T = proj.shape[0]
        q, k, v, gate, iraw, fraw = torch.split(proj, [self.qk_ch, self.qk_ch, self.v_ch, self.v_ch, self.nh, self.nh], dim=-1)
        cap = self.gate_cap
        log_i = cap * torch.tanh((iraw.float() + self.igate_bias.float()) / cap)
        log_f = F.logsigmoid(cap * torch.tanh((fraw.float() + self.fgate_bias.float()) / cap))
        if inference_context is not None:
            if inference_context.is_static_batching():
                raise NotImplementedError("recurrent mixers serve through the dynamic engine")
            pb = inference_context.packed
            key = self.layer_number
            S = inference_context.recurrent_state(("mlstm.S", key), (self.nh, self.d, self.dv), torch.float32)
            n = inference_context.recurrent_state(("mlstm.n", key), (self.nh, self.d), torch.float32)
            m = inference_context.recurrent_state(("mlstm.m", key), (self.nh,), torch.float32)
        else:
            pb = seqmix.PackedBatch.dense(s, b, proj.device)
            S = torch.zeros(b, self.nh, self.d, self.dv, dtype=torch.float32, device=proj.device)
            n = torch.zeros(b, self.nh, self.d, dtype=torch.float32, device=proj.device)
            m = torch.zeros(b, self.nh, dtype=torch.float32, device=proj.device)
        o = seqmix.mlstm_scan(q.reshape(T, self.nh, self.d), k.reshape(T, self.nh, self.d), v.reshape(T, self.nh, self.dv),
                              log_i, log_f, pb, S, n, m, self.d ** -0.5, self.denom_eps)
        y = seqmix.gated_head_rms_norm(o, self.norm_weight, gate, self.eps, proj.dtype)
        return self.out_proj(unpacked_tokens(y, s, b))
