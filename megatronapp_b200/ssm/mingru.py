"""minGRU mixer: a per-channel gated recurrence whose gates do not depend on the previous state, which makes it a linear scan.

    z = sigmoid(W_z h + b_z);  u = W_x h + b_x;  c = u + 1/2 where u >= 0, sigmoid(u) elsewhere
    S <- (1 - z) S + z c;  y = W_o (S * silu(W_g h))

Feng et al., "Were RNNs All We Needed?" (the candidate's activation is the positive function used there for the
log-space form).  One fused input projection with the row segments ``[z | x | g]``; the state (one fp32 value per channel
and sequence) lives in the inference context; gates, candidate and state are fp32.
"""
from __future__ import annotations

import torch

from ..ops import seqmix
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear
from ..transformer.module import MegatronModule
from .gated_delta import packed_tokens, unpacked_tokens


class MinGRUMixer(MegatronModule):
    def __init__(self, config, layer_number: int, width: int):
        super().__init__(config)
        self.layer_number, self.width = layer_number, int(width)
        self.in_proj = ColumnParallelLinear(config.hidden_size, 3 * self.width, config=config, init_method=config.init_method,
                                            bias=True, skip_bias_add=False, gather_output=False)
        self.out_proj = RowParallelLinear(self.width, config.hidden_size, config=config, init_method=config.output_layer_init_method,
                                          bias=False, input_is_parallel=True, skip_bias_add=True)

    def segments(self):
        """Row counts of the ``[z | x | g]`` segments of ``in_proj``."""
        return [("z", self.width), ("x", self.width), ("g", self.width)]

    def forward(self, hidden_states, inference_context=None, cache_index=None, **_):
        s, b = hidden_states.shape[0], hidden_states.shape[1]
        key = self.layer_number if cache_index is None else cache_index
        proj, _ = self.in_proj(hidden_states)
        proj = packed_tokens(proj)
        z_pre, u_pre, g_pre = torch.split(proj, [self.width] * 3, dim=-1)
        if inference_context is not None:
            if inference_context.is_static_batching():
                raise NotImplementedError("recurrent mixers serve through the dynamic engine")
            pb = inference_context.packed
            state = inference_context.recurrent_state(("mingru.S", key), (self.width,), torch.float32)
        else:
            pb = seqmix.PackedBatch.dense(s, b, proj.device)
            state = torch.zeros(b, self.width, dtype=torch.float32, device=proj.device)
        y = seqmix.mingru_scan(z_pre, u_pre, g_pre, pb, state)
        return self.out_proj(unpacked_tokens(y, s, b))
