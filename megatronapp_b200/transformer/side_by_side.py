"""Two sequence mixers side by side on the same input.  Each output is RMS-normed over the model width with its own
plain weight and the layer's result is half their sum; the norms and the mean are left to the layer's output norm
(``norms.OutputRMSNormAdd`` takes the ``BranchPair`` returned here and does all of it in one kernel)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .module import MegatronModule
from .norms import BranchPair


class SideBySideMixer(MegatronModule):
    def __init__(self, config, layer_number: int, left: nn.Module, right: nn.Module):
        super().__init__(config)
        self.layer_number = layer_number
        self.left, self.right = left, right
        dev = "cpu" if (config.use_cpu_initialization or not torch.cuda.is_available()) else torch.cuda.current_device()
        self.left_out_weight = nn.Parameter(torch.ones(config.hidden_size, dtype=config.params_dtype, device=dev))
        self.right_out_weight = nn.Parameter(torch.ones(config.hidden_size, dtype=config.params_dtype, device=dev))

    def forward(self, hidden_states, inference_context=None, cache_index=None, **kw):
        a, bias_a = self.left(hidden_states, inference_context=inference_context, cache_index=cache_index, **kw)
        b, bias_b = self.right(hidden_states, inference_context=inference_context, cache_index=cache_index, **kw)
        if bias_a is not None:
            a = a + bias_a
        if bias_b is not None:
            b = b + bias_b
        return BranchPair(a, b, self.left_out_weight, self.right_out_weight), None
