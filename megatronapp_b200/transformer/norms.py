"""LayerNorm / RMSNorm / L2Norm modules backed by the fused sm_100a norm kernel.

Parity: reference ``fusions/fused_layer_norm.py:30-169`` (``FusedLayerNorm``, zero-centred gamma,
``sequence_parallel`` attribute on the params) and ``transformer/torch_norm.py:9-96``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class FusedLayerNorm(nn.Module):
    def __init__(self, config, hidden_size: int, eps: float = 1e-5, persist_layer_norm: bool = True,
                 zero_centered_gamma: bool = False, normalization: str = "LayerNorm"):
        super().__init__()
        self.config = config
        self.zero_centered_gamma = config.layernorm_zero_centered_gamma if config is not None else zero_centered_gamma
        self.normalization = config.normalization if config is not None else normalization
        if self.normalization not in ("LayerNorm", "RMSNorm"):
            raise ValueError(f"unsupported normalization {self.normalization}")
        self.eps = eps
        self.hidden_size = hidden_size
        dtype = config.params_dtype if config is not None else torch.float32
        dev = "cpu" if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        init = 0.0 if self.zero_centered_gamma else 1.0
        self.weight = nn.Parameter(torch.full((hidden_size,), init, dtype=dtype, device=dev))
        if self.normalization == "LayerNorm":
            self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=dev))
        else:
            self.register_parameter("bias", None)
        sp = bool(config.sequence_parallel) if config is not None else False
        setattr(self.weight, "sequence_parallel", sp)
        if self.bias is not None:
            setattr(self.bias, "sequence_parallel", sp)

    def forward(self, x):
        return ops.layer_norm(x, self.weight, self.bias, self.eps, rms=self.normalization == "RMSNorm",
                              zero_centered=self.zero_centered_gamma)


WrappedTorchNorm = FusedLayerNorm
LNImpl = FusedLayerNorm


class L2Norm(nn.Module):
    def __init__(self, hidden_size: int = 0, eps: float = 1e-6, **_):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x)


class IdentityOp(nn.Module):
    def __init__(self, *a, **k):
        super().__init__()

    def forward(self, x, *a, **k):
        return x


class IdentityFuncOp(IdentityOp):
    def forward(self, *a, **k):
        return super().forward


class ResidualRMSNorm(nn.Module):
    """RMS norm of an fp32 residual stream, fused with the addition that precedes it: ``forward(x, delta)`` adds
    ``delta`` (any dtype) into the fp32 ``x`` in place and returns ``(x, x / sqrt(mean(x^2) + eps) * weight)`` with the
    normalised copy in ``out_dtype`` (the dtype the following projections run in)."""

    def __init__(self, config, hidden_size: int, eps: float = 1e-5, out_dtype=None, weight_offset: float = 0.0):
        super().__init__()
        self.eps, self.hidden_size = eps, hidden_size
        self.weight_offset = float(weight_offset)     # 1.0: zero-centred weight, applied as 1 + w
        dtype = config.params_dtype if config is not None else torch.float32
        self.out_dtype = out_dtype          # None: the weight's dtype at call time
        dev = "cpu" if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.full((hidden_size,), 1.0 - self.weight_offset, dtype=dtype, device=dev))
        setattr(self.weight, "sequence_parallel", bool(config.sequence_parallel) if config is not None else False)

    def forward(self, x, delta=None):
        from ..ops import seqmix

        shape = x.shape
        x2, y = seqmix.add_rms_norm(x.view(-1, shape[-1]), None if delta is None else delta.reshape(-1, shape[-1]),
                                    self.weight, self.eps, self.out_dtype or self.weight.dtype, self.weight_offset)
        return x2.view(shape), y.view(shape)


class BranchPair:
    """Outputs of two mixers that ran side by side on the same input, with the plain RMS-norm weight of each: the layer's
    result is ``(rms_norm(a) * weight_a + rms_norm(b) * weight_b) / 2``, which ``OutputRMSNormAdd`` computes inside its
    kernel."""

    def __init__(self, a, b, weight_a, weight_b):
        self.a, self.b, self.weight_a, self.weight_b = a, b, weight_a, weight_b


class OutputRMSNormAdd(nn.Module):
    """RMS norm of a sublayer's *output*, fused with the addition to the fp32 residual stream: ``forward(x, out)`` updates
    ``x += rms_norm(out) * (weight_offset + weight)`` in place and returns ``(x, x in out_dtype)``, the copy the next
    sublayer reads.  ``out`` may be a ``BranchPair``.  Statistics and the sum are fp32."""

    def __init__(self, config, hidden_size: int, eps: float = 1e-5, out_dtype=None, weight_offset: float = 0.0):
        super().__init__()
        self.eps, self.hidden_size, self.out_dtype = eps, hidden_size, out_dtype
        self.weight_offset = float(weight_offset)
        dtype = config.params_dtype if config is not None else torch.float32
        dev = "cpu" if (config is None or config.use_cpu_initialization or not torch.cuda.is_available()) \
            else torch.cuda.current_device()
        self.weight = nn.Parameter(torch.full((hidden_size,), 1.0 - self.weight_offset, dtype=dtype, device=dev))
        setattr(self.weight, "sequence_parallel", bool(config.sequence_parallel) if config is not None else False)

    def forward(self, x, out):
        from ..ops import seqmix

        shape, h = x.shape, x.shape[-1]
        dt = self.out_dtype or self.weight.dtype
        if isinstance(out, BranchPair):
            x2, y = seqmix.norm_add(x.view(-1, h), out.a.reshape(-1, h), self.weight, self.eps, dt, self.weight_offset,
                                    out.b.reshape(-1, h), out.weight_a, out.weight_b)
        else:
            x2, y = seqmix.norm_add(x.view(-1, h), out.reshape(-1, h), self.weight, self.eps, dt, self.weight_offset)
        return x2.view(shape), y.view(shape)
