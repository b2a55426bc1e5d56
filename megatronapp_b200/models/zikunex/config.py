"""Configuration of Zikunex models: the ``config.json`` reader and its mapping onto the framework's configs.

``config.json`` keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``: a list
whose entries carry ``type`` (``latent_attention`` | ``channel_delta`` | ``mlstm``), the mixer's sizes under ``mixer``
and the feed-forward under ``mlp`` (``null``: none; ``kind`` ``dense`` with ``ff``; ``kind`` ``moe`` with ``expert.ff``,
``router.experts / top / groups.count / groups.keep`` and optionally ``shared.ff``).  Sizes that the file does not give
(the ranks of the low-rank decay and gate projections of ``channel_delta``) are read from the tensor shapes by the
loader, which stores them in the mixer's dict as ``decay_rank`` / ``gate_rank``.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from ...config.transformer_config import TransformerConfig
from ...transformer.mlp import squared_relu

MIXER_TYPES = ("latent_attention", "channel_delta", "mlstm")


@dataclass
class ZikunexLayerConfig:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]] = None


@dataclass
class ZikunexConfig:
    vocab: int
    width: int
    layers: List[ZikunexLayerConfig]
    norm_eps: float = 1e-5
    embedding_scale: float = 1.0
    architecture: str = "Zikunex"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ZikunexConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            layers.append(ZikunexLayerConfig(l["type"], dict(l["mixer"]), dict(l["mlp"]) if l.get("mlp") else None))
        for i, l in enumerate(layers):
            src = l.mixer.get("kv_from")
            if src is not None:
                if not (0 <= src < i) or layers[src].type != "latent_attention" or layers[src].mixer.get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier latent_attention layer that owns its latents")
                if layers[src].mixer["kv_rank"] != l.mixer["kv_rank"]:
                    raise ValueError(f"layer {i}: kv_rank differs from that of layer {src}")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), layers=layers,
                   norm_eps=float((d.get("norm") or {}).get("eps", 1e-5)),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   architecture=d.get("architecture", "Zikunex"))

    @classmethod
    def from_json(cls, path: str) -> "ZikunexConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    # -- mapping onto the framework's TransformerConfig ---------------------------------------------------------------------
    def base_transformer_config(self, params_dtype=torch.bfloat16, use_cpu_initialization: Optional[bool] = None,
                                perform_initialization: bool = True, **overrides) -> TransformerConfig:
        cpu = (not torch.cuda.is_available()) if use_cpu_initialization is None else use_cpu_initialization
        kw = dict(num_layers=len(self.layers), hidden_size=self.width, num_attention_heads=1, kv_channels=self.width,
                  ffn_hidden_size=self.width, normalization="RMSNorm", layernorm_epsilon=self.norm_eps, add_bias_linear=False,
                  gated_linear_unit=False, activation_func=squared_relu, hidden_dropout=0.0, attention_dropout=0.0,
                  params_dtype=params_dtype, bf16=params_dtype == torch.bfloat16, fp16=params_dtype == torch.float16,
                  fp32_residual_connection=True, use_cpu_initialization=cpu, perform_initialization=perform_initialization,
                  bias_activation_fusion=False)
        kw.update(overrides)
        return TransformerConfig(**kw)

    def mlp_transformer_config(self, base: TransformerConfig, mlp: Dict[str, Any]) -> TransformerConfig:
        """The config a layer's feed-forward is built from: dense width, or the MoE sizes and routing rule."""
        if mlp["kind"] == "dense":
            return dataclasses.replace(base, ffn_hidden_size=int(mlp["ff"]), num_moe_experts=None)
        if mlp["kind"] != "moe":
            raise ValueError(f"unknown mlp kind {mlp['kind']!r}")
        r = mlp["router"]
        groups = r.get("groups") or {"count": 1, "keep": 1}
        shared = mlp.get("shared")
        return dataclasses.replace(
            base, num_moe_experts=int(r["experts"]), moe_router_topk=int(r["top"]), moe_ffn_hidden_size=int(mlp["expert"]["ff"]),
            ffn_hidden_size=int(mlp["expert"]["ff"]), moe_router_num_groups=int(groups["count"]),
            moe_router_group_topk=int(groups["keep"]), moe_router_group_score="max", moe_router_pre_softmax=True,
            moe_router_renormalize=True, moe_router_score_function="softmax", moe_router_dtype="fp32",
            moe_router_load_balancing_type="none", moe_aux_loss_coeff=0.0, moe_token_dispatcher_type="allgather",
            moe_grouped_gemm=True, moe_shared_expert_intermediate_size=int(shared["ff"]) if shared else None)
