"""Configuration of Lerorax models: the ``config.json`` reader and its mapping onto the framework's configs.

``config.json`` keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.bigram`` (``buckets``, ``mul_prev``,
``mul_cur``; absent: no bigram table) and ``layers``: a list whose entries carry ``type`` (``parallel`` | ``mingru``), the
mixer's sizes under ``mixer`` and the feed-forward under ``mlp`` (``null``: none; ``kind`` ``dense`` with ``ff`` and
``limit``).  An entry with ``weights_of: j`` owns no tensors: it runs layer ``j``'s modules with a cache / state of its own.

* ``parallel``: ``mixer.left`` = attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` taps, ``scale``, ``rot`` with
  ``dims``, ``base`` and optionally ``scaling`` = ``factor / low / high / original``); ``mixer.right`` = delta memory
  (``heads``, ``dim``).  The rank of the right mixer's low-rank decay projection is read from the tensor shapes by the loader
  (``decay_rank``).
* ``mingru``: ``mixer.width``.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from ...config.transformer_config import TransformerConfig
from ...transformer.mlp import ClampedGLU

MIXER_TYPES = ("parallel", "mingru")
DEFAULT_DECAY_RANK = 16


@dataclass
class LeroraxLayerConfig:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]] = None
    weights_of: Optional[int] = None


@dataclass
class LeroraxConfig:
    vocab: int
    width: int
    layers: List[LeroraxLayerConfig]
    norm_eps: float = 1e-5
    bigram: Optional[Dict[str, int]] = None
    architecture: str = "Lerorax"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LeroraxConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if l.get("mlp") and l["mlp"].get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown mlp kind {l['mlp'].get('kind')!r}")
            src = l.get("weights_of")
            layers.append(LeroraxLayerConfig(l["type"], dict(l["mixer"]), dict(l["mlp"]) if l.get("mlp") else None,
                                             None if src is None else int(src)))
        cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), layers=layers,
                  norm_eps=float((d.get("norm") or {}).get("eps", 1e-5)),
                  bigram=dict((d.get("embedding") or {}).get("bigram") or {}) or None,
                  architecture=d.get("architecture", "Lerorax"))
        for i in range(len(layers)):
            j = cfg.owner(i)
            if layers[j].type != layers[i].type:
                raise ValueError(f"layer {i}: weights_of names a layer of another type")
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "LeroraxConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def owner(self, i: int) -> int:
        """The layer whose tensors layer ``i`` uses (itself unless ``weights_of`` says otherwise)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen or not 0 <= self.layers[i].weights_of < len(self.layers):
                raise ValueError(f"layer {i}: weights_of does not lead to a layer with tensors")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    def owners(self) -> List[int]:
        """Indices of the layers that own tensors, in order."""
        return [i for i, l in enumerate(self.layers) if l.weights_of is None]

    # -- mapping onto the framework's TransformerConfig ---------------------------------------------------------------------
    def base_transformer_config(self, params_dtype=torch.bfloat16, use_cpu_initialization: Optional[bool] = None,
                                perform_initialization: bool = True, **overrides) -> TransformerConfig:
        cpu = (not torch.cuda.is_available()) if use_cpu_initialization is None else use_cpu_initialization
        kw = dict(num_layers=len(self.layers), hidden_size=self.width, num_attention_heads=1, kv_channels=self.width,
                  ffn_hidden_size=self.width, normalization="RMSNorm", layernorm_epsilon=self.norm_eps, add_bias_linear=False,
                  gated_linear_unit=True, activation_func=ClampedGLU(1.0), hidden_dropout=0.0, attention_dropout=0.0,
                  params_dtype=params_dtype, bf16=params_dtype == torch.bfloat16, fp16=params_dtype == torch.float16,
                  fp32_residual_connection=True, use_cpu_initialization=cpu, perform_initialization=perform_initialization,
                  bias_activation_fusion=False)
        kw.update(overrides)
        return TransformerConfig(**kw)

    @staticmethod
    def mlp_transformer_config(base: TransformerConfig, mlp: Dict[str, Any]) -> TransformerConfig:
        return dataclasses.replace(base, ffn_hidden_size=int(mlp["ff"]), num_moe_experts=None, gated_linear_unit=True,
                                   activation_func=ClampedGLU(float(mlp["limit"])))
