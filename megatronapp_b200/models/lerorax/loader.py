"""Weight loading for Lerorax models: the mapping from checkpoint tensor names to the modules' (fused) parameters.

Checkpoint names: ``embed``, ``bigram``, ``head``, ``final.norm``, and for every layer that owns tensors ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.<name>``, ``l<i>.mlp.<name>``.  Linear weights are stored ``[out, in]`` like the framework's
linears, so a mapping is a copy into a (row slice of a) parameter:

* ``parallel``, left: ``left.q, left.k, left.v, left.g`` (+ ``.b`` for q / k / v) are the row segments of the fused
  ``in_proj`` (and of its bias; the gate's part stays zero); ``left.q.conv, left.k.conv, left.v.conv`` those of the
  convolution; ``left.q.norm, left.k.norm, left.talk, left.o``;
* ``parallel``, right: ``right.r, right.k, right.v, right.g, right.a, right.w1`` are the segments of ``in_proj``
  (``right.a.b`` its only bias rows); ``right.w2, right.w0, right.norm, right.o``;
* ``left.out / right.out``: the branch norms of the side-by-side mixer;
* ``mingru``: ``z, x, g`` (+ ``z.b, x.b``) the segments of ``in_proj``; ``o``;
* feed-forward: ``gate`` and ``up`` are the two halves of ``linear_fc1``, ``down`` is ``linear_fc2``.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..zikunex.loader import _copy, read_safetensors, read_safetensors_header


def shapes_into_config(config: dict, shapes: Dict[str, list]) -> dict:
    """Fill the sizes ``config.json`` leaves to the tensor shapes into the mixer dicts: the rank of the right mixer's
    low-rank decay projection, and the number of convolution taps where the file omits it."""
    for i, l in enumerate(config["layers"]):
        j = i
        while config["layers"][j].get("weights_of") is not None:
            j = config["layers"][j]["weights_of"]
        if l["type"] != "parallel":
            continue
        w1 = shapes.get(f"l{j}.mix.right.w1")
        if w1 is not None:
            l["mixer"]["right"]["decay_rank"] = int(w1[0])
        conv = shapes.get(f"l{j}.mix.left.q.conv")
        if conv is not None and "conv" not in l["mixer"]["left"]:
            l["mixer"]["left"]["conv"] = int(conv[1])
    return config


def load_lerorax_weights(model, tensors: Dict[str, torch.Tensor], strict: bool = True):
    """Copy checkpoint tensors into ``model`` (a ``LeroraxModel`` on a single tensor-parallel rank).  A tensor the model
    needs must be there; tensors the model has no parameter for raise under ``strict`` and are returned otherwise."""
    used = set()

    def take(name):
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        used.add(name)
        return tensors[name]

    def segments(param, pre, segs, suffix="", only=None):
        o = 0
        for seg, n in segs:
            if only is None or seg in only:
                _copy(param, take(f"{pre}{seg}{suffix}"), f"{pre}{seg}{suffix}", (o, o + n))
            o += n

    _copy(model.embedding.word_embeddings.weight, take("embed"), "embed")
    if model.bigram_embedding is not None:
        _copy(model.bigram_embedding.weight, take("bigram"), "bigram")
    _copy(model.output_layer.weight, take("head"), "head")
    _copy(model.decoder.final_layernorm.weight, take("final.norm"), "final.norm")
    for layer, i in zip(model.decoder.layers, model.lcfg.owners()):
        kind, mixer, p = model.lcfg.layers[i].type, layer.mixer, f"l{i}.mix."
        _copy(layer.mixer_norm.weight, take(f"l{i}.norm1"), f"l{i}.norm1")
        if kind == "mingru":
            segments(mixer.in_proj.weight, p, mixer.segments())
            mixer.in_proj.bias.data.zero_()
            segments(mixer.in_proj.bias, p, mixer.segments(), ".b", only=("z", "x"))
            _copy(mixer.out_proj.weight, take(p + "o"), p + "o")
        else:
            a, r = mixer.left, mixer.right
            segments(a.in_proj.weight, p + "left.", a.segments())
            a.in_proj.bias.data.zero_()
            segments(a.in_proj.bias, p + "left.", a.segments(), ".b", only=("q", "k", "v"))
            segments(a.conv_weight, p + "left.", a.segments()[:3], ".conv")
            for n, prm in (("q.norm", a.q_norm_weight), ("k.norm", a.k_norm_weight), ("talk", a.talk), ("o", a.out_proj.weight)):
                _copy(prm, take(p + "left." + n), p + "left." + n)
            segments(r.in_proj.weight, p + "right.", r.segments())
            r.in_proj.bias.data.zero_()
            segments(r.in_proj.bias, p + "right.", r.segments(), ".b", only=("a",))
            for n, prm in (("w2", r.decay_up.weight), ("w0", r.decay_bias), ("norm", r.norm_weight), ("o", r.out_proj.weight)):
                _copy(prm, take(p + "right." + n), p + "right." + n)
            _copy(mixer.left_out_weight, take(p + "left.out"), p + "left.out")
            _copy(mixer.right_out_weight, take(p + "right.out"), p + "right.out")
        if layer.mlp is None:
            continue
        m = f"l{i}.mlp."
        _copy(layer.mlp_norm.weight, take(f"l{i}.norm2"), f"l{i}.norm2")
        ff = layer.mlp.linear_fc2.weight.shape[1]
        _copy(layer.mlp.linear_fc1.weight, take(m + "gate"), m + "gate", (0, ff))
        _copy(layer.mlp.linear_fc1.weight, take(m + "up"), m + "up", (ff, 2 * ff))
        _copy(layer.mlp.linear_fc2.weight, take(m + "down"), m + "down")
    extra = sorted(set(tensors) - used)
    if extra and strict:
        raise ValueError(f"checkpoint tensors without a parameter: {extra[:8]}{' ...' if len(extra) > 8 else ''}")
    return extra


def load_model_dir(path: str, params_dtype=torch.bfloat16, device=None, **config_overrides):
    """Build a ``LeroraxModel`` from a folder with ``config.json`` (+ ``model.safetensors``: without it the weights stay
    at their random initialisation) and move it to ``device``."""
    from ...parallel import state as ps
    from .config import LeroraxConfig
    from .model import LeroraxModel

    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    with open(os.path.join(path, "config.json")) as f:
        raw = json.load(f)
    st = os.path.join(path, "model.safetensors")
    tensors = None
    if os.path.exists(st):
        meta, _ = read_safetensors_header(st)
        raw = shapes_into_config(raw, {k: v["shape"] for k, v in meta.items()})
        tensors = read_safetensors(st)
    lcfg = LeroraxConfig.from_dict(raw)
    base = lcfg.base_transformer_config(params_dtype, use_cpu_initialization=True, perform_initialization=tensors is None,
                                        **config_overrides)
    model = LeroraxModel(lcfg, base)
    if tensors is not None:
        extra = load_lerorax_weights(model, tensors, strict=False)
        if extra:
            import sys

            print(f"[lerorax] {len(extra)} checkpoint tensors have no parameter and were ignored: {extra[:4]}", file=sys.stderr)
    if device is not None:
        model = model.to(device)
    return model.eval()
