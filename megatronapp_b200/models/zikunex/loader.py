"""Weight loading for Zikunex models: a dependency-free safetensors reader and the mapping from checkpoint tensor names
to the modules' (fused) parameters.

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.<name>``, ``l<i>.mlp.<name>``.  Linear weights are stored ``[out, in]`` like the framework's linears, so a
mapping is a copy into a (row slice of a) parameter:

* latent attention: ``dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o``;
* channel_delta: ``q, k, v, a1, g1, b`` are the row segments of the fused ``in_proj``; ``q.conv, k.conv, v.conv`` those of
  the convolution; ``a2, g2, A_log, dt_bias, norm, o``;
* mlstm: ``q, k, v, g, i, f`` are the segments of ``in_proj``; ``i.b, f.b, norm, o``;
* feed-forward: ``up, down`` (dense); ``router``, ``e<j>.up / e<j>.down`` (rows ``j`` of the grouped expert weights) and
  ``shared.up / shared.down`` (MoE).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Tuple

import torch

_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64, "I32": torch.int32,
           "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}


def read_safetensors_header(path: str) -> Tuple[Dict[str, dict], int]:
    """``(name -> {dtype, shape, data_offsets}, offset of the data section)``."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
    meta.pop("__metadata__", None)
    return meta, 8 + n


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of a safetensors file (8-byte little-endian header length, JSON header, raw little-endian data)."""
    meta, base = read_safetensors_header(path)
    out = {}
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        for name, m in meta.items():
            a, b = m["data_offsets"]
            dt = _DTYPES[m["dtype"]]
            if b == a:
                out[name] = torch.empty(m["shape"], dtype=dt)
                continue
            out[name] = torch.frombuffer(bytearray(mm[base + a:base + b]), dtype=dt).reshape(m["shape"])
        mm.close()
    return out


def shapes_into_config(config: dict, shapes: Dict[str, list]) -> dict:
    """Fill the sizes ``config.json`` leaves to the tensor shapes into the mixer dicts: always the low-rank decay / gate
    widths of ``channel_delta``; the latent ranks and the number of convolution taps only where the file omits them."""
    def dim(i, name, axis):
        t = shapes.get(f"l{i}.mix.{name}")
        return None if t is None else int(t[axis])

    for i, l in enumerate(config["layers"]):
        mx = l["mixer"]
        if l["type"] == "channel_delta":
            for key, name in (("decay_rank", "a1"), ("gate_rank", "g1")):
                if dim(i, name, 0) is not None:
                    mx[key] = dim(i, name, 0)
            if "conv" not in mx and dim(i, "q.conv", 1) is not None:
                mx["conv"] = dim(i, "q.conv", 1)
        elif l["type"] == "latent_attention":
            if "q_rank" not in mx and dim(i, "dq", 0) is not None:
                mx["q_rank"] = dim(i, "dq", 0)
            if "kv_rank" not in mx and dim(i, "uk", 1) is not None:
                mx["kv_rank"] = dim(i, "uk", 1)
    return config


def _copy(param: torch.Tensor, src: torch.Tensor, name: str, rows: Tuple[int, int] = None):
    dst = param.data if rows is None else param.data[rows[0]:rows[1]]
    if tuple(dst.shape) != tuple(src.shape):
        raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} does not fit parameter shape {tuple(dst.shape)}")
    dst.copy_(src.to(dst.dtype))


def load_zikunex_weights(model, tensors: Dict[str, torch.Tensor], strict: bool = True):
    """Copy checkpoint tensors into ``model`` (a ``ZikunexModel`` on a single tensor-parallel rank).  A tensor the model
    needs must be there; tensors the model has no parameter for raise under ``strict`` and are returned otherwise."""
    used = set()

    def take(name):
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        used.add(name)
        return tensors[name]

    def segments(param, pre, segs, suffix=""):
        o = 0
        for seg, n in segs:
            _copy(param, take(f"{pre}{seg}{suffix}"), f"{pre}{seg}{suffix}", (o, o + n))
            o += n

    _copy(model.embedding.word_embeddings.weight, take("embed"), "embed")
    _copy(model.output_layer.weight, take("head"), "head")
    _copy(model.decoder.final_layernorm.weight, take("final.norm"), "final.norm")
    for i, layer in enumerate(model.decoder.layers):
        kind, mixer, p = model.zcfg.layers[i].type, layer.mixer, f"l{i}.mix."
        _copy(layer.input_layernorm.weight, take(f"l{i}.norm1"), f"l{i}.norm1")
        if kind == "latent_attention":
            pairs = [("dq", mixer.linear_q_down_proj.weight), ("dq.norm", mixer.q_layernorm.weight), ("uq", mixer.linear_q_up_proj.weight),
                     ("uk", mixer.linear_k_up_proj.weight), ("uv", mixer.linear_v_up_proj.weight), ("o", mixer.linear_proj.weight)]
            if mixer.linear_kv_down_proj is not None:
                pairs += [("dkv", mixer.linear_kv_down_proj.weight), ("dkv.norm", mixer.kv_layernorm.weight)]
            for n, prm in pairs:
                _copy(prm, take(p + n), p + n)
        elif kind == "channel_delta":
            segments(mixer.in_proj.weight, p, mixer.segments())
            segments(mixer.conv_weight, p, mixer.segments()[:3], ".conv")
            for n, prm in (("a2", mixer.decay_up.weight), ("g2", mixer.gate_up.weight), ("A_log", mixer.A_log),
                           ("dt_bias", mixer.dt_bias), ("norm", mixer.norm_weight), ("o", mixer.out_proj.weight)):
                _copy(prm, take(p + n), p + n)
        else:
            segments(mixer.in_proj.weight, p, mixer.segments())
            for n, prm in (("i.b", mixer.igate_bias), ("f.b", mixer.fgate_bias), ("norm", mixer.norm_weight),
                           ("o", mixer.out_proj.weight)):
                _copy(prm, take(p + n), p + n)
        mlp, m = layer.mlp, f"l{i}.mlp."
        if mlp is None:
            continue
        _copy(layer.pre_mlp_layernorm.weight, take(f"l{i}.norm2"), f"l{i}.norm2")
        if model.zcfg.layers[i].mlp["kind"] == "dense":
            _copy(mlp.linear_fc1.weight, take(m + "up"), m + "up")
            _copy(mlp.linear_fc2.weight, take(m + "down"), m + "down")
            continue
        _copy(mlp.router.weight, take(m + "router"), m + "router")
        ex, h = mlp.experts, model.config.hidden_size
        for e in range(ex.num_local_experts):
            _copy(ex.weight1, take(f"{m}e{e}.up"), f"{m}e{e}.up", (e * ex.fc1_out, (e + 1) * ex.fc1_out))
            _copy(ex.weight2, take(f"{m}e{e}.down"), f"{m}e{e}.down", (e * h, (e + 1) * h))
        if mlp.shared_experts is not None:
            _copy(mlp.shared_experts.linear_fc1.weight, take(m + "shared.up"), m + "shared.up")
            _copy(mlp.shared_experts.linear_fc2.weight, take(m + "shared.down"), m + "shared.down")
    extra = sorted(set(tensors) - used)
    if extra and strict:
        raise ValueError(f"checkpoint tensors without a parameter: {extra[:8]}{' ...' if len(extra) > 8 else ''}")
    return extra


def load_model_dir(path: str, params_dtype=torch.bfloat16, device=None, **config_overrides):
    """Build a ``ZikunexModel`` from a folder with ``config.json`` (+ ``model.safetensors``: without it the weights stay
    at their random initialisation) and move it to ``device``."""
    from ...parallel import state as ps
    from .config import ZikunexConfig
    from .model import ZikunexModel

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
    zcfg = ZikunexConfig.from_dict(raw)
    base = zcfg.base_transformer_config(params_dtype, use_cpu_initialization=True, perform_initialization=tensors is None,
                                        **config_overrides)
    model = ZikunexModel(zcfg, base)
    if tensors is not None:
        extra = load_zikunex_weights(model, tensors, strict=False)
        if extra:
            import sys

            print(f"[zikunex] {len(extra)} checkpoint tensors have no parameter and were ignored: {extra[:4]}", file=sys.stderr)
    if device is not None:
        model = model.to(device)
    return model.eval()
