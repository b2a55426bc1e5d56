"""Lerorax models in the framework against a plain, slow evaluation of the design's equations (``lerorax_oracle``).

Each test builds its own small configuration and random (or hand-made) weights, loads them through the product loader
and drives the model through the dynamic engine -- whole prompts, prompts cut into portions, token-by-token decoding,
mixed batches, reused pages and state rows -- on the CPU (PyTorch op path) and, marked ``gpu``, on the sm_100a kernels.
"""
import copy
import json
import math
import os
import struct
import subprocess

import pytest
import torch

import lerorax_oracle as oracle
from megatronapp_b200.data.tokenizer import NullTokenizer
from megatronapp_b200.inference import DynamicInferenceEngine, SamplingParams
from megatronapp_b200.inference.trace import TraceReplayer
from megatronapp_b200.models.lerorax import LeroraxConfig, LeroraxModel, load_lerorax_weights
from megatronapp_b200.models.lerorax.loader import shapes_into_config
from megatronapp_b200.ops import seqmix
from megatronapp_b200.parallel import state as ps
from megatronapp_b200.transformer.mixed_head_attention import dense_pages

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
VOCAB = 80

ROT = {"base": 5000.0, "dims": 8, "scaling": {"factor": 4.0, "low": 2.0, "high": 8.0, "original": 64}}
LEFT = {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 3, "scale": 0.2, "rot": ROT}
LEFT_B = {"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 8, "conv": 2, "scale": 0.5, "rot": {"base": 100.0, "dims": 8}}      # rotates all
LEFT_C = {"heads": 4, "kv_heads": 1, "dim": 12, "vdim": 20, "conv": 1, "scale": 0.3, "rot": {"base": 10000.0, "dims": 4}}  # one tap
RIGHT = {"heads": 3, "dim": 8}
RIGHT_B = {"heads": 1, "dim": 40}
PAR = {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT}}
PAR_B = {"type": "parallel", "mixer": {"left": LEFT_B, "right": RIGHT_B}}
PAR_C = {"type": "parallel", "mixer": {"left": LEFT_C, "right": RIGHT}}
GRU = {"type": "mingru", "mixer": {"width": 40}}
GRU_B = {"type": "mingru", "mixer": {"width": 7}}
FF = {"kind": "dense", "ff": 56, "limit": 0.8}
FF_B = {"kind": "dense", "ff": 24, "limit": 2.5}


def layer(spec, mlp=None, weights_of=None):
    l = copy.deepcopy(spec)
    l["mlp"] = copy.deepcopy(mlp)
    if weights_of is not None:
        l["weights_of"] = weights_of
    return l


def config_of(layers, width=48, vocab=VOCAB, eps=1e-6, bigram=True):
    cfg = {"architecture": "Lerorax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": 37, "mul_prev": 5, "mul_cur": 3}}
    return cfg


HYBRID = config_of([layer(PAR, FF), layer(GRU, FF_B), layer(PAR_B), layer(PAR, FF, weights_of=0), layer(GRU_B, FF),
                    layer(GRU, FF_B, weights_of=1), layer(PAR_C, FF_B), layer(PAR, FF, weights_of=3)])


def build(cfg, device, dtype=torch.float32, seed=0, weights=None):
    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    W = weights if weights is not None else oracle.random_weights(cfg, seed)
    raw = shapes_into_config(copy.deepcopy(cfg), {k: list(v.shape) for k, v in W.items()})
    lcfg = LeroraxConfig.from_dict(raw)
    model = LeroraxModel(lcfg, lcfg.base_transformer_config(dtype, use_cpu_initialization=True, perform_initialization=False))
    load_lerorax_weights(model, W)
    return model.to(device).eval(), W


def replayer(model, max_tokens=512, block_size=4, max_requests=4):
    return TraceReplayer(model, max_tokens, block_size=block_size, max_requests=max_requests, max_sequence_length=4096)


def run_cut(rp, rid, tokens, cuts):
    """Feed ``tokens`` in portions of the given sizes (the rest one by one); logits of every position."""
    outs, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(tokens) - at)
        outs.append(rp.step([{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}]))
        at += n
    rp.step([], end=[rid])
    return torch.cat(outs)


def tokens_of(n, vocab=VOCAB, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def close(got, want, tol):
    want = want.to(torch.float64)
    err = (got.to(torch.float64).cpu() - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), f"max error {err:.3e} (scale {want.abs().max().item():.3e})"


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


# ---------------------------------------------------------------------------------------------------------------------
# every mechanism alone: one layer, whole prompt and cut prompt
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("spec", [layer(PAR), layer(PAR_B), layer(PAR_C), layer(GRU), layer(GRU_B), layer(GRU_B, FF), layer(GRU_B, FF_B)],
                         ids=["parallel", "parallel_full_rotation", "parallel_one_tap_one_kv", "mingru", "mingru_odd", "ff", "ff_wide_limit"])
def test_single_mechanism_matches_oracle(spec, device):
    cfg = config_of([spec])
    model, W = build(cfg, device)
    toks = tokens_of(37)
    want, layers = oracle.forward(cfg, W, toks, return_layers=True)
    seen = []
    model.decoder.tap = lambda i, x: seen.append(x.detach().float().cpu().clone())
    rp = replayer(model)
    close(run_cut(rp, "a", toks, [len(toks)]), want, TOL[torch.float32])
    close(seen[0].view(len(toks), -1), layers[0], TOL[torch.float32])
    model.decoder.tap = None
    close(run_cut(rp, "b", toks, [17, 2, 16]), want, TOL[torch.float32])


def test_model_without_bigram_table_and_whole_sequence_forward_without_a_context():
    """The training-style call (``[b, s]`` ids, no inference context) runs the same mixers from zero state."""
    for cfg in (HYBRID, config_of([layer(PAR_B, FF), layer(GRU)], bigram=False)):
        model, W = build(cfg, "cpu")
        a, b = tokens_of(21, seed=1), tokens_of(21, seed=2)
        out = model(torch.tensor([a, b]), None, None)
        close(out[0], oracle.forward(cfg, W, a), TOL[torch.float32])
        close(out[1], oracle.forward(cfg, W, b), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_ops_match_the_oracle_functions(device):
    """The op level: output norm with two branches, q / k norm + rotation, head-mixing attention, delta memory, minGRU, the
    clamped gate -- each against the oracle's function for that mechanism."""
    g = torch.Generator().manual_seed(3)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    T, h = 11, 20
    # output norm of the mean of two normed branches, added to the stream
    x, a, b, wa, wb, w = rn(T, h), rn(T, h), rn(T, h), rn(h), rn(h), rn(h) * 0.2
    want = x.double() + oracle.one_plus_norm(0.5 * (oracle.rms(a.double(), 1e-5) * wa.double() + oracle.rms(b.double(), 1e-5) * wb.double()),
                                             w.double(), 1e-5)
    xs, y = seqmix.norm_add(x.clone().to(device), a.to(device), w.to(device), 1e-5, torch.float32, 1.0, b.to(device), wa.to(device),
                            wb.to(device))
    close(xs, want, 1e-5)
    close(y, want, 1e-5)
    xs, _ = seqmix.norm_add(x.clone().to(device), a.to(device), w.to(device), 1e-5, torch.float32, 0.0)
    close(xs, x.double() + oracle.rms(a.double(), 1e-5) * w.double(), 1e-5)
    # q / k norm + rotation at scattered positions; an odd head count and a k narrower than q
    H, G, d, rot = 5, 1, 12, {"base": 300.0, "dims": 6, "scaling": {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 40}}
    fr = oracle.rotary_frequencies(rot)
    q, k, wq, wk = rn(T, H * d), rn(T, G * d), rn(H * d), rn(G * d)
    pos = torch.tensor([0, 1, 2, 3, 100, 101, 7, 1000, 1001, 5000, 12])
    qo, ko = seqmix.norm_rope(q.to(device), k.to(device), wq.to(device), wk.to(device), pos.to(device),
                              torch.tensor(fr, dtype=torch.float32, device=device), d, rot["dims"], 1e-5)
    for got, src, ww, n in ((qo, q, wq, H), (ko, k, wk, G)):
        ref = torch.stack([oracle.rotate((oracle.rms(src[t].double(), 1e-5) * ww.double()).view(n, d), int(pos[t]), fr) for t in range(T)])
        close(got.view(T, n, d), ref, 3e-4)          # fp32 angles at position 5000 carry ~1e-4 rad of rounding
    # the clamped gate: values on both sides of every clamp
    xg = torch.tensor([[-3.0, -0.5, 0.4, 0.8, 5.0, 0.1, -2.0, 0.3, 0.79, 9.0]])
    yg = seqmix.clamped_glu(xg.to(device), 0.8)
    gg, uu = xg[:, :5].double().clamp(max=0.8), xg[:, 5:].double().clamp(-0.8, 0.8)
    close(yg, gg * torch.sigmoid(1.702 * gg) * (uu + 1), 1e-6)
    # minGRU and the delta memory from a given state, two sequences of unequal length in one packed batch
    C = 9
    zp, up, gp = rn(T, C), rn(T, C) * 2, rn(T, C)
    pb = seqmix.PackedBatch([0, 4, T], [2, 0], device)
    S0 = rn(3, C)
    st = S0.clone().to(device)
    y = seqmix.mingru_scan(zp.to(device), up.to(device), gp.to(device), pb, st)
    for lo, hi, row in ((0, 4, 2), (4, T, 0)):
        Sref, Send = oracle.mingru_loop(torch.sigmoid(zp[lo:hi].double()), up[lo:hi].double(), S0[row].double())
        close(y[lo:hi], Sref * gp[lo:hi].double() * torch.sigmoid(gp[lo:hi].double()), 1e-5)
        close(st[row], Send, 1e-5)
    close(st[1], S0[1].double(), 0.0)
    Hh, dd, dv = 2, 6, 10
    r, k2, v2, wp, ap, wb0 = rn(T, Hh, dd), rn(T, Hh, dd), rn(T, Hh, dv), rn(T, Hh * dd), rn(T, Hh * dd), rn(Hh * dd)
    M0 = rn(3, Hh, dd, dv)
    st = M0.clone().to(device)
    o = seqmix.gen_delta_scan(r.to(device), k2.to(device), v2.to(device), wp.to(device), ap.to(device), wb0.to(device), pb, st, 0.6)
    wd = torch.exp(-0.6 * torch.sigmoid(wp.double() + wb0.double())).view(T, Hh, dd)
    ad = torch.sigmoid(ap.double()).view(T, Hh, dd)
    for lo, hi, row in ((0, 4, 2), (4, T, 0)):
        oref, Send = oracle.delta_memory_loop(r[lo:hi].double(), k2[lo:hi].double(), v2[lo:hi].double(), wd[lo:hi], ad[lo:hi], M0[row].double())
        close(o[lo:hi], oref, 1e-5)
        close(st[row], Send, 1e-5)


# ---------------------------------------------------------------------------------------------------------------------
# the hybrid stack: portions, decoding, batches, reuse
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cuts", [[50], [1], [2, 2, 2], [15, 16, 17], [16, 16], [33, 3], [47]], ids=str)
def test_portions_and_decoding_match_whole_prompt(cuts, device):
    """Chunk edges of the scans, page edges (4), the convolution's window and the first tokens all fall inside some portion."""
    model, W = build(HYBRID, device)
    toks = tokens_of(50, seed=3)
    want = oracle.forward(HYBRID, W, toks)
    close(run_cut(replayer(model), "a", toks, cuts), want, TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_unequal_batch_matches_each_alone_and_rows_are_reused(device):
    model, W = build(HYBRID, device)
    reqs = {"a": tokens_of(1, seed=4), "b": tokens_of(23, seed=5), "c": tokens_of(9, seed=6)}
    want = {k: oracle.forward(HYBRID, W, v) for k, v in reqs.items()}
    rp = replayer(model, max_requests=3)
    got = {k: [] for k in reqs}
    first = {k: max(1, len(v) - 5) for k, v in reqs.items()}
    out = rp.step([{"id": k, "tokens": v[:first[k]], "want": list(range(first[k]))} for k, v in reqs.items()],
                  end=[k for k, v in reqs.items() if first[k] == len(v)])
    at = 0
    for k in reqs:
        got[k].append(out[at:at + first[k]])
        at += first[k]
    pos = dict(first)
    while any(pos[k] < len(reqs[k]) for k in reqs):
        live = [k for k in reqs if pos[k] < len(reqs[k])]
        out = rp.step([{"id": k, "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live],
                      end=[k for k in live if pos[k] + 1 == len(reqs[k])])
        for j, k in enumerate(live):
            got[k].append(out[j:j + 1])
            pos[k] += 1
    for k in reqs:
        close(torch.cat(got[k]), want[k], TOL[torch.float32])
    ctx = rp.engine.context
    assert not ctx.seqs and ctx.allocator.free == ctx.num_blocks and len(ctx._free_rows) == 3
    # the freed pages and state rows now serve other requests: a stale window, memory, key or previous token would show
    for k, v in (("d", tokens_of(30, seed=7)), ("e", tokens_of(6, seed=8))):
        close(run_cut(rp, k, v, [len(v) - 3]), oracle.forward(HYBRID, W, v), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_other_sizes_five_taps_no_rotation_many_heads_per_group(device):
    """Sizes none of the other tests use: five convolution taps (the generic convolution kernel and a four-row window), no
    rotated dimensions at all, eight query heads per key/value head, a value width that is a multiple of the key width, an
    odd minGRU width first in the stack, a model without bigram table and a feed-forward limit that never binds."""
    left = {"heads": 16, "kv_heads": 2, "dim": 8, "vdim": 48, "conv": 5, "scale": 0.3, "rot": {"base": 100.0, "dims": 0}}
    left2 = {"heads": 5, "dim": 24, "conv": 1, "scale": 0.11, "rot": {"base": 777.0, "dims": 24,
                                                                       "scaling": {"factor": 2.0, "low": 2.0, "high": 4.0, "original": 16}}}
    cfg = config_of([layer(GRU_B, {"kind": "dense", "ff": 24, "limit": 50.0}),
                     layer({"type": "parallel", "mixer": {"left": left, "right": {"heads": 5, "dim": 16}}}, FF),
                     layer({"type": "parallel", "mixer": {"left": left2, "right": {"heads": 1, "dim": 96}}})],
                    width=136, vocab=300, eps=1e-5, bigram=False)
    model, W = build(cfg, device)
    toks = tokens_of(61, vocab=300, seed=16)
    want = oracle.forward(cfg, W, toks)
    rp = replayer(model)
    close(run_cut(rp, "a", toks, [61]), want, TOL[torch.float32])
    close(run_cut(rp, "b", toks, [3, 2, 40]), want, TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding(device):
    cfg = config_of([layer(PAR, FF_B), layer(GRU), layer(PAR, FF_B, weights_of=0)])
    model, W = build(cfg, device)
    toks = tokens_of(140, seed=9)
    close(run_cut(replayer(model, block_size=16), "a", toks, [3]), oracle.forward(cfg, W, toks), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_long_prompt_takes_the_run_parallel_scan(device):
    """Prompts above four runs of 64 tokens go through the reduce / carry / apply kernels of the minGRU scan; cut at a point
    that is no run edge, the second portion starts from the carried state."""
    cfg = config_of([layer(GRU, FF), layer(PAR_B)], width=24)
    model, W = build(cfg, device)
    toks = tokens_of(333, seed=14)
    want = oracle.forward(cfg, W, toks)
    rp = replayer(model, max_tokens=1024, block_size=16)
    close(run_cut(rp, "a", toks, [333]), want, TOL[torch.float32])
    close(run_cut(rp, "b", toks, [301, 30]), want, TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_engine(device):
    """``DynamicInferenceEngine.generate``: scheduler, chunked prefill under a token budget, sampling; the oracle re-reads
    the whole sequence for every new token."""
    model, W = build(HYBRID, device)
    eng = DynamicInferenceEngine(model, NullTokenizer(VOCAB - 1), max_sequence_length=64, num_blocks=24, block_size=4,
                                 max_tokens_per_step=7, max_requests=3)
    prompts = [tokens_of(11, seed=10), tokens_of(2, seed=11), tokens_of(5, seed=12), tokens_of(8, seed=13)]
    out = eng.generate([" ".join(map(str, p)) for p in prompts], SamplingParams(top_k=1, num_tokens_to_generate=5))
    for p, o in zip(prompts, out):
        toks = list(p)
        for _ in range(o.generated_length):
            toks.append(int(oracle.forward(HYBRID, W, toks)[-1, :VOCAB].argmax()))
        assert toks[len(p):] == o.generated_tokens.tolist()
    assert eng.context.allocator.free == 24 and not eng.context.seqs


def test_bfloat16_serving_stays_within_rounding():
    model, W = build(HYBRID, "cpu", torch.bfloat16)
    Wr = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    toks = tokens_of(40, seed=15)
    close(run_cut(replayer(model), "a", toks, [25, 2]), oracle.forward(HYBRID, Wr, toks), TOL[torch.bfloat16] * 4)


@pytest.mark.gpu
def test_bfloat16_kernels_stay_within_rounding():
    model, W = build(HYBRID, "cuda", torch.bfloat16)
    Wr = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    toks = tokens_of(40, seed=15)
    before = seqmix.kernel_calls["mixed_attention_paged"]
    close(run_cut(replayer(model), "a", toks, [25, 2]), oracle.forward(HYBRID, Wr, toks), TOL[torch.bfloat16] * 4)
    assert seqmix.kernel_calls["mixed_attention_paged"] > before


# ---------------------------------------------------------------------------------------------------------------------
# hand-made inputs: what random weights would hide
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dv", [6, 8], ids=["scalar_kernel", "vector_kernel"])
@pytest.mark.parametrize("ctx_len,far", [(5, 0), (64, 0), (65, 1), (300, 3), (300, 4), (1200, 7), (1200, 1199)])
def test_attention_finds_one_far_key_across_pages(ctx_len, far, dv, device):
    """One key among hundreds matches the last query; its value must come through whatever page or tile edge it sits at, and
    only through the heads that the mixing matrix routes it to."""
    H, G, d, bs = 4, 2, 8, 4
    g = torch.Generator().manual_seed(ctx_len + far)
    k = torch.randn(ctx_len, G, d, generator=g) * 0.1
    v = torch.randn(ctx_len, G, dv, generator=g)
    q = torch.randn(1, H, d, generator=g) * 0.1
    q[0, 1] = 0.0
    q[0, 1, 3] = 30.0                                   # head 1 (kv head 0) asks for channel 3 ...
    k[far, 0, 3] = 30.0                                 # ... which only the far key has
    talk = torch.zeros(H, H)
    talk[0, 0] = talk[1, 1] = talk[2, 2] = 1.0
    talk[3, 1] = 2.0                                    # head 3 (kv head 1) uses head 1's weights, doubled
    nb = -(-ctx_len // bs)
    table = torch.randperm(nb, generator=g).to(torch.int32).view(1, nb)
    kc, vc = torch.zeros(nb * bs, G, d), torch.zeros(nb * bs, G, dv)
    pos = torch.arange(ctx_len)
    slots = table[0].long()[pos // bs] * bs + pos % bs
    kc[slots], vc[slots] = k, v
    to = lambda t: t.to(device)  # noqa: E731
    o = seqmix.mixed_attention_paged(to(q), to(kc), to(vc), to(table), to(torch.zeros(1, dtype=torch.int32)),
                                     to(torch.tensor([ctx_len], dtype=torch.int32)), bs, 1.0, to(talk), None, ctx_len).view(H, dv)
    close(o[1], v[far, 0], 1e-4)
    close(o[3], 2.0 * v[far, 1], 1e-4)
    ref = oracle.head_mixing_attention(torch.cat([torch.zeros(ctx_len - 1, H, d), q]).double(), k.double(), v.double(), 1.0, talk.double())[-1]
    close(o, ref, 1e-4)
    # one token earlier the far key is the only thing that changes: leave it out of sight and the answer must move
    if far == ctx_len - 1 and ctx_len > 1:
        o2 = seqmix.mixed_attention_paged(to(q), to(kc), to(vc), to(table), to(torch.zeros(1, dtype=torch.int32)),
                                          to(torch.tensor([ctx_len - 1], dtype=torch.int32)), bs, 1.0, to(talk), None, ctx_len).view(H, dv)
        assert (o2[1].cpu() - v[far, 0]).abs().max() > 0.1


@pytest.mark.parametrize("device", DEVICES)
def test_delta_memory_recalls_an_early_write_after_hundreds_of_tokens(device):
    """Decay near one and no removal along other keys: a value written at token 2 under a key that no later token touches is
    read back at the end; with removal switched on along that very key it is gone."""
    T, H, d = 400, 2, 8
    g = torch.Generator().manual_seed(1)
    k = torch.zeros(T, H, d)
    k[:, :, 1:5] = torch.randn(T, H, 4, generator=g)            # later keys live in channels 1..4
    k[2] = 0.0
    k[2, :, 7] = 1.0                                            # the early write uses channel 7 alone
    v = torch.randn(T, H, d, generator=g)
    r = torch.zeros(T, H, d)
    r[-1, :, 7] = 1.0
    w_pre = torch.full((T, H * d), -30.0)                       # sigmoid -> 0: decay exp(0) = 1
    a_pre = torch.full((T, H * d), 30.0)                        # full removal along the current unit key
    pb = seqmix.PackedBatch([0, T], [0], device)
    to = lambda t: t.to(device)  # noqa: E731
    st = torch.zeros(1, H, d, d, device=device)
    o = seqmix.gen_delta_scan(to(r), to(k), to(v), to(w_pre), to(a_pre), None, pb, st, math.exp(-0.5))
    close(o[-1], v[2], 1e-4)
    k2 = k.clone()
    k2[300, :, :] = 0.0
    k2[300, :, 7] = 2.0                                         # a later token with the same direction removes and rewrites
    st = torch.zeros(1, H, d, d, device=device)
    o = seqmix.gen_delta_scan(to(r), to(k2), to(v), to(w_pre), to(a_pre), None, pb, st, math.exp(-0.5))
    close(o[-1], 2.0 * v[300], 1e-4)


@pytest.mark.parametrize("device", DEVICES)
def test_short_convolution_window_and_previous_token_across_steps_of_one_and_two_tokens(device):
    """Convolution without activation: the window carries exactly ``taps - 1`` projected rows over steps shorter than itself;
    the bigram row of a step's first token pairs it with the last token of the step before."""
    g = torch.Generator().manual_seed(2)
    C, taps, T = 6, 4, 9
    x, w = torch.randn(T, C, generator=g), torch.randn(C, taps, generator=g)
    want = oracle.short_conv(x.double(), w.double())
    win = torch.zeros(2, taps - 1, C, device=device)
    parts, at = [], 0
    for n in (1, 2, 1, 1, 2, 2):
        parts.append(seqmix.causal_conv(x[at:at + n].to(device), w.to(device), seqmix.PackedBatch([0, n], [1], device), win))
        at += n
    close(torch.cat(parts), want, 1e-5)
    close(win[1], x[-(taps - 1):].double(), 0.0)
    assert float(win[0].abs().sum()) == 0.0
    cfg = config_of([layer(GRU_B)])
    model, W = build(cfg, device)
    toks = [7, 7, 3, 7, 3, 3, 12, 7]
    close(run_cut(replayer(model), "a", toks, [1, 2, 1, 2]), oracle.forward(cfg, W, toks), TOL[torch.float32])
    rows = model.bigram_embedding.rows(torch.tensor([7, 7, 3]), torch.tensor([-1, 7, 7]))
    assert rows.tolist() == [37, (7 * 5 + 7 * 3) % 37, (7 * 5 + 3 * 3) % 37]


def test_rotary_frequency_scaling_has_three_regimes():
    from megatronapp_b200.models.common.embeddings import llama3_scaled_frequencies

    rot = {"base": 50.0, "dims": 16, "scaling": {"factor": 5.0, "low": 1.0, "high": 4.0, "original": 32}}
    got = llama3_scaled_frequencies(16, 50.0, rot["scaling"])
    want = torch.tensor(oracle.rotary_frequencies(rot), dtype=torch.float64)
    plain = torch.tensor(oracle.rotary_frequencies({"base": 50.0, "dims": 16}), dtype=torch.float64)
    close(got, want, 1e-6)
    ratio = (want / plain).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 0.2) < 1e-12 and any(0.21 < x < 0.99 for x in ratio)


def test_config_rejects_bad_layer_references():
    with pytest.raises(ValueError):
        LeroraxConfig.from_dict(config_of([layer(PAR), layer(GRU, weights_of=0)]))          # another type
    with pytest.raises(ValueError):
        LeroraxConfig.from_dict(config_of([layer(GRU, weights_of=1), layer(GRU, weights_of=0)]))   # nobody owns tensors
    lcfg = LeroraxConfig.from_dict(HYBRID)
    assert lcfg.owners() == [0, 1, 2, 4, 6] and lcfg.owner(7) == 0


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_attention_prompt_portions_of_several_sequences_in_one_batch(dtype, device):
    """Three sequences with 0, 9 and 130 cached tokens bring 70, 1 and 3 new ones: query blocks of the vector kernel straddle
    the sequences, and every query sees exactly its own prefix.  Both kernels against the oracle's attention."""
    H, G, d, dv, bs = 4, 2, 16, 8, 4
    g = torch.Generator().manual_seed(11)
    before, new = [0, 9, 130], [70, 1, 3]
    talk = torch.eye(H) * 0.6 + torch.randn(H, H, generator=g) * 0.3
    nb = [-(-(b + n) // bs) for b, n in zip(before, new)]
    perm = torch.randperm(sum(nb), generator=g)
    table = torch.zeros(3, max(nb), dtype=torch.int32)
    kc, vc = torch.zeros(sum(nb) * bs, G, d), torch.zeros(sum(nb) * bs, G, dv)
    qs, req, lens, want, at = [], [], [], [], 0
    for r, (b, n) in enumerate(zip(before, new)):
        table[r, :nb[r]] = perm[at:at + nb[r]].to(torch.int32)
        at += nb[r]
        L = b + n
        q, k, v = (torch.randn(L, H, d, generator=g), torch.randn(L, G, d, generator=g), torch.randn(L, G, dv, generator=g))
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
        pos = torch.arange(L)
        slots = table[r].long()[pos // bs] * bs + pos % bs
        kc[slots], vc[slots] = k, v
        want.append(oracle.head_mixing_attention(q.double(), k.double(), v.double(), 0.25, talk.double())[b:])
        qs.append(q[b:])
        req += [r] * n
        lens += list(range(b + 1, L + 1))
    gate = torch.randn(sum(new), H * dv, generator=g).to(dtype)
    ref = torch.cat(want).reshape(-1, H * dv) * torch.sigmoid(gate.double())
    to = lambda t: t.to(device)  # noqa: E731
    for generic in (False, True):
        o = seqmix.mixed_attention_paged(to(torch.cat(qs).to(dtype)), to(kc.to(dtype)), to(vc.to(dtype)), to(table),
                                         to(torch.tensor(req, dtype=torch.int32)), to(torch.tensor(lens, dtype=torch.int32)), bs, 0.25,
                                         to(talk), to(gate), 133, force_generic=generic)
        close(o, ref, 1e-4 if dtype == torch.float32 else 2e-2)


# ---------------------------------------------------------------------------------------------------------------------
# model folder -> registry -> trace runner
# ---------------------------------------------------------------------------------------------------------------------
def write_model_folder(path, cfg, W):
    with open(path / "config.json", "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for k, v in W.items():
        b = v.to(torch.bfloat16).contiguous().view(torch.uint8).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    h = json.dumps(header).encode()
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def test_model_folder_through_registry_trace_runner_and_cli(tmp_path):
    import numpy as np

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = config_of([layer(PAR_C, FF), layer(GRU), layer(PAR_C, FF, weights_of=0)])
    W = {k: v.to(torch.bfloat16).float() for k, v in oracle.random_weights(cfg, 5, decay_rank=3).items()}
    write_model_folder(tmp_path, cfg, W)
    a, b = tokens_of(19, seed=20), tokens_of(6, seed=21)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:16], "want": [0, 7, 15]}, {"id": "y", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[16:17], "want": []}, {"id": "y", "tokens": b[4:5], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[17:18], "want": [0]}, {"id": "y", "tokens": b[5:6], "want": [0]}], "end": ["y"]},
             {"step": 3, "entries": [{"id": "x", "tokens": a[18:19], "want": [0]}], "end": ["x"]}]
    out = tmp_path / "out"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    wa, wb = oracle.forward(cfg, W, a), oracle.forward(cfg, W, b)
    got = {n: torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, VOCAB).copy()) for n in (0, 1, 2, 3)}
    close(got[0], torch.stack([wa[0], wa[7], wa[15], wb[3]]), TOL[torch.float32])
    close(got[1], wb[4:5], TOL[torch.float32])
    close(got[2], torch.stack([wa[17], wb[5]]), TOL[torch.float32])
    close(got[3], wa[18:19], TOL[torch.float32])
    # the generation command line on the same folder: greedy tokens of the oracle
    import sys

    r = subprocess.run([sys.executable, os.path.join(root, "tools", "run_text_generation_server.py"), "--model-dir", str(tmp_path),
                        "--dtype", "float32", "--prompts", " ".join(map(str, b)), "--num-tokens-to-generate", "4"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    toks = list(b)
    for _ in range(4):
        toks.append(int(oracle.forward(cfg, W, toks)[-1].argmax()))
    assert r.stdout.strip().splitlines()[-1].endswith("-> " + repr(" ".join(map(str, toks[len(b):]))))
