"""Zikunex models in the framework against a plain, slow evaluation of the design's equations (``zikunex_oracle``).

Each test builds its own small configuration and random (or hand-made) weights, loads them through the product loader
and drives the model through the dynamic engine -- whole prompts, prompts cut into portions, token-by-token decoding,
mixed batches, reused pages and state rows -- on the CPU (PyTorch op path) and, marked ``gpu``, on the sm_100a kernels.
"""
import copy

import pytest
import torch

import zikunex_oracle as oracle
from megatronapp_b200.data.tokenizer import NullTokenizer
from megatronapp_b200.inference import DynamicInferenceEngine, SamplingParams
from megatronapp_b200.inference.trace import TraceReplayer
from megatronapp_b200.models.zikunex import ZikunexConfig, ZikunexModel, load_zikunex_weights
from megatronapp_b200.models.zikunex.loader import shapes_into_config
from megatronapp_b200.ops import seqmix
from megatronapp_b200.parallel import state as ps

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]

MOE_A = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}},
         "shared": {"ff": 40}}
MOE_B = {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 6, "top": 1}}        # no groups, no shared expert, top 1
DELTA = {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 3}}
DELTA_B = {"type": "channel_delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 40, "vdim": 72, "conv": 2}}
MLSTM = {"type": "mlstm", "mixer": {"heads": 2, "dim": 40, "vdim": 72, "gate_cap": 10.0}}
MLSTM_B = {"type": "mlstm", "mixer": {"heads": 3, "dim": 8, "vdim": 8, "gate_cap": 4.0}}
LAT = {"type": "latent_attention", "mixer": {"heads": 2, "dim": 24, "vdim": 16, "kv_rank": 40, "q_rank": 24, "scale": 0.2}}
LAT_B = {"type": "latent_attention", "mixer": {"heads": 5, "dim": 8, "vdim": 12, "kv_rank": 72, "q_rank": 16, "scale": 0.35}}


def layer(spec, mlp=None, **mixer_extra):
    l = copy.deepcopy(spec)
    l["mixer"].update(mixer_extra)
    l["mlp"] = copy.deepcopy(mlp)
    return l


def config_of(layers, width=64, vocab=96, eps=1e-5, scale=0.7):
    return {"architecture": "Zikunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


HYBRID = config_of([layer(DELTA, {"kind": "dense", "ff": 96}), layer(LAT, MOE_A), layer(MLSTM), layer(LAT, MOE_B, kv_from=1),
                    layer(LAT_B, {"kind": "dense", "ff": 32}), layer(DELTA_B, MOE_A), layer(MLSTM_B, MOE_B)])


def build(cfg, device, dtype=torch.float32, seed=0, weights=None):
    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(1, 1)
    W = weights if weights is not None else oracle.random_weights(cfg, seed, low_rank=12)
    raw = shapes_into_config(copy.deepcopy(cfg), {k: list(v.shape) for k, v in W.items()})
    zcfg = ZikunexConfig.from_dict(raw)
    model = ZikunexModel(zcfg, zcfg.base_transformer_config(dtype, use_cpu_initialization=True, perform_initialization=False))
    load_zikunex_weights(model, W)
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


def tokens_of(n, vocab=96, seed=0):
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
@pytest.mark.parametrize("spec", [layer(DELTA), layer(DELTA_B), layer(MLSTM), layer(MLSTM_B), layer(LAT), layer(LAT_B),
                                  layer(MLSTM_B, {"kind": "dense", "ff": 40}), layer(MLSTM_B, MOE_A), layer(MLSTM_B, MOE_B)],
                         ids=["delta", "delta_1head", "mlstm", "mlstm_small", "latent", "latent_5heads", "dense_ff", "moe_groups",
                              "moe_top1"])
def test_single_mechanism_matches_oracle(spec, device):
    cfg = config_of([spec])
    model, W = build(cfg, device)
    toks = tokens_of(37)
    want, layers = oracle.forward(cfg, W, toks, return_layers=True)
    seen = []
    model.decoder.tap = lambda i, x: seen.append(x.detach().float().cpu())
    rp = replayer(model)
    close(run_cut(rp, "a", toks, [len(toks)]), want, TOL[torch.float32])
    close(seen[0].view(len(toks), -1), layers[0], TOL[torch.float32])
    model.decoder.tap = None
    close(run_cut(rp, "b", toks, [17, 2, 16]), want, TOL[torch.float32])


def test_whole_sequence_forward_without_a_context_matches_oracle():
    """The training-style call (``[b, s]`` ids, no inference context) runs the same mixers from zero state."""
    model, W = build(HYBRID, "cpu")
    a, b = tokens_of(21, seed=1), tokens_of(21, seed=2)
    out = model(torch.tensor([a, b]), None, None)
    close(out[0], oracle.forward(HYBRID, W, a), TOL[torch.float32])
    close(out[1], oracle.forward(HYBRID, W, b), TOL[torch.float32])


# ---------------------------------------------------------------------------------------------------------------------
# the hybrid stack: portions, decoding, batches, reuse
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cuts", [[50], [1], [2, 2, 2], [15, 16, 17], [16, 16], [33, 3], [47]], ids=str)
def test_portions_and_decoding_match_whole_prompt(cuts, device):
    """Chunk edges of the scans (16), page edges (4) and the first tokens all fall inside some portion here."""
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
    # prefill all but the last 5 tokens together, then decode together; shorter requests leave earlier
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
    # the freed pages and state rows now serve other requests: stale state or latents would show
    for k, v in (("d", tokens_of(30, seed=7)), ("e", tokens_of(6, seed=8))):
        close(run_cut(rp, k, v, [len(v) - 3]), oracle.forward(HYBRID, W, v), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding(device):
    cfg = config_of([layer(DELTA, MOE_B), layer(LAT), layer(MLSTM_B)])
    model, W = build(cfg, device)
    toks = tokens_of(140, seed=9)
    close(run_cut(replayer(model, block_size=16), "a", toks, [3]), oracle.forward(cfg, W, toks), TOL[torch.float32])


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_engine(device):
    """``DynamicInferenceEngine.generate``: scheduler, chunked prefill under a token budget, sampling; the oracle re-reads
    the whole sequence for every new token."""
    model, W = build(HYBRID, device)
    eng = DynamicInferenceEngine(model, NullTokenizer(95), max_sequence_length=64, num_blocks=24, block_size=4,
                                 max_tokens_per_step=7, max_requests=3)
    prompts = [tokens_of(11, seed=10), tokens_of(2, seed=11), tokens_of(5, seed=12), tokens_of(8, seed=13)]
    out = eng.generate([" ".join(map(str, p)) for p in prompts], SamplingParams(top_k=1, num_tokens_to_generate=5))
    for p, o in zip(prompts, out):
        toks = list(p)
        for _ in range(o.generated_length):
            toks.append(int(oracle.forward(HYBRID, W, toks)[-1, :96].argmax()))
        assert toks[len(p):] == o.generated_tokens.tolist()
    assert eng.context.allocator.free == 24 and not eng.context.seqs


def test_preempted_request_recomputes_its_state_from_zero():
    """Out of pages in mid-decode: the engine evicts a request (pages and state row go back) and prefills it again later;
    a state row that kept anything of the first attempt would change the tokens."""
    cfg = config_of([layer(DELTA, {"kind": "dense", "ff": 48}), layer(LAT), layer(MLSTM_B, MOE_A)])
    model, W = build(cfg, "cpu")
    eng = DynamicInferenceEngine(model, NullTokenizer(95), max_sequence_length=64, num_blocks=8, block_size=4,
                                 max_tokens_per_step=16, max_requests=3)
    prompts = [tokens_of(4, seed=40), tokens_of(4, seed=41), tokens_of(4, seed=42)]
    out = eng.generate([" ".join(map(str, p)) for p in prompts], SamplingParams(top_k=1, num_tokens_to_generate=10))
    assert eng.num_preemptions >= 1
    for p, o in zip(prompts, out):
        toks = list(p)
        for _ in range(o.generated_length):
            toks.append(int(oracle.forward(cfg, W, toks)[-1, :96].argmax()))
        assert toks[len(p):] == o.generated_tokens.tolist()
    assert eng.context.allocator.free == 8 and len(eng.context._free_rows) == 3


@pytest.mark.gpu
def test_bfloat16_serving_stays_within_rounding():
    """bf16 projections around fp32 state, scores and residual.  A router's close call may flip an expert under bf16
    rounding and move single positions, so the bound is on the typical position, with a loose one on all."""
    cfg = config_of([layer(DELTA, {"kind": "dense", "ff": 96}), layer(LAT, MOE_A), layer(MLSTM), layer(LAT, MOE_A, kv_from=1),
                     layer(DELTA_B, {"kind": "dense", "ff": 32})])
    model, W = build(cfg, "cuda", torch.bfloat16)
    Wb = {k: v.to(torch.bfloat16).float() if v.is_floating_point() else v for k, v in W.items()}
    toks = tokens_of(60, seed=14)
    want = oracle.forward(cfg, Wb, toks)
    got = run_cut(replayer(model), "a", toks, [40, 5])
    d = got.double().cpu() - want
    d = d - d.mean(-1, keepdim=True)
    rel = d.pow(2).mean(-1).sqrt() / want.std(-1)
    assert rel.median().item() < 0.03 and rel.max().item() < 0.5, (rel.median().item(), rel.max().item())
    assert seqmix.kernel_calls["delta_rule_scan"] and seqmix.kernel_calls["latent_attention_paged"]


@pytest.mark.gpu
def test_fresh_prompts_through_the_flash_kernel_match_the_paged_kernel_and_the_oracle(monkeypatch):
    """bf16 prompts with a head shape the tcgen05 flash kernel takes are expanded to K / V for their first step; lengths off
    the kernel's tile sizes, two prompts in one step, a layer that shares latents, then decoding from the pages."""
    from megatronapp_b200 import ops

    lat64 = {"type": "latent_attention", "mixer": {"heads": 3, "dim": 64, "vdim": 64, "kv_rank": 40, "q_rank": 24, "scale": 0.15}}
    cfg = config_of([layer(lat64, {"kind": "dense", "ff": 96}), layer(MLSTM_B), layer(lat64, kv_from=0)])
    model, W = build(cfg, "cuda", torch.bfloat16)
    Wb = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    reqs = {"a": tokens_of(203, seed=30), "b": tokens_of(70, seed=31)}
    want = {k: oracle.forward(cfg, Wb, v) for k, v in reqs.items()}

    def run(flag):
        monkeypatch.setenv("B200_LATENT_FLASH_PREFILL", flag)
        rp = replayer(model, max_tokens=1024, block_size=16)
        first = {"a": 199, "b": 65}
        outs = {k: [] for k in reqs}
        o = rp.step([{"id": k, "tokens": reqs[k][:first[k]], "want": list(range(first[k]))} for k in reqs])
        outs["a"].append(o[:199])
        outs["b"].append(o[199:])
        for j in range(4):
            o = rp.step([{"id": k, "tokens": [reqs[k][first[k] + j]], "want": [0]} for k in reqs])
            outs["a"].append(o[0:1])
            outs["b"].append(o[1:2])
        return {k: torch.cat(v) for k, v in outs.items()}

    before = ops.fallback_counts["attention_sdpa"]
    flash, paged_ = run("1"), run("0")
    assert ops.fallback_counts["attention_sdpa"] == before and ops.native_attention_available()
    for k in reqs:
        n = flash[k].shape[0]
        for got in (flash[k], paged_[k]):
            d = got.double().cpu() - want[k][:n]
            d = d - d.mean(-1, keepdim=True)
            rel = d.pow(2).mean(-1).sqrt() / want[k][:n].std(-1)
            assert rel.median().item() < 0.03 and rel.max().item() < 0.2, (k, rel.median().item(), rel.max().item())


# ---------------------------------------------------------------------------------------------------------------------
# ops with inputs made so that one far entry decides the result
# ---------------------------------------------------------------------------------------------------------------------
def paged(ctx_len, block_size, r, device, seed=0):
    """Latents of one sequence scattered over shuffled pages; returns (cache, block_table, latents in order)."""
    g = torch.Generator().manual_seed(seed)
    n_blocks = -(-ctx_len // block_size)
    order = torch.randperm(n_blocks + 3, generator=g)[:n_blocks]
    c = torch.randn(ctx_len, r, generator=g) * 0.3
    cache = torch.randn((n_blocks + 3) * block_size, r, generator=g)          # unused slots hold garbage, not zeros
    pos = torch.arange(ctx_len)
    cache[order[pos // block_size] * block_size + pos % block_size] = c
    return cache.to(device), order.to(torch.int32).view(1, -1).to(device), c


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("ctx_len,far", [(300, 2), (64, 63), (65, 64), (63, 0), (17, 16), (1, 0)])
def test_latent_attention_finds_one_far_key_across_pages(ctx_len, far, device):
    r, H, bs = 40, 3, 16
    cache, table, c = paged(ctx_len, bs, r, device, seed=ctx_len)
    q = torch.randn(1, H, r, generator=torch.Generator().manual_seed(1)) * 0.3
    c = c.clone()
    c[far] = q[0, 1] / q[0, 1].norm() * 6.0                                 # head 1 must lock onto this key
    q[0, 1] = q[0, 1] / q[0, 1].norm() * 6.0
    pos = torch.arange(ctx_len)
    cache[table[0].long().cpu()[pos // bs].to(device) * bs + (pos % bs).to(device)] = c.to(device)
    one = torch.ones(1, dtype=torch.int32, device=device)
    for visible in {ctx_len, max(1, far), far + 1}:
        out = seqmix.latent_attention_paged(q.to(device), cache, table, 0 * one, visible * one, bs, 1.0)
        k = c[:visible].view(visible, 1, r).expand(visible, H, r)
        want = oracle.causal_attention_loop(q.expand(visible, H, r).double(), k.double(), k.double(), 1.0)[-1]
        close(out[0], want, 1e-5)
        if far < visible:
            assert (out[0, 1].cpu() - c[far]).norm() < 0.05 * c[far].norm()
        else:
            assert (out[0, 1].cpu() - c[far]).norm() > 0.5 * c[far].norm()


@pytest.mark.parametrize("device", DEVICES)
def test_delta_rule_recalls_an_early_write_after_hundreds_of_tokens(device):
    T, H, KH, d, dv = 260, 2, 1, 20, 70
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(T, KH, d, generator=g), torch.randn(T, KH, d, generator=g)
    v, beta = torch.randn(T, H, dv, generator=g), torch.rand(T, H, generator=g) * 0.1
    log_decay = -torch.rand(T, H, d, generator=g) * 1e-3
    # token 3 writes along e_0 with beta 1; later keys avoid e_0, so only the decay touches that row; the last query reads e_0
    k[:, :, 0] = 0.0
    k[3] = 0.0
    k[3, 0, 0] = 1.0
    beta[3] = 1.0
    q[-1] = 0.0
    q[-1, 0, 0] = 1.0
    pb = seqmix.PackedBatch([0, T], [1], device)
    state = torch.zeros(3, H, d, dv, device=device)
    state[0] = 7.0                                                           # another sequence's row must stay untouched
    out = seqmix.delta_rule_scan(q.to(device), k.to(device), v.to(device), log_decay.to(device), beta.to(device), pb, state,
                                 unit_eps=None, q_scale=1.0)
    want = oracle.delta_rule_loop(q.double(), k.double(), v.double(), torch.exp(log_decay.double()), beta.double())
    close(out, want, 1e-5)
    kept = torch.exp(log_decay[4:, :, 0].sum(0))                             # what the decays left of the write
    close(out[-1], v[3] * kept.view(H, 1), 1e-4)
    assert bool((state[0] == 7.0).all()) and bool((state[2] == 0.0).all())
    # the same scan cut into two steps carries the memory in its row
    state2 = torch.zeros(3, H, d, dv, device=device)
    parts = []
    for a, b in ((0, 131), (131, T)):
        parts.append(seqmix.delta_rule_scan(q[a:b].to(device), k[a:b].to(device), v[a:b].to(device), log_decay[a:b].to(device),
                                            beta[a:b].to(device), seqmix.PackedBatch([0, b - a], [1], device), state2,
                                            unit_eps=None, q_scale=1.0))
    close(torch.cat(parts), want, 1e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_mlstm_gates_with_large_and_small_maxima(device):
    """Input gates far above and far below the running maximum; a fresh sequence begins with maximum 0, so tiny early gates
    must be weighed against e^0 and not against themselves."""
    T, H, d, dv = 70, 2, 12, 66
    g = torch.Generator().manual_seed(2)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, H, d, generator=g), torch.randn(T, H, dv, generator=g)
    log_i = torch.randn(T, H, generator=g) * 4.0
    log_i[:5] = -9.0                                                         # below the initial maximum: e^(-m) dominates
    log_i[40] = 12.0
    log_f = -torch.rand(T, H, generator=g)
    pb = seqmix.PackedBatch([0, 33, T], [2, 0], device)                    # two sequences, rows out of order
    S, n, m = (torch.zeros(3, H, d, dv, device=device), torch.zeros(3, H, d, device=device), torch.zeros(3, H, device=device))
    out = seqmix.mlstm_scan(q.to(device), k.to(device), v.to(device), log_i.to(device), log_f.to(device), pb, S, n, m, 0.5)
    for a, b in ((0, 33), (33, T)):
        want = oracle.mlstm_loop(q[a:b].double() * 0.5, k[a:b].double(), v[a:b].double(), log_i[a:b].double(), log_f[a:b].double())
        close(out[a:b], want, 1e-5)
    assert float(m[1].abs().max()) == 0.0 and float(m[2].abs().max()) > 0.0


@pytest.mark.parametrize("device", DEVICES)
def test_short_convolution_window_across_steps_of_one_and_two_tokens(device):
    C, taps, T = 10, 4, 23
    g = torch.Generator().manual_seed(3)
    x, w = torch.randn(T, C, generator=g), torch.randn(C, taps, generator=g)
    want = oracle.short_conv_silu(x.double(), w.double())
    for cuts in ([T], [1] * T, [2] * 12, [3, 1, 2, 17]):
        window = torch.zeros(2, taps - 1, C, device=device)
        parts, at = [], 0
        for n in cuts:
            n = min(n, T - at)
            if n:
                parts.append(seqmix.causal_conv_silu(x[at:at + n].to(device), w.to(device), seqmix.PackedBatch([0, n], [1], device),
                                                     window))
            at += n
        close(torch.cat(parts), want, 1e-5)
        assert float(window[0].abs().max()) == 0.0


@pytest.mark.parametrize("device", DEVICES)
def test_group_limited_router_keeps_the_best_groups_only(device):
    E, G = 12, 4
    z = torch.full((3, E), -2.0)
    z[0, 0], z[0, 1], z[0, 2] = 3.0, 2.9, 2.8         # group 0 holds the three largest; group 2 the fourth
    z[0, 7] = 2.0
    z[1, 11], z[1, 3], z[1, 6], z[1, 10] = 1.0, 0.9, 0.8, -1.0      # three groups compete for two places: expert 6 loses to 10
    z[2] = torch.arange(E).float() * 0.1
    probs, rmap = seqmix.group_limited_router(z.to(device), 3, G, 2)
    s = torch.softmax(z.double(), -1)
    for t in range(3):
        ids, w = oracle.route(z[t].double(), 3, G, 2)
        assert sorted(ids) == rmap[t].nonzero().flatten().tolist()
        close(probs[t, ids], w, 1e-6)
    assert rmap[0].nonzero().flatten().tolist() == [0, 1, 2]
    assert rmap[1].nonzero().flatten().tolist() == [3, 10, 11]
    raw, _ = seqmix.group_limited_router(z.to(device), 3, G, 2, renormalize=False)
    close(raw[0, [0, 1, 2]], s[0, [0, 1, 2]], 1e-6)


def test_config_rejects_a_latent_source_that_owns_nothing():
    bad = config_of([layer(LAT, kv_from=1), layer(LAT, kv_from=0)])
    with pytest.raises(ValueError):
        ZikunexConfig.from_dict(bad)


# ---------------------------------------------------------------------------------------------------------------------
# model folder -> registry -> trace runner / generation command line
# ---------------------------------------------------------------------------------------------------------------------
def write_model_folder(path, cfg, W):
    """``config.json`` + ``model.safetensors`` (bf16 tensors; 8-byte header length, JSON header, raw data)."""
    import json
    import struct

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
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = config_of([layer(DELTA, MOE_A), layer(LAT), layer(MLSTM_B, {"kind": "dense", "ff": 40}), layer(LAT, kv_from=1)])
    W = {k: v.to(torch.bfloat16).float() for k, v in oracle.random_weights(cfg, 5, low_rank=12).items()}
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
    got = {n: torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, 96).copy()) for n in (0, 1, 2, 3)}
    close(got[0], torch.stack([wa[0], wa[7], wa[15], wb[3]]), TOL[torch.float32])
    close(got[1], wb[4:5], TOL[torch.float32])
    close(got[2], torch.stack([wa[17], wb[5]]), TOL[torch.float32])
    close(got[3], wa[18:19], TOL[torch.float32])
    # the generation command line on the same folder: greedy tokens of the oracle
    r = subprocess.run([sys.executable, os.path.join(root, "tools", "run_text_generation_server.py"), "--model-dir", str(tmp_path),
                        "--dtype", "float32", "--prompts", " ".join(map(str, b)), "--num-tokens-to-generate", "4"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    toks = list(b)
    for _ in range(4):
        toks.append(int(oracle.forward(cfg, W, toks)[-1].argmax()))
    assert r.stdout.strip().splitlines()[-1].endswith("-> " + repr(" ".join(map(str, toks[len(b):]))))
