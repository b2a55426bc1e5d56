"""Replay of a token trace through the dynamic engine: given token ids go in step by step, logits come out.

Nothing is sampled.  Every step is one call of ``DynamicInferenceEngine.forward_tokens`` -- the forward the engine's own
``step()`` runs -- over the packed batch of the step's entries, against the paged cache and the recurrent state rows the
earlier steps left; finished requests give their pages and rows back.  Used by ``bin/trace_run`` to check a model's
numerics under a serving schedule (whole prompts, prompts cut into portions, decoding, mixed batches).

Protocol: one JSON object per input line,
``{"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [ids]}``; for a step with wanted
positions ``<out>/<n>.f32`` receives their logits (little-endian fp32, ``[wanted, vocab]``, in entry / want order);
``done <n>`` is printed after every step.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Iterable, Optional

import torch

from .dynamic import DynamicInferenceEngine


class TraceReplayer:
    def __init__(self, model, max_tokens: int, block_size: int = 16, max_requests: int = 256,
                 max_sequence_length: Optional[int] = None):
        from ..data.tokenizer import NullTokenizer

        blocks = -(-max_tokens // block_size) + max_requests          # every request may leave its last page half empty
        self.engine = DynamicInferenceEngine(model, NullTokenizer(max(1, getattr(model, "vocab_size", 2) - 1)),
                                             max_sequence_length=max_sequence_length or max_tokens, num_blocks=blocks,
                                             block_size=block_size, max_tokens_per_step=max_tokens, max_requests=max_requests)
        self.live = set()

    def step(self, entries, end=()) -> Optional[torch.Tensor]:
        """Run one step; returns the logits ``[wanted, vocab]`` (fp32, on the host) or ``None`` if nothing is wanted."""
        ctx = self.engine.context
        work = []
        for e in entries:
            if e["id"] not in self.live:
                ctx.add_request(e["id"])
                self.live.add(e["id"])
            if e["tokens"]:
                work.append((e["id"], list(e["tokens"])))
        out = None
        if work:
            logits, _ = self.engine.forward_tokens(work)
            rows, base = [], 0
            for e in entries:
                rows += [base + int(w) for w in e.get("want", ())]
                base += len(e["tokens"])
            if rows:
                idx = torch.tensor(rows, dtype=torch.long, device=logits.device)
                out = logits.index_select(0, idx).float().cpu()
        for rid in end:
            if rid in self.live:
                ctx.release(rid)
                self.live.discard(rid)
        return out


def replay(model, lines: Iterable[str], out_dir: str, max_tokens: int, report=None) -> int:
    """Feed the JSON ``lines`` through ``model``; returns the number of steps run."""
    rp = TraceReplayer(model, max_tokens)
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        out = rp.step(st.get("entries", []), st.get("end", []))
        if out is not None:
            tmp = os.path.join(out_dir, f".{st['step']}.f32.part")
            with open(tmp, "wb") as f:
                f.write(out.contiguous().numpy().astype("<f4", copy=False).tobytes())
            os.replace(tmp, os.path.join(out_dir, f"{st['step']}.f32"))
        if report is not None:
            report(st["step"])
        n += 1
    return n


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="replay a token trace through a model folder and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, default=4096)
    ap.add_argument("--device", default=None, help="default: cuda:0 if there is one")
    a = ap.parse_args(argv)
    torch.backends.cuda.matmul.allow_tf32 = False            # float32 means fp32 products
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    dev = a.device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    if dev.startswith("cuda"):
        torch.cuda.set_device(torch.device(dev))
    from ..models.registry import build_model_from_dir

    model = build_model_from_dir(a.model, torch.bfloat16 if a.dtype == "bfloat16" else torch.float32, dev)
    os.makedirs(a.out, exist_ok=True)

    def report(step):
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()

    with torch.no_grad():
        replay(model, sys.stdin, a.out, a.max_tokens, report)
    return 0


if __name__ == "__main__":
    sys.exit(main())
