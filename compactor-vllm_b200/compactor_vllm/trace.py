"""Trace replay: feed given token ids through the engine step by step and write the logits it is asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N  < steps.jsonl

Every input line is one engine step, `{"step": n, "entries": [{"id", "tokens", "want"}...], "end": [ids]}`: all
entries run as ONE batch through `ModelRunner.run_step` (portions of prompts beside single tokens), continuing from
the cache earlier steps left; `want` lists the places among an entry's tokens whose logits go to OUT/<n>.f32
(little-endian fp32 [wanted, vocab], in entry order); requests in `end` give their slot and pages back.  After each
step `done <n>` is printed.  Nothing is sampled.  The cache pool holds --max-tokens tokens (per request rounded up to
whole pages) and four slots, so pages and slots are reused as requests come and go.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_SIZE = 64
MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens the cache pool holds")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    a = ap.parse_args(argv)

    import numpy as np
    import torch

    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.core.model_runner import ModelRunner
    from compactor_vllm.utils.sequence import Sequence

    if not torch.cuda.is_available():
        print("trace_run needs a CUDA device (there is no CPU path)", file=sys.stderr)
        return 2
    ps = int(a.page_size)
    # a request's share of --max-tokens is rounded to 64; with larger pages each live request may need one more
    pages = -(-a.max_tokens // ps) + (MAX_LIVE if ps > 64 else 0)
    cfg = LLMConfig(model=a.model, path=a.model, dtype=a.dtype, max_num_seqs=MAX_LIVE, kvcache_page_size=ps,
                    max_model_len=pages * ps)
    runner = ModelRunner(cfg, num_pages=pages, device_allocator=False)
    if not runner.mixed_steps:
        print(f"model type {cfg.hf_config.model_type!r} cannot run portions of prompts", file=sys.stderr)
        return 2
    os.makedirs(a.out, exist_ok=True)
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries, rows, base = [], [], 0
        for e in step.get("entries", []):
            seq = live.get(e["id"])
            if seq is None:
                seq = live[e["id"]] = Sequence(prompt_token_ids=[])
            toks = [int(t) for t in e["tokens"]]
            seq.prompt_token_ids.extend(toks)
            entries.append((seq, toks))
            rows.extend(base + int(w) for w in e.get("want", []))
            base += len(toks)
        if entries:
            logits = runner.run_step(entries, rows if rows else [0])
            if rows:
                arr = logits.float().cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(a.out, f".{step['step']}.part")
                with open(tmp, "wb") as f:
                    f.write(np.ascontiguousarray(arr).tobytes())
                os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        ended = [live.pop(i) for i in step.get("end", []) if i in live]
        if ended:
            runner.release(ended)
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
