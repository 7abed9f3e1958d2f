"""Command line of the layer-list serving path:

    python -m blazr_b200 generate --model DIR --prompt 1,2,3 [--prompt ...] [--max-new N] [--temperature T] [--top-k K] [--top-p P]
    python -m blazr_b200 trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N     (also bin/trace_run)

`trace` replays externally scheduled steps through the engine: one JSON object per line on standard input,
    {"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [ids]}
runs all entries of a step as one batch from the cache and state the earlier steps left, writes the logits of the wanted places
to <out>/<step>.f32 (little-endian f32 [wanted, vocab], entry order) when any are wanted, and prints "done <step>".
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _load(path: str, dtype: str):
    import torch

    from . import registry
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: this framework has no CPU path")
    return registry.load_model(path, "cuda:0", dtype)


def cmd_trace(a) -> int:
    from . import seqops
    from .engine import Engine
    model = _load(a.model, a.dtype)
    eng = Engine(model, max_tokens=a.max_tokens, max_seqs=a.max_seqs, block_size=a.block_size)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        req = json.loads(line)
        logits = eng.run_entries(req.get("entries", []), req.get("end", []))
        if logits is not None:
            tmp = os.path.join(a.out, f".{req['step']}.part")
            with open(tmp, "wb") as f:
                f.write(logits.astype("<f4", copy=False).tobytes())
            os.replace(tmp, os.path.join(a.out, f"{req['step']}.f32"))
        sys.stdout.write(f"done {req['step']}\n")
        sys.stdout.flush()
    flags = seqops.error_flags()
    if flags:
        print(f"device error flags {flags:#x}", file=sys.stderr)
        return 1
    return 0


def cmd_generate(a) -> int:
    from .engine import Engine, SamplingParams
    model = _load(a.model, a.dtype)
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt]
    need = sum(-(-(len(p) + a.max_new) // a.block_size) * a.block_size for p in prompts[:a.max_seqs]) if a.max_tokens <= 0 else a.max_tokens
    eng = Engine(model, max_tokens=need, max_seqs=a.max_seqs, block_size=a.block_size)
    outs = eng.generate(prompts, SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, seed=a.seed, max_new_tokens=a.max_new))
    for p, o in zip(prompts, outs):
        print(json.dumps({"prompt": p, "tokens": o}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="blazr_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("trace", "generate"):
        p = sub.add_parser(name)
        p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
        p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
        p.add_argument("--max-seqs", type=int, default=4, help="state slots: most requests live at a time")
        p.add_argument("--block-size", type=int, default=16, help="tokens per KV page")
        if name == "trace":
            p.add_argument("--out", required=True)
            p.add_argument("--max-tokens", type=int, required=True, help="tokens the KV pool holds")
        else:
            p.add_argument("--prompt", action="append", required=True, help="token ids with commas; may be repeated")
            p.add_argument("--max-new", type=int, default=16)
            p.add_argument("--max-tokens", type=int, default=0, help="tokens the KV pool holds (0: sized for the prompts)")
            p.add_argument("--temperature", type=float, default=0.0)
            p.add_argument("--top-k", type=int, default=0)
            p.add_argument("--top-p", type=float, default=1.0)
            p.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    return cmd_trace(a) if a.cmd == "trace" else cmd_generate(a)
