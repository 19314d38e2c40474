"""Trace replay: feed given token ids through a model step by step and write the logits of chosen positions. Nothing is sampled.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   < steps.jsonl

Every input line is one engine step, {"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}, ...], "end": [...]}:
all entries run as one batch through engine.Engine.step (the step function generation uses), against a page pool of N tokens and
four sequence slots; requests listed under "end" give their pages and slot back after the step. For a step that wants logits
the rows are written to DIR/<step>.f32 (little-endian fp32, [wanted, vocab], in entry and want order); after every step the line
"done <step>" is printed. The model class follows config.json (registry.py).
"""
import argparse
import json
import os
import sys


def main(argv=None):
    ap = argparse.ArgumentParser(prog='trace_run', description=__doc__.split('\n')[0])
    ap.add_argument('--model', required=True, help='folder with config.json and model.safetensors')
    ap.add_argument('--dtype', default='bfloat16', choices=['bfloat16', 'float32'])
    ap.add_argument('--out', required=True)
    ap.add_argument('--max-tokens', type=int, required=True, help='tokens the page pool holds')
    ap.add_argument('--slots', type=int, default=4, help='sequences that can be live at once')
    a = ap.parse_args(argv)
    from . import _lib
    _lib.ensure_built(full=False)
    import torch
    from . import registry
    from .engine import Engine
    model = registry.load_model(a.model, dtype=getattr(torch, a.dtype))
    if not hasattr(model, 'forward') or not hasattr(model, 'kv_layout'):
        print(f'{type(model).__name__} does not run on the continuous-batching engine', file=sys.stderr)
        return 3
    eng = Engine(model, a.max_tokens, a.slots)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        s = json.loads(line)
        entries = [(e['id'], e['tokens'], e.get('want', [])) for e in s['entries']]
        logits = eng.step(entries, s.get('end', []))
        if logits is not None:
            data = logits.to('cpu', torch.float32).contiguous().numpy().astype('<f4', copy=False)
            tmp = os.path.join(a.out, f".{s['step']}.part")
            with open(tmp, 'wb') as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, f"{s['step']}.f32"))
        else:
            torch.cuda.synchronize()
        sys.stdout.write(f"done {s['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == '__main__':
    sys.exit(main())
