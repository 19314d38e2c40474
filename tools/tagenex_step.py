"""One prefill step and a few decode steps of a Tagenex model at layer sizes of a real model (random weights), for profiling:
    python tools/tagenex_step.py [--layers 2] [--batch 2] [--prompt 1024] [--decode 2] [--moe]
Small by default (two layers, 2 x 1024 tokens) so that an ncu capture of one kernel ends quickly."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402
import phi3_b200  # noqa: E402,F401
from phi3_b200 import weights  # noqa: E402
from phi3_b200.engine import Engine  # noqa: E402
from phi3_b200.tagenex import TagenexB200  # noqa: E402
from bench import _tagenex_cfg  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--layers', type=int, default=2)
    ap.add_argument('--batch', type=int, default=2)
    ap.add_argument('--prompt', type=int, default=1024)
    ap.add_argument('--decode', type=int, default=2)
    ap.add_argument('--moe', action='store_true')
    a = ap.parse_args()
    cfg = _tagenex_cfg(3072, 32, 8, 96, 8192, a.layers, 1024, 32064, a.moe)
    m = TagenexB200(cfg, weights.random_tagenex_weights(cfg, 0, device='cuda'), dtype=torch.bfloat16)
    eng = Engine(m, a.batch * (a.prompt + 64 + a.decode), a.batch)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32064, (a.prompt,), generator=g).tolist() for _ in range(a.batch)]
    eng.step([(i, prompts[i], [a.prompt - 1]) for i in range(a.batch)])
    for s in range(a.decode):
        eng.step([(i, [s + 1], [0]) for i in range(a.batch)])
    torch.cuda.synchronize()
    print('ok')


if __name__ == '__main__':
    main()
