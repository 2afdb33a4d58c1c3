"""One prompt in panels and a few decoded tokens of a bench model of koifish_b200/bench_arch.py: the workload for launch lists and
single-kernel captures under ncu (few launches, nothing timed here).

    python tools/arch_prompt_run.py [--arch kivorax|kivorax_dense|sedotar|fazolorn|sipazen] [--size m] [--prompt 2048] [--panel 512] [--decode 3] [--window]

--window: the profiler range (cudaProfilerStart / Stop) covers the last panel and the decoded tokens only, for `ncu --profile-from-start off`.
"""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import koifish_b200 as kf  # noqa: E402
from koifish_b200 import bench_arch as B  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--arch", default="kivorax", choices=["kivorax", "kivorax_dense", "sedotar", "fazolorn", "sipazen"])
ap.add_argument("--size", default="m")
ap.add_argument("--prompt", type=int, default=2048)
ap.add_argument("--panel", type=int, default=512)
ap.add_argument("--decode", type=int, default=3)
ap.add_argument("--window", action="store_true")
args = ap.parse_args()
p = B.PRESETS[args.size]
ctx = kf.Context(0)
cfg = {"kivorax": B.kivorax_config, "kivorax_dense": B.kivorax_dense_config, "sedotar": B.sedotar_config, "fazolorn": B.fazolorn_config,
       "sipazen": B.sipazen_config}[args.arch](p)
model = kf.Model(ctx, {"hf_config": cfg, "gpt": {"max_seq_len": args.prompt + 64, "max_batch": 1, "max_prefill": args.panel},
                       "init": {"sigma": 0.02, "norm_sigma": 0.02}})
model.init_random()
if args.arch in ("kivorax", "kivorax_dense"):
    B.kivorax_fixups(model, cfg)
if args.window:
    import torch
print("launches before the prompt", ctx.launches)
toks = ((np.arange(args.prompt) * 37 + 11) % p["vocab"]).astype(np.int32)
for lo in range(0, args.prompt, args.panel):
    part = toks[lo:lo + args.panel]
    if args.window and lo + args.panel >= args.prompt:
        ctx.sync()
        print("launches before the last panel", ctx.launches)
        torch.cuda.profiler.start()
    model.forward(part, np.arange(lo, lo + part.size), seq_mode=2, want_logits=False, want_next=lo + args.panel >= args.prompt)
print("launches after the prompt", ctx.launches)
for i in range(args.decode):
    model.forward(np.array([5], dtype=np.int32), np.array([args.prompt + i]), seq_mode=2, want_logits=False, want_next=True)
print("launches at the end", ctx.launches)
if args.window:
    ctx.sync()
    torch.cuda.profiler.stop()
