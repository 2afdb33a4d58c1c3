"""Prefill and decode throughput of a hybrid stack (bench.py --compare-arch sipazen | kivorax | sedotar | fazolorn) beside the closest existing
models at equal width, depth and active feed-forward width: Sipazen beside Qwen3; Kivorax beside Sipazen (the other recurrence + attention +
experts stack of this runtime) and Qwen3; Sedotar (sliding-window attention beside a delta rule, dense feed-forward) beside Kivorax with
dense feed-forwards (delta-rule layers and attention layers alternating) and Qwen3; Fazolorn (minGRU, sigmoid block attention and latent
attention layers with routed experts) beside Sipazen (state-space and latent attention layers with routed experts) and Qwen3.  All bf16
with random weights.  One JSON line per (model, size).

    prefill: a prompt of --prompt tokens through the model's own step function in panels, timed with CUDA events after 3 warm-up prompts
    decode : the device-resident greedy loop (one CUDA-graph replay per token) at context --prompt, after W warm-up tokens

The weights of every size exceed the 126 MB L2, so nothing is reused between steps.
"""
import json
import time

PRESETS = {
    # width, vocab, layers (m = state-space, a = latent attention), mixer sizes, experts
    "s": dict(width=1024, vocab=32768, pattern="mmamma",
              ssm=dict(heads=32, vdim=64, state=64, groups=1, norm_groups=1, conv=4),
              att=dict(heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256),
              moe=dict(experts=16, top=2, ff=512, shared=1024),
              kvx=dict(pattern="ddgpdg", heads=8, dim=64, rank=32),
              sdt=dict(heads=8, kv_heads=2, window=1024, ff=4096)),
    "m": dict(width=2048, vocab=65536, pattern="mmammama",
              ssm=dict(heads=64, vdim=64, state=128, groups=8, norm_groups=8, conv=4),
              att=dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512),
              moe=dict(experts=64, top=6, ff=1408, shared=2816),
              kvx=dict(pattern="ddgpddgp", heads=16, dim=64, rank=64),
              sdt=dict(heads=16, kv_heads=4, window=1024, ff=8192)),
    "l": dict(width=4096, vocab=65536, pattern="mmam",
              ssm=dict(heads=128, vdim=64, state=128, groups=8, norm_groups=8, conv=4),
              att=dict(heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512),
              moe=dict(experts=32, top=4, ff=2048, shared=4096),
              kvx=dict(pattern="dgpd", heads=32, dim=64, rank=64),
              sdt=dict(heads=32, kv_heads=8, window=2048, ff=16384)),
}


def sipazen_config(p):
    layers = []
    for ch in p["pattern"]:
        if ch == "m":
            mixer, typ = dict(p["ssm"]), "mamba2"
        else:
            a = p["att"]
            mixer, typ = dict(a, rot=dict(base=1e6, dims=a["rot_dim"]), scale=(a["dim"] + a["rot_dim"]) ** -0.5), "latent_attention"
        m = p["moe"]
        layers.append({"type": typ, "mixer": mixer,
                       "mlp": {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"]}, "expert": {"ff": m["ff"]}, "shared": {"ff": m["shared"]}}})
    return {"architecture": "Sipazen", "vocab": p["vocab"], "width": p["width"], "residual_mult": 0.7, "norm": {"eps": 1e-5, "groups": 4}, "layers": layers}


def kivorax_config(p):
    """layers d = gated delta rule, g = gated linear attention, p = attention beside a gated LRU; the first layer's feed-forward is dense"""
    w, m, k = p["width"], p["moe"], p["kvx"]
    layers = []
    for i, ch in enumerate(k["pattern"]):
        if ch == "d":
            mixer, typ = dict(heads=k["heads"], kv_heads=k["heads"] // 2, dim=k["dim"], vdim=2 * k["dim"], conv=4, a_rank=k["rank"], g_rank=k["rank"]), "channel_delta"
        elif ch == "g":
            mixer, typ = dict(heads=k["heads"], dim=k["dim"], vdim=2 * k["dim"], tau=8.0, a_rank=k["rank"]), "gla"
        else:
            mixer = dict(left=dict(heads=k["heads"], kv_heads=max(1, k["heads"] // 4), dim=128, vdim=128, scale=128 ** -0.5, q_temp=dict(coef=0.4, every=512)),
                         right=dict(width=w, blocks=k["heads"], conv=4))
            typ = "parallel"
        mlp = {"kind": "dense", "ff": m["top"] * m["ff"]} if i == 0 else {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"]}, "expert": {"ff": m["ff"]}}
        layers.append({"type": typ, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Kivorax", "vocab": p["vocab"], "width": w, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "token_side": {"dim": 64}, "layers": layers}


def sedotar_config(p):
    """every layer: attention (head size 128, 4 query heads per kv head, half of each head rotated, window, cap 50, sink) beside the delta
    rule (as many value heads of 128, half as many key heads of 64), then the relu-gated feed-forward"""
    w, d = p["width"], p["sdt"]
    lf = dict(heads=d["heads"], kv_heads=d["kv_heads"], dim=128, vdim=128, conv=4, scale=128 ** -0.5, softcap=50.0, mask=dict(size=d["window"]),
              rot=dict(base=1e6, dims=64, scaling=dict(factor=4.0, original=8192, fast=16.0, slow=2.0)))
    rt = dict(heads=d["heads"], kv_heads=d["heads"] // 2, dim=64, vdim=128, conv=4)
    ly = {"type": "parallel", "mixer": {"left": lf, "right": rt, "left_scale": 0.7, "right_scale": 0.7}, "mlp": {"kind": "dense", "ff": d["ff"]}}
    return {"architecture": "Sedotar", "vocab": p["vocab"], "width": w, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "layers": [ly] * len(p["pattern"])}


def fazolorn_config(p):
    """as many layers as the preset's pattern, in the order sigmoid block attention (head size 128, 4 query heads per kv head, half of each
    head rotated, blocks of 1024 positions), minGRU (2 x width channels), latent attention (the preset's sizes, queries through a latent of
    1.5 x kv_rank, stretched frequencies); the first feed-forward dense and clamped, the others routed experts (the preset's count and top,
    4 groups of which 2 are kept) whose width makes the active width equal to the preset's experts + shared expert"""
    w, a, m = p["width"], p["att"], p["moe"]
    heads = w // 128
    ff = (m["ff"] + m["shared"] // m["top"] + 127) // 128 * 128
    mixers = [("attention", dict(heads=heads, kv_heads=max(1, heads // 4), dim=128, vdim=128, scale=128 ** -0.5, mask=dict(size=1024), rot=dict(base=1e6, dims=64))),
              ("mingru", dict(width=2 * w)),
              ("latent_attention", dict(a, q_rank=a["kv_rank"] * 3 // 2, scale=(a["dim"] + a["rot_dim"]) ** -0.5,
                                        rot=dict(base=1e6, dims=a["rot_dim"], scaling=dict(factor=4.0, original=8192, fast=16.0, slow=2.0))))]
    layers = []
    for i in range(len(p["pattern"])):
        typ, mixer = mixers[i % 3]
        mlp = {"kind": "dense", "ff": m["top"] * ff, "limit": 7.0} if i == 0 else \
            {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": m["experts"], "top": m["top"], "scale": 2.0, "groups": {"count": 4, "keep": 2}}}
        layers.append({"type": typ, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Fazolorn", "vocab": p["vocab"], "width": w, "norm": {"eps": 1e-5}, "logit_scale": 0.25,
            "loop": {"start": 0, "stop": len(layers), "times": 1}, "layers": layers}


def kivorax_dense_config(p):
    """Kivorax at the size of sedotar_config: delta-rule layers and attention (+ LRU) layers alternating, a dense feed-forward of the same
    width in every layer, no side input"""
    w, d = p["width"], p["sdt"]
    layers = []
    for i in range(len(p["pattern"])):
        if i % 2 == 0:
            mixer, typ = dict(heads=d["heads"], kv_heads=d["heads"] // 2, dim=64, vdim=128, conv=4, a_rank=64, g_rank=64), "channel_delta"
        else:
            mixer = dict(left=dict(heads=d["heads"], kv_heads=d["kv_heads"], dim=128, vdim=128, scale=128 ** -0.5, q_temp=dict(coef=0.4, every=512)),
                         right=dict(width=w, blocks=d["heads"], conv=4))
            typ = "parallel"
        layers.append({"type": typ, "mixer": mixer, "mlp": {"kind": "dense", "ff": d["ff"]}})
    return {"architecture": "Kivorax", "vocab": p["vocab"], "width": w, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "layers": layers}


def kivorax_fixups(model, cfg):
    """tensors that random normal weights would make meaningless: positive distance-penalty numbers, depth weights (0, .., 0, 1), unit norms"""
    import numpy as np
    import torch

    def bits(a):
        return (torch.tensor(np.asarray(a, dtype=np.float32)).view(torch.int32).numpy().astype(np.uint32) >> 16).astype(np.uint16)
    for i, ly in enumerate(cfg["layers"]):
        model.set_tensor("l%d.dwa" % i, bits([0.0] * (i + 1) + [1.0]))
        if ly["type"] == "parallel":
            h = ly["mixer"]["left"]["heads"]
            model.set_tensor("l%d.mix.left.r1" % i, bits([0.5] * h))
            model.set_tensor("l%d.mix.left.r2" % i, bits([0.25] * h))


def run(args, ctx, stream):
    import numpy as np
    import torch
    import koifish_b200 as kf
    sizes = [s for s in args.arch_sizes.split(",") if s]
    P, panel = args.prompt, args.panel
    out = []
    for size in sizes:
        p = PRESETS[size]
        n_layer = len(p["pattern"])
        ff_active = p["moe"]["top"] * p["moe"]["ff"] + p["moe"]["shared"]
        cfgs = {}
        gpt = {"max_seq_len": P + args.steps + args.warmup + 64, "max_batch": 1, "max_prefill": panel}
        if args.compare_arch == "sedotar":
            kcfg = kivorax_dense_config(p)
            ff_active = p["sdt"]["ff"]
            cfgs["sedotar"] = {"hf_config": sedotar_config(p), "gpt": dict(gpt), "init": {"sigma": 0.02, "norm_sigma": 0.02}}
            cfgs["kivorax"] = {"hf_config": kcfg, "gpt": dict(gpt), "init": {"sigma": 0.02, "norm_sigma": 0.02}}
        if args.compare_arch == "kivorax":
            kcfg = kivorax_config(p)
            cfgs["kivorax"] = {"hf_config": kcfg, "gpt": {"max_seq_len": P + args.steps + args.warmup + 64, "max_batch": 1, "max_prefill": panel},
                               "init": {"sigma": 0.02, "norm_sigma": 0.02}}
        if args.compare_arch == "fazolorn":
            cfgs["fazolorn"] = {"hf_config": fazolorn_config(p), "gpt": dict(gpt), "init": {"sigma": 0.02, "norm_sigma": 0.02}}
        if args.compare_arch != "sedotar":
            cfgs["sipazen"] = {"hf_config": sipazen_config(p), "gpt": {"max_seq_len": P + args.steps + args.warmup + 64, "max_batch": 1, "max_prefill": panel},
                               "init": {"sigma": 0.02, "norm_sigma": 0.02}}
        cfgs["qwen3"] = kf.qwen3_config(n_layer, p["width"], (ff_active + 127) // 128 * 128, p["width"] // 128, max(1, p["width"] // 512), 128, p["vocab"], None, False,
                                        P + args.steps + args.warmup + 64, 1, 42, 1e6, max_prefill=panel)
        for name, cfg in cfgs.items():
            model = kf.Model(ctx, cfg)
            model.init_random()
            if name == "kivorax":
                kivorax_fixups(model, kcfg)
            toks = ((np.arange(P) * 37 + 11) % p["vocab"]).astype(np.int32)

            def prompt():
                nxt = None
                for lo in range(0, P, panel):
                    part = toks[lo:lo + panel]
                    last = lo + panel >= P
                    _, nxt = model.forward(part, np.arange(lo, lo + part.size), seq_mode=2, want_logits=False, want_next=last)
                return nxt

            for _ in range(3):
                prompt()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps, l0 = 3, ctx.launches
            e0.record(stream)
            for _ in range(reps):
                nxt = prompt()
            e1.record(stream)
            torch.cuda.synchronize()
            prefill_ms = e0.elapsed_time(e1) / reps
            prefill_launches = (ctx.launches - l0) / reps
            model.decode_loop(max(3, args.warmup), 1)
            torch.cuda.synchronize()
            l0 = ctx.launches
            e0.record(stream)
            model.decode_loop(args.steps, 1)
            e1.record(stream)
            torch.cuda.synchronize()
            decode_ms = e0.elapsed_time(e1) / args.steps
            info = model.info
            line = {"bench": "arch-compare", "model": name, "size": size, "width": p["width"], "layers": n_layer, "pattern": p["pattern"] if name in ("sipazen", "qwen3") else "".join(ly["type"][0] for ly in cfg["hf_config"]["layers"]),
                    "weight_gb": round(info.weight_bytes / 1e9, 3), "prompt": P, "panel": panel,
                    "prefill_tok_s": round(P / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3), "prefill_launches": prefill_launches,
                    "decode_tok_s": round(1e3 / decode_ms, 1), "decode_ms": round(decode_ms, 4), "decode_launches_per_token": (ctx.launches - l0) / args.steps,
                    "dtype": "bf16", "data": "synthetic", "steps": args.steps, "warmup": max(3, args.warmup), "timing": "cuda events, weights exceed L2"}
            print(json.dumps(line), flush=True)
            out.append(line)
            model.close()
            time.sleep(0.1)
    return out
