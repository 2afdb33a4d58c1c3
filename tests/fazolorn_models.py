"""Small random Fazolorn models for the tests: layer cards, a config.json, weights drawn on the bf16 grid (optionally shaped so that a
fault shows), bf16 bit patterns, random token lists."""
import numpy as np
import torch


def gru(width=40):
    return "mingru", {"width": width}


def attn(heads=4, kv_heads=2, dim=12, block=9, rot_dims=8, base=10000.0, scale=None, scaling=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale or dim ** -0.5)
    if block:
        m["mask"] = {"size": block}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = scaling
    return "attention", m


def latent(heads=3, dim=10, rot_dim=6, vdim=9, kv_rank=20, q_rank=14, base=10000.0, scaling=True, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale or (dim + rot_dim) ** -0.5)
    m["rot"] = {"base": base, "dims": rot_dim}
    if scaling:
        m["rot"]["scaling"] = scaling if isinstance(scaling, dict) else {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    return "latent_attention", m


def dense(ff=40, limit=1.25):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=6, top=2, ff=12, groups=(3, 2), scale=1.7):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def layer(mixer, mlp=None):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def config(layers, width=48, vocab=96, eps=1e-5, logit_scale=0.6, loop=None):
    c = {"architecture": "Fazolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": list(layers)}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def bf16_grid(t):
    return t.to(torch.bfloat16).to(torch.float32)


def weights(cfg, seed=0, q_gain=1.0, pb=0.0, z_bias=0.0, correction=0.3):
    """q_gain scales the query projections (weights near 0 or 1 in the sigmoid attention, a peaked softmax in the latent attention), pb shifts
    the per-head bias inside the sigmoid, z_bias the update gate of the recurrence (very negative: the state barely moves), correction is
    the spread of the router's selection correction"""
    g = torch.Generator().manual_seed(seed)
    E, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, r, c, s=None):
        W[name] = bf16_grid(torch.randn(r, c, generator=g) * (s if s is not None else c ** -0.5))

    def vec(name, n, mean=0.0, s=0.3):
        W[name] = bf16_grid(mean + s * torch.randn(n, generator=g))

    mat("embed", V, E, 1.0)
    mat("head", V, E)
    vec("final.norm", E, 1.0, 0.2)
    if cfg.get("loop"):
        mat("loop.step", cfg["loop"]["times"], E, 0.5)
    for i, ly in enumerate(cfg["layers"]):
        p, m, q = "l%d." % i, ly["mixer"], "l%d.mix." % i
        vec(p + "norm1", E, 1.0, 0.2)
        if ly["type"] == "mingru":
            n = m["width"]
            mat(q + "z", n, E), vec(q + "z.b", n, z_bias, 0.5)
            mat(q + "x", n, E), vec(q + "x.b", n, 0.0, 0.5)
            mat(q + "g", n, E), mat(q + "o", E, n)
        elif ly["type"] == "attention":
            H, G, dk = m["heads"], m.get("kv_heads") or m["heads"], m["dim"]
            mat(q + "q", H * dk, E, q_gain * E ** -0.5), vec(q + "q.b", H * dk, 0.0, 0.3 * q_gain)
            mat(q + "k", G * dk, E), vec(q + "k.b", G * dk, 0.0, 0.3)
            vec(q + "pb", H, pb, 0.5)
            mat(q + "o", E, H * dk, 0.5 * (H * dk) ** -0.5)
        else:
            H, dn, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            mat(q + "dq", Q, E), vec(q + "dq.norm", Q, 1.0, 0.2)
            mat(q + "uq", H * (dn + dr), Q, q_gain * Q ** -0.5)
            mat(q + "dkv", R + dr, E), vec(q + "dkv.norm", R, 1.0, 0.2)
            mat(q + "uk", H * dn, R), mat(q + "uv", H * dv, R)
            mat(q + "o", E, H * dv)
        f = ly.get("mlp")
        if not f:
            continue
        vec(p + "norm2", E, 1.0, 0.2)
        if f["kind"] == "dense":
            mat(p + "mlp.gate", f["ff"], E, 2.0 * E ** -0.5), mat(p + "mlp.up", f["ff"], E, 2.0 * E ** -0.5), mat(p + "mlp.down", E, f["ff"])
        else:
            X, F = f["router"]["experts"], f["expert"]["ff"]
            mat(p + "mlp.router", X, E, 2.0 * E ** -0.5)
            vec(p + "mlp.correction", X, 0.0, correction)
            for e in range(X):
                mat("%smlp.e%d.gate" % (p, e), F, E), mat("%smlp.e%d.up" % (p, e), F, E), mat("%smlp.e%d.down" % (p, e), E, F)
    return W


def bits(t):
    return (t.contiguous().view(torch.int32).numpy().astype(np.uint32) >> 16).astype(np.uint16)


def tokens(n, vocab, seed):
    return np.random.RandomState(seed).randint(0, vocab, n).tolist()
