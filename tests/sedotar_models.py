"""Small random Sedotar models for the tests: layer cards, a config.json, weights drawn on the bf16 grid (optionally shaped so that a
fault shows), bf16 bit patterns, random token lists."""
import numpy as np
import torch


def left(heads=4, kv_heads=2, dim=12, vdim=10, conv=3, window=9, softcap=20.0, rot_dims=8, base=10000.0, scaling=True, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, scale=scale or dim ** -0.5)
    if window:
        m["mask"] = {"size": window}
    if softcap:
        m["softcap"] = softcap
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = scaling if isinstance(scaling, dict) else {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    return m


def right(heads=4, kv_heads=2, dim=10, vdim=14, conv=2):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


def layer(l=None, r=None, ff=40, left_scale=0.7, right_scale=1.2):
    return {"type": "parallel", "mixer": {"left": l or left(), "right": r or right(), "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=48, vocab=96, eps=1e-5, scale=5.0):
    return {"architecture": "Sedotar", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": list(layers)}


def bf16_grid(t):
    return t.to(torch.bfloat16).to(torch.float32)


def weights(cfg, seed=0, q_gain=1.0, sink=0.0, a_log=-1.0, dt_bias=0.0):
    """q_gain scales the query norm weights (a peaked softmax), sink shifts the sinks, a_log / dt_bias set how fast the states decay"""
    g = torch.Generator().manual_seed(seed)
    E, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, r, c, s=None):
        W[name] = bf16_grid(torch.randn(r, c, generator=g) * (s if s is not None else c ** -0.5))

    def vec(name, n, mean=0.0, s=0.3):
        W[name] = bf16_grid(mean + s * torch.randn(n, generator=g))

    mat("embed", V, E, 1.0 / cfg["embedding"]["scale"])
    vec("final.norm", E, 0.0, 0.2)
    for i, ly in enumerate(cfg["layers"]):
        p, m = "l%d." % i, ly["mixer"]
        vec(p + "norm1", E, 0.0, 0.2)
        a, r = m["left"], m["right"]
        H, G, dk, dv = a["heads"], a.get("kv_heads") or a["heads"], a["dim"], a["vdim"]
        q = p + "mix.left."
        for n, c in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
            mat(q + n, c, E)
            mat(q + n + ".conv", c, a["conv"], 0.6)
        vec(q + "q.norm", H * dk, q_gain, 0.2 * q_gain)
        vec(q + "k.norm", G * dk, 1.0, 0.2)
        vec(q + "sink", H, sink, 0.5)
        mat(q + "o", E, H * dv)
        H, G, dk, dv = r["heads"], r.get("kv_heads") or r["heads"], r["dim"], r["vdim"]
        q = p + "mix.right."
        for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
            mat(q + n, c, E)
            mat(q + n + ".conv", c, r["conv"], 0.6)
        mat(q + "b", H, E), mat(q + "a", H, E)
        vec(q + "A_log", H, a_log, 0.3), vec(q + "dt_bias", H, dt_bias, 0.5)
        vec(q + "norm", dv, 1.0)
        mat(q + "g", H * dv, E), mat(q + "o", E, H * dv)
        if ly["mlp"]:
            vec(p + "norm2", E, 0.0, 0.2)
            F = ly["mlp"]["ff"]
            mat(p + "mlp.gate", F, E), mat(p + "mlp.up", F, E), mat(p + "mlp.down", E, F)
    return W


def bits(t):
    return (t.contiguous().view(torch.int32).numpy().astype(np.uint32) >> 16).astype(np.uint16)


def tokens(n, vocab, seed):
    return np.random.RandomState(seed).randint(0, vocab, n).tolist()
