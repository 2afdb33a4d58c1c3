"""Plain float64 restatement of the Fazolorn stack, one function per mechanism, token-by-token loops where a mechanism has a state or a mask.
It shares no code with the library: it is what the GPU tests compare the framework against.

    x_0 = embed[token];   layers a .. b-1 run n times in a row on the same weights (a cache / state of their own each time); before run
    t of them  x <- x + [t > 0] x_0 + step[t];   the other layers run once, in order
    layer:  x <- x + mixer(norm(x; w1));   x <- x + ff(norm(x; w2));   norm(y; w) = y / sqrt(mean(y^2) + eps) * w
    mingru:            z = sigmoid(W_z h + b_z), u = W_x h + b_x, c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0);  S <- (1 - z) S + z c;
                       out = W_o (S * silu(W_g h))
    attention:         q = W_q h + b_q, k = W_k h + b_k, v = k (before the rotation); rotate q, k in halves (i, i + dims/2);
                       w_ij = sigmoid(scale q_i . k_j + pb_h) for j <= i in the same block of `size` positions; out = W_o sum_j w_ij v_j
    latent_attention:  c_q = norm(W_dq h), q = W_uq c_q = [plain | rotated] per head;  W_dkv h = [c | r], c <- norm(c), r rotated in
                       neighbouring pairs (2i, 2i+1) with stretched frequencies; k = [W_uk c | r], v = W_uv c; causal softmax; W_o
    dense ff:          g = min(W_g h, L), u = clamp(W_u h, -L, L);  W_d (g sigmoid(1.702 g) (u + 1))
    experts:           s = sigmoid(W_r h); choice = s + correction; contiguous groups ranked by the sum of their top-2 choices, only
                       the best `keep` groups stay; the `top` largest choices are taken; weights scale_r * s (not renormalised);
                       expert = W_d (silu(W_g h) * W_u h)
    logits = logit_scale * W_head norm(x; w_final)
"""
import math

import torch

D = torch.float64


def rmsnorm(y, w, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w.to(D)


def silu(z):
    return z * torch.sigmoid(z)


def lin(W, name, h, bias=False):
    y = h @ W[name].to(D).T
    return y + W[name + ".b"].to(D) if bias else y


def frequencies(rot):
    """(f_i, amplitude) of a rotation over rot['dims'] entries; with rot['scaling'] a frequency is divided by `factor` where its wavelength
    is long, left alone where it is short, blended linearly between, and the amplitude grows with the logarithm of the factor"""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def index_of(turns):
        return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, pos, rot, halves):
    """x [heads, n] at position pos: the first rot['dims'] entries turn by pos * f_i, paired (i, i + dims/2) or (2i, 2i+1); the rest stay"""
    if not rot or not rot.get("dims"):
        return x
    f, amp = frequencies(rot)
    half = rot["dims"] // 2
    out = x.clone()
    for i, fi in enumerate(f):
        c, s = math.cos(pos * fi) * amp, math.sin(pos * fi) * amp
        ia, ib = (i, i + half) if halves else (2 * i, 2 * i + 1)
        a, b = x[:, ia], x[:, ib]
        out[:, ia] = a * c - b * s
        out[:, ib] = b * c + a * s
    return out


def mingru(h, m, W, p, pos0=0, state=None):
    """h [T, E]; returns (out [T, E], state after the last token)"""
    z = torch.sigmoid(lin(W, p + "z", h, True))
    u = lin(W, p + "x", h, True)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = silu(lin(W, p + "g", h))
    S = torch.zeros(m["width"], dtype=D) if state is None else state
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S * g[t])
    return torch.stack(rows) @ W[p + "o"].to(D).T, S


def block_attention(h, m, W, p):
    """sigmoid-weighted attention inside blocks of mask.size positions aligned to position 0; v = un-rotated k"""
    T = h.shape[0]
    H, dk = m["heads"], m["dim"]
    G = m.get("kv_heads") or H
    size = (m.get("mask") or {}).get("size", 0)
    q = lin(W, p + "q", h, True).view(T, H, dk)
    k = lin(W, p + "k", h, True).view(T, G, dk)
    qr = torch.stack([rotate(q[t], t, m.get("rot"), True) for t in range(T)])
    kr = torch.stack([rotate(k[t], t, m.get("rot"), True) for t in range(T)])
    pb = W[p + "pb"].to(D)
    out = torch.zeros(T, H, dk, dtype=D)
    for i in range(T):
        lo = (i // size) * size if size else 0
        for hh in range(H):
            g = hh // (H // G)
            s = (kr[lo:i + 1, g] @ qr[i, hh]) * m["scale"] + pb[hh]
            out[i, hh] = torch.sigmoid(s) @ k[lo:i + 1, g]
    return out.reshape(T, H * dk) @ W[p + "o"].to(D).T


def latent_attention(h, m, W, p, eps):
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rmsnorm(lin(W, p + "dq", h), W[p + "dq.norm"], eps)
    q = lin(W, p + "uq", cq).view(T, H, dn + dr)
    ckr = lin(W, p + "dkv", h)
    c = rmsnorm(ckr[:, :R], W[p + "dkv.norm"], eps)
    rot = m.get("rot")
    r = torch.stack([rotate(ckr[t:t + 1, R:], t, rot, False)[0] for t in range(T)])
    qrot = torch.stack([rotate(q[t, :, dn:], t, rot, False) for t in range(T)])
    kn = lin(W, p + "uk", c).view(T, H, dn)
    v = lin(W, p + "uv", c).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=D)
    for i in range(T):
        for hh in range(H):
            s = (kn[:i + 1, hh] @ q[i, hh, :dn] + r[:i + 1] @ qrot[i, hh]) * m["scale"]
            out[i, hh] = torch.softmax(s, 0) @ v[:i + 1, hh]
    return out.reshape(T, H * dv) @ W[p + "o"].to(D).T


def dense_ff(h, f, W, p):
    L = f["limit"]
    g = torch.clamp(lin(W, p + "gate", h), max=L)
    u = torch.clamp(lin(W, p + "up", h), -L, L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].to(D).T


def route(h, f, W, p, margins=None):
    """per token: (chosen experts, their weights); margins (a list) receives, per token, the smallest gap that decided anything -- between
    the last kept and the first dropped group, between the last chosen and the first rejected expert"""
    r = f["router"]
    X, top = r["experts"], r["top"]
    gr = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(lin(W, p + "router", h))
    choice = s + W[p + "correction"].to(D)
    per = X // gr["count"]
    picks = []
    for t in range(h.shape[0]):
        ch = choice[t].clone()
        score = [ch[g * per:(g + 1) * per].topk(min(2, per)).values.sum().item() for g in range(gr["count"])]
        kept = sorted(range(gr["count"]), key=lambda g: (-score[g], g))[:gr["keep"]]
        for g in range(gr["count"]):
            if g not in kept:
                ch[g * per:(g + 1) * per] = -math.inf
        order = sorted(range(X), key=lambda e: (-ch[e].item(), e))
        idx = order[:top]
        picks.append((idx, [s[t, e] * r["scale"] for e in idx]))
        if margins is not None:
            by_score = sorted(score, reverse=True)
            gap = by_score[gr["keep"] - 1] - by_score[gr["keep"]] if gr["keep"] < gr["count"] else math.inf
            if top < X and ch[order[top]] > -math.inf:
                gap = min(gap, (ch[order[top - 1]] - ch[order[top]]).item())
            margins.append(gap)
    return picks


def experts_ff(h, f, W, p, margins=None):
    out = torch.zeros_like(h)
    for t, (idx, wgt) in enumerate(route(h, f, W, p, margins)):
        for e, w in zip(idx, wgt):
            q = "%se%d." % (p, e)
            y = silu(lin(W, q + "gate", h[t])) * lin(W, q + "up", h[t])
            out[t] += w * (y @ W[q + "down"].to(D).T)
    return out


def layer_runs(cfg):
    """[(layer index, pass number or None)] in the order the layers run; a pass number marks the first layer of a repeated pass"""
    L = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp or lp["times"] < 1 or lp["stop"] <= lp["start"]:
        return [(i, None) for i in range(L)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], L)]


def forward(cfg, W, tokens, trace=None, margins=None):
    """logits [T, vocab] of one sequence from position 0; trace (a list) receives x after every layer run; margins (a list) one list of
    per-token routing gaps for every run of a layer with experts"""
    eps = cfg["norm"]["eps"]
    x0 = W["embed"].to(D)[torch.tensor(tokens)]
    x = x0.clone()
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"].to(D)[t]
        ly, p = cfg["layers"][i], "l%d." % i
        h = rmsnorm(x, W[p + "norm1"], eps)
        kind, m = ly["type"], ly["mixer"]
        if kind == "mingru":
            y = mingru(h, m, W, p + "mix.")[0]
        elif kind == "attention":
            y = block_attention(h, m, W, p + "mix.")
        else:
            y = latent_attention(h, m, W, p + "mix.", eps)
        x = x + y
        f = ly.get("mlp")
        if f:
            h = rmsnorm(x, W[p + "norm2"], eps)
            if f["kind"] == "dense":
                x = x + dense_ff(h, f, W, p + "mlp.")
            else:
                gaps = [] if margins is not None else None
                x = x + experts_ff(h, f, W, p + "mlp.", gaps)
                if margins is not None:
                    margins.append(gaps)
        if trace is not None:
            trace.append(x.clone())
    return rmsnorm(x, W["final.norm"], eps) @ W["head"].to(D).T * cfg.get("logit_scale", 1.0)
