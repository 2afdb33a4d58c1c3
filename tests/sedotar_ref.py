"""Plain float64 restatement of the Sedotar stack, one function per mechanism, token-by-token loops where a mechanism has a state.
It shares no code with the library: it is what the GPU tests compare the framework against.

    x_0 = scale_e * embed[token]
    y   = a_l * left(x) + a_r * right(x);   x <- x + norm(y; w1);   x <- x + norm(ff(x); w2);   norm(y; w) = y / rms(y) * (1 + w)
    left : q, k, v = conv(W x); q, k <- rownorm(q), rownorm(k) (one mean over the whole row); rotate; scores over the last `size` positions,
           capped c * tanh(s / c); softmax whose denominator also holds e^{sink_h}; W_o
    right: q, k, v = silu(conv(W x)); q, k unit per head, q / sqrt(dim); S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q;
           rms(o) * w * silu(W_g x); W_o
    ff   : W_down (relu(W_gate x) * W_up x)
    logits = embed . norm(x; w_final)
"""
import math

import torch

D = torch.float64


def rms_unit(y, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def norm_one_plus(y, w, eps):
    return rms_unit(y, eps) * (1.0 + w.to(D))


def causal_conv(u, w):
    """u [T, C], w [C, taps]; the last column multiplies the current token, zeros before the start"""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros(T, C, dtype=D)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += w[:, j].to(D) * u[src]
    return out


def silu(z):
    return z * torch.sigmoid(z)


def frequencies(rot):
    """(f_i, amplitude) of a rotation over rot['dims'] entries; with rot['scaling'] the frequencies are divided by `factor` where the
    wavelength is long, left alone where it is short, and blended linearly between"""
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


def rotate(x, pos, rot):
    """x [heads, dim] at position pos: entries (2i, 2i+1), i < dims/2, turn by pos * f_i; the rest stay"""
    if not rot:
        return x
    f, amp = frequencies(rot)
    out = x.clone()
    for i, fi in enumerate(f):
        c, s = math.cos(pos * fi) * amp, math.sin(pos * fi) * amp
        a, b = x[:, 2 * i], x[:, 2 * i + 1]
        out[:, 2 * i] = a * c - b * s
        out[:, 2 * i + 1] = b * c + a * s
    return out


def window_attention(h, m, W, p, eps):
    """h [T, E] -> [T, E]"""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    w = lambda n: W[p + n].to(D)
    q, k, v = h @ w("q").T, h @ w("k").T, h @ w("v").T
    if m.get("conv"):
        q, k, v = causal_conv(q, W[p + "q.conv"]), causal_conv(k, W[p + "k.conv"]), causal_conv(v, W[p + "v.conv"])
    q, k = rms_unit(q, eps) * w("q.norm"), rms_unit(k, eps) * w("k.norm")
    rot, size, cap = m.get("rot"), (m.get("mask") or {}).get("size"), m.get("softcap")
    scale = m.get("scale") or dk ** -0.5
    qs = torch.stack([rotate(q[t].reshape(H, dk), t, rot) for t in range(T)])  # [T, H, dk]
    ks = torch.stack([rotate(k[t].reshape(G, dk), t, rot) for t in range(T)])  # [T, G, dk]
    vs = v.reshape(T, G, dv)
    out = torch.zeros(T, H * dv, dtype=D)
    for t in range(T):
        first = max(0, t - size + 1) if size else 0  # the token itself and the size - 1 before it
        for hh in range(H):
            g = hh // (H // G)
            s = (ks[first:t + 1, g] @ qs[t, hh]) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            e = torch.exp(s)
            den = e.sum() + (math.exp(float(W[p + "sink"][hh])) if p + "sink" in W else 0.0)  # the sink: no key, no value, counted once
            out[t, hh * dv:(hh + 1) * dv] = (e[:, None] * vs[first:t + 1, g]).sum(0) / den
    return out @ w("o").T


def scalar_delta_rule(h, m, W, p, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    w = lambda n: W[p + n].to(D)
    q = silu(causal_conv(h @ w("q").T, W[p + "q.conv"]))
    k = silu(causal_conv(h @ w("k").T, W[p + "k.conv"]))
    v = silu(causal_conv(h @ w("v").T, W[p + "v.conv"]))
    beta = torch.sigmoid(h @ w("b").T)
    decay = torch.exp(-torch.exp(w("A_log")) * torch.nn.functional.softplus(h @ w("a").T + w("dt_bias")))
    gate = silu(h @ w("g").T)
    S = [torch.zeros(dk, dv, dtype=D) for _ in range(H)]
    out = torch.zeros(T, H * dv, dtype=D)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            qt, kt = q[t, g * dk:(g + 1) * dk], k[t, g * dk:(g + 1) * dk]
            qt = qt / torch.sqrt((qt * qt).sum() + 1e-6) * dk ** -0.5
            kt = kt / torch.sqrt((kt * kt).sum() + 1e-6)
            vt = v[t, hh * dv:(hh + 1) * dv]
            S[hh] = decay[t, hh] * S[hh]
            u = beta[t, hh] * (vt - S[hh].T @ kt)
            S[hh] = S[hh] + torch.outer(kt, u)
            o = S[hh].T @ qt
            out[t, hh * dv:(hh + 1) * dv] = rms_unit(o, eps) * w("norm") * gate[t, hh * dv:(hh + 1) * dv]
    return out @ w("o").T


def feed_forward(h, W, p):
    w = lambda n: W[p + n].to(D)
    return (torch.relu(h @ w("gate").T) * (h @ w("up").T)) @ w("down").T


def forward(cfg, W, toks, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = W["embed"].to(D)[torch.tensor(list(toks))] * (cfg.get("embedding") or {}).get("scale", 1.0)
    for i, ly in enumerate(cfg["layers"]):
        p, m = "l%d." % i, ly["mixer"]
        y = m.get("left_scale", 1.0) * window_attention(x, m["left"], W, p + "mix.left.", eps) + \
            m.get("right_scale", 1.0) * scalar_delta_rule(x, m["right"], W, p + "mix.right.", eps)
        x = x + norm_one_plus(y, W[p + "norm1"], eps)
        if ly.get("mlp"):
            x = x + norm_one_plus(feed_forward(x, W, p + "mlp."), W[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, W["final.norm"], eps) @ W["embed"].to(D).T
