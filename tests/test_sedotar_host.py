"""Host-side tests of the Sedotar entry of the model registry (no GPU): config parsing and refusals through the C ABI, and sanity of the
plain float64 restatement the GPU tests compare against: it is causal, its window, sink, cap and frequency stretch do what they say, its
recurrence agrees with a closed form, and the shaped weights of the GPU tests do what they are meant to."""
import ctypes as C
import json
import math

import numpy as np
import pytest
import torch

import koifish_b200 as kf
from koifish_b200 import _lib as L
import sedotar_ref as ref
from sedotar_models import config, layer, left, right, tokens, weights


def dims(cfg):
    lib = kf.load()
    info, err = L.ModelInfo(), C.c_void_p()
    st = lib.kf_config_dims(json.dumps(cfg).encode(), C.byref(info), C.byref(err))
    msg = C.cast(err, C.c_char_p).value.decode() if err.value else ""
    if err.value:
        lib.kf_string_free(err)
    return st, info, msg


def small():
    return config([layer(), layer(left(window=0, softcap=0, rot_dims=0), ff=0)], width=24, vocab=50)


def test_config_is_parsed_by_its_registry_entry():
    st, info, msg = dims({"hf_config": small(), "gpt": {"max_seq_len": 96, "max_batch": 3, "compute_dtype": "float32"}})
    assert st == kf.KF_OK, msg
    assert (info.n_layers, info.n_embd, info.vocab, info.max_seq_len, info.max_batch) == (2, 24, 50, 96, 3)
    st, info, msg = dims(small())  # the bare config.json
    assert st == kf.KF_OK and info.n_layers == 2, msg


def test_optional_keys_may_be_null_or_absent():
    cfg = small()
    a = cfg["layers"][0]["mixer"]["left"]
    a["mask"], a["softcap"], a["rot"]["scaling"] = None, None, None
    a.pop("kv_heads"), a.pop("scale")
    cfg["layers"][0]["mixer"].pop("left_scale")
    cfg["layers"][1]["mlp"] = None
    st, _, msg = dims({"hf_config": cfg})
    assert st == kf.KF_OK, msg


@pytest.mark.parametrize("edit, words", [
    (lambda c: c["layers"][0].update(type="lstm"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads must divide heads"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=3), "kv_heads must divide heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims even"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=14), "rot.dims even"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(factor=0.0), "must be positive"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].pop("size"), "mask.size is missing"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "is not built"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c.pop("layers"), "layers"),
])
def test_bad_configs_are_refused_with_a_message(edit, words):
    cfg = small()
    edit(cfg)
    st, _, msg = dims({"hf_config": cfg})
    assert st != kf.KF_OK and words in msg, msg


def test_float32_is_a_mode_of_this_architecture():
    st, _, msg = dims({"hf_config": small(), "gpt": {"compute_dtype": "float32"}})
    assert st == kf.KF_OK, msg


# ------------------------------------------------------------------------------------------------------------ the oracle itself
def test_oracle_is_causal():
    cfg = config([layer(), layer(left(window=5), ff=0)])
    W = weights(cfg, seed=1)
    toks = tokens(40, cfg["vocab"], 2)
    full = ref.forward(cfg, W, toks)
    part = ref.forward(cfg, W, toks[:23])
    assert torch.allclose(full[:23], part, atol=1e-12)


def test_window_of_one_sees_only_the_token_itself():
    """with a window of 1 and no convolution reach, no rotation matters and attention of a token is v * e^s / (e^s + e^sink)"""
    m = left(heads=1, kv_heads=1, dim=4, vdim=3, conv=1, window=1, softcap=0, rot_dims=4)
    cfg = config([layer(m, ff=0, left_scale=1.0, right_scale=0.0)], width=8, vocab=10)
    W = weights(cfg, seed=2)
    h = torch.randn(6, 8, dtype=torch.float64)
    got = ref.window_attention(h, m, W, "l0.mix.left.", 1e-5)
    p = "l0.mix.left."
    w = lambda n: W[p + n].double()
    q = ref.rms_unit((h @ w("q").T) * w("q.conv")[:, 0], 1e-5) * w("q.norm")
    k = ref.rms_unit((h @ w("k").T) * w("k.conv")[:, 0], 1e-5) * w("k.norm")
    v = (h @ w("v").T) * w("v.conv")[:, 0]
    s = (q * k).sum(-1) * m["scale"] * (0.1 * math.log(4.0) + 1.0) ** 2  # a rotation by the same angle keeps q . k, the amplitude squares
    wgt = torch.exp(s) / (torch.exp(s) + math.exp(float(W[p + "sink"][0])))
    assert torch.allclose(got, (wgt[:, None] * v) @ w("o").T, atol=1e-10)


def test_stretched_frequencies():
    f, amp = ref.frequencies({"dims": 8, "base": 100.0})
    assert amp == 1.0 and np.allclose(f, [1.0, 100 ** -0.25, 0.1, 100 ** -0.75])
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    g, amp = ref.frequencies({"dims": 8, "base": 100.0, "scaling": sc})
    assert abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    lo = math.floor(8 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(100.0)))
    hi = math.ceil(8 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(100.0)))
    assert (lo, hi) == (0, 3)
    for i in range(4):
        r = min(1.0, max(0.0, (i - lo) / (hi - lo)))
        assert abs(g[i] - f[i] * (r / 4.0 + 1.0 - r)) < 1e-15
    assert g[0] == f[0] and g[3] == f[3] / 4.0


def test_delta_rule_with_orthogonal_keys_stores_and_recalls():
    """beta = 1, no decay, unit orthogonal keys: after writing (k_1, v_1), (k_2, v_2) the state reads v_j back with q = k_j"""
    S = torch.zeros(3, 2, dtype=torch.float64)
    ks = [torch.tensor([1.0, 0, 0], dtype=torch.float64), torch.tensor([0, 1.0, 0], dtype=torch.float64)]
    vs = [torch.tensor([2.0, -1.0], dtype=torch.float64), torch.tensor([0.5, 4.0], dtype=torch.float64)]
    for k, v in zip(ks, vs):
        S = 1.0 * S
        u = 1.0 * (v - S.T @ k)
        S = S + torch.outer(k, u)
    assert torch.allclose(S.T @ ks[0], vs[0]) and torch.allclose(S.T @ ks[1], vs[1])
    # writing k_1 again with another value REPLACES the old one (that is the delta in the rule)
    v3 = torch.tensor([7.0, 7.0], dtype=torch.float64)
    S = S + torch.outer(ks[0], v3 - S.T @ ks[0])
    assert torch.allclose(S.T @ ks[0], v3) and torch.allclose(S.T @ ks[1], vs[1])


def test_shaped_weights_do_what_the_gpu_tests_rely_on():
    cfg = config([layer(left(heads=4, kv_heads=2, dim=16, vdim=12, window=23, softcap=6.0, rot_dims=12, base=100.0), ff=0, left_scale=1.0, right_scale=0.3)])
    W = weights(cfg, seed=9, q_gain=12.0, sink=5.0)
    toks = tokens(120, cfg["vocab"], 7)
    want = ref.forward(cfg, W, toks)

    def moved(c, w=W):
        d = ref.forward(c, w, toks) - want
        return float(d.std() / want.std())

    def edited(fn):
        c = json.loads(json.dumps(cfg))
        fn(c["layers"][0]["mixer"]["left"])
        return c

    assert moved(edited(lambda a: a["mask"].update(size=24))) > 1e-3
    assert moved(edited(lambda a: a["mask"].update(size=22))) > 1e-3
    assert moved(edited(lambda a: a.pop("softcap"))) > 1e-3
    assert moved(cfg, {k: v for k, v in W.items() if not k.endswith(".sink")}) > 1e-3
