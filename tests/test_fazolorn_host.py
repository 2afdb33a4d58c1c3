"""Host-side tests of the Fazolorn entry of the model registry (no GPU): config parsing and refusals through the C ABI, and sanity of the
plain float64 restatement the GPU tests compare against: it is causal, its blocks, recurrence, routing rule and repeated layers do what
they say, and the shaped weights of the GPU tests do what they are meant to."""
import ctypes as C
import json
import math

import numpy as np
import pytest
import torch

import koifish_b200 as kf
from koifish_b200 import _lib as L
import fazolorn_ref as ref
from fazolorn_models import attn, config, dense, gru, latent, layer, moe, tokens, weights


def dims(cfg):
    lib = kf.load()
    info, err = L.ModelInfo(), C.c_void_p()
    st = lib.kf_config_dims(json.dumps(cfg).encode(), C.byref(info), C.byref(err))
    msg = C.cast(err, C.c_char_p).value.decode() if err.value else ""
    if err.value:
        lib.kf_string_free(err)
    return st, info, msg


def small():
    return config([layer(attn(), dense()), layer(latent(), moe()), layer(gru(), None)], width=24, vocab=50, loop=(0, 2, 3))


def test_config_is_parsed_by_its_registry_entry():
    st, info, msg = dims({"hf_config": small(), "gpt": {"max_seq_len": 96, "max_batch": 3, "compute_dtype": "float32"}})
    assert st == kf.KF_OK, msg
    assert (info.n_layers, info.n_embd, info.vocab, info.max_seq_len, info.max_batch) == (3, 24, 50, 96, 3)
    st, info, msg = dims(small())  # the bare config.json
    assert st == kf.KF_OK and info.n_layers == 3, msg


def test_optional_keys_may_be_null_or_absent():
    cfg = small()
    a = cfg["layers"][0]["mixer"]
    a["mask"], a["rot"] = None, None
    a.pop("kv_heads"), a.pop("scale"), a.pop("vdim")
    cfg["layers"][1]["mixer"]["rot"]["scaling"] = None
    cfg["layers"][1]["mlp"]["router"].pop("groups")
    cfg["layers"][1]["mlp"]["router"]["scale"] = None
    cfg["loop"] = None
    cfg.pop("logit_scale")
    st, _, msg = dims({"hf_config": cfg})
    assert st == kf.KF_OK, msg


def test_query_latent_size_from_the_tensor_shapes():
    cfg = small()
    cfg["layers"][1]["mixer"].pop("q_rank")
    st, _, msg = dims({"hf_config": cfg})
    assert st != kf.KF_OK and "q_rank" in msg
    st, _, msg = dims({"hf_config": dict(cfg, tensor_shapes={"l1.mix.dq": [14, 24]})})
    assert st == kf.KF_OK, msg


@pytest.mark.parametrize("edit, words", [
    (lambda c: c["layers"][0].update(type="lstm"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads must divide heads"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=5), "vdim must equal dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims must be even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "dims must be even"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "mask.size is missing"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0), "must be positive"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=700), "kv_rank + rot_dim <= 640"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "is not built"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit is missing"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top <= keep"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "must divide experts"),
    (lambda c: c["layers"][2]["mixer"].pop("width"), "width is missing"),
    (lambda c: c["loop"].update(stop=4), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refusals(edit, words):
    cfg = small()
    edit(cfg)
    st, _, msg = dims({"hf_config": cfg})
    assert st != kf.KF_OK and words in msg, msg


def test_no_device_no_model():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(kf.KoifishError):
        kf.Context(0)


# ------------------------------------------------------------------------------------------------------------ the oracle itself
def test_oracle_is_causal():
    cfg = small()
    W = weights(cfg, seed=1)
    a = tokens(30, cfg["vocab"], 2)
    b = list(a)
    b[20] = (a[20] + 1) % cfg["vocab"]
    la, lb = ref.forward(cfg, W, a), ref.forward(cfg, W, b)
    assert torch.equal(la[:20], lb[:20]) and not torch.allclose(la[20:], lb[20:])
    assert torch.allclose(ref.forward(cfg, W, a[:11]), la[:11], atol=1e-12)


def test_blocks_are_counted_from_position_zero():
    """one head, queries and keys made constant so that every weight is sigmoid(pb): the output is the weight times the SUM of the values of
    the block so far, which restarts at every multiple of the block size"""
    m = attn(heads=1, kv_heads=1, dim=4, block=5, rot_dims=0)[1]
    E, T = 6, 17
    g = torch.Generator().manual_seed(0)
    W = {"q": torch.zeros(4, E), "q.b": torch.zeros(4), "k": torch.randn(4, E, generator=g), "k.b": torch.randn(4, generator=g), "pb": torch.tensor([0.7]),
         "o": torch.eye(E, 4)}
    h = torch.randn(T, E, generator=g, dtype=torch.float64)
    out = ref.block_attention(h, m, W, "")
    k = h @ W["k"].double().T + W["k.b"].double()
    for t in range(T):
        want = torch.sigmoid(torch.tensor(0.7, dtype=torch.float64)) * k[(t // 5) * 5:t + 1].sum(0)
        assert torch.allclose(out[t, :4], want, atol=1e-12)


def test_recurrence_against_its_closed_form():
    """constant gates: S_t = (1 - z)^t-weighted sum of the candidates; the candidate is u + 1/2 above zero and sigmoid(u) below"""
    n, E, T = 3, 3, 9
    W = {"z": torch.zeros(n, E), "z.b": torch.full((n,), -1.0), "x": torch.eye(n, E), "x.b": torch.zeros(n), "g": torch.zeros(n, E), "o": torch.eye(E, n)}
    h = torch.linspace(-2, 2, T * E, dtype=torch.float64).view(T, E)
    z = 1 / (1 + math.e)
    S = torch.zeros(n, dtype=torch.float64)
    for t in range(T):
        cand = torch.where(h[t] >= 0, h[t] + 0.5, torch.sigmoid(h[t]))
        S = (1 - z) * S + z * cand
    _, last = ref.mingru(h, {"width": n}, W, "")
    assert torch.allclose(last, S, atol=1e-12)
    out, _ = ref.mingru(h, {"width": n}, W, "")
    assert torch.all(out == 0)  # silu(0) = 0 gates everything away


def test_routing_rule_on_a_hand_example():
    f = moe(experts=6, top=2, groups=(3, 1), scale=2.0)
    # scores (after the sigmoid) rise with the logits; the correction lifts the last group above the first although its scores are lower
    W = {"router": torch.tensor([[3.0], [2.5], [0.0], [0.1], [1.0], [0.5]]), "correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 0.6, 0.6])}
    (idx, wgt), = ref.route(torch.ones(1, 1, dtype=torch.float64), f, W, "")
    assert idx == [4, 5]
    assert abs(wgt[0].item() - 2.0 / (1 + math.exp(-1.0))) < 1e-12 and abs(wgt[1].item() - 2.0 / (1 + math.exp(-0.5))) < 1e-12  # weights without the correction
    f["router"]["groups"]["keep"] = 3
    (idx, _), = ref.route(torch.ones(1, 1, dtype=torch.float64), f, W, "")
    assert idx == [4, 5]  # 0.731 + 0.6 and 0.622 + 0.6 still lead
    W["correction"] = torch.zeros(6)
    (idx, _), = ref.route(torch.ones(1, 1, dtype=torch.float64), f, W, "")
    assert idx == [0, 1]


def test_order_of_the_layer_runs():
    cfg = config([layer(gru(), None)] * 5, loop=(1, 3, 3))
    assert ref.layer_runs(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None), (4, None)]
    assert ref.layer_runs(config([layer(gru(), None)] * 2)) == [(0, None), (1, None)]


def test_stretched_frequencies_by_hand():
    f, amp = ref.frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    at = lambda turns: 8 * math.log(64 / (2 * math.pi * turns)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(at(8.0)), 0), min(math.ceil(at(1.0)), 7)
    assert (lo, hi) == (0, 3)
    plain = [100.0 ** (-2 * i / 8) for i in range(4)]
    for i in range(4):
        r = min(1.0, max(0.0, (i - lo) / (hi - lo)))
        assert abs(f[i] - (plain[i] / 4 * r + plain[i] * (1 - r))) < 1e-15
    assert abs(amp - (0.1 * math.log(4.0) + 1)) < 1e-15


def test_dense_clamps_bite_with_the_test_weights():
    cfg = config([layer(gru(), dense(56, 0.4))], width=32)
    W = weights(cfg, seed=3)
    h = torch.randn(50, 32, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    g = h @ W["l0.mlp.gate"].double().T
    assert (g > 0.4).double().mean() > 0.1 and (g.abs() < 0.4).double().mean() > 0.1
