"""Host-side pieces of the Girolorn design: the config reader (every size and constant from config.json, layers that run
with another layer's tensors, refusals) and the oracle's own mechanisms against closed forms."""
import ctypes as C
import json
import math

import torch

from oracle import girolorn as og


def spec_of(kge, path):
    L = kge.lib()
    h = L.kge_model_open(str(path).encode())
    assert h, L.kge_last_error()
    buf = C.create_string_buffer(1 << 16)
    assert L.kge_model_spec_json(h, buf, 1 << 16) > 0
    L.kge_model_close(h)
    return json.loads(buf.value)


def test_config_reader_takes_every_size_and_constant(kge, tmp_path):
    cfg = og.make_config(vocab=77, width=40, n_layers=4, heads=6, kv_heads=3, dim=10, rot_dims=6, base=777.0, scaling=(3.0, 50, 8.0, 0.5),
                         scale=0.41, softcap=5.5, experts=7, top=3, expert_ff=9, expert_limit=2.25, shared_ff=13, shared_limit=0.5,
                         mlps=(True, False, True, True), weights_of={3: 0}, eps=3e-4, logit_softcap=4.5)
    og.save_model_dir(str(tmp_path), cfg, og.make_weights(cfg))
    spec = spec_of(kge, tmp_path)
    assert (spec["model_type"], spec["vocab"], spec["d"], spec["L"]) == ("girolorn", 77, 40, 4) and spec["has_weights"]
    assert abs(spec["eps"] - 3e-4) < 1e-9 and abs(spec["logit_softcap"] - 4.5) < 1e-6
    a, b, c, d = spec["layers"]
    assert (a["mixer"], a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["rot_dims"], a["mlp"], a["experts"], a["top"], a["expert_ff"], a["shared_ff"]) == \
        (2, 6, 3, 10, 10, 6, 2, 7, 3, 9, 13)
    assert abs(a["scale"] - 0.41) < 1e-6 and abs(a["softcap"] - 5.5) < 1e-6 and a["rot_base"] == 777.0
    assert (a["yarn_factor"], a["yarn_original"], a["yarn_fast"], a["yarn_slow"]) == (3.0, 50.0, 8.0, 0.5)
    assert abs(a["expert_limit"] - 2.25) < 1e-6 and abs(a["shared_limit"] - 0.5) < 1e-6 and (a["route"], a["glu"]) == (1, 1)
    assert b["mlp"] == 0 and (a["weights_of"], d["weights_of"]) == (-1, 0)


def test_config_reader_refusals(kge, tmp_path):
    L = kge.lib()

    def refused(change, text):
        cfg = og.make_config(n_layers=2)
        change(cfg)
        with open(tmp_path / "config.json", "w") as fh:
            json.dump(cfg, fh)
        assert not L.kge_model_open(str(tmp_path).encode())
        assert text in L.kge_last_error(), L.kge_last_error()
    refused(lambda c: c["layers"][0].update(type="rglru"), b"unknown layer type")
    refused(lambda c: c["layers"][1].update(weights_of=1), b"weights_of")
    refused(lambda c: c["layers"][1].update(weights_of=5), b"weights_of")
    refused(lambda c: c["layers"][0]["mixer"].update(vdim=16), b"vdim")
    refused(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), b"attention sizes")
    refused(lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), b"limit")


def test_oracle_rotary_is_a_rotation_and_keeps_the_rest():
    rot = {"base": 100.0, "dims": 4}
    x = torch.randn(5, 2, 6, dtype=og.DT)
    y = og.rotary(x, torch.arange(5), rot)
    assert torch.equal(y[..., 4:], x[..., 4:]) and torch.equal(y[0], x[0])
    assert torch.allclose(y[..., :4].pow(2).sum(-1), x[..., :4].pow(2).sum(-1))
    # position 3, pair 1 turns by 3 * 100^(-2/4) = 0.3
    a, b = x[3, 0, 2], x[3, 0, 3]
    assert torch.allclose(y[3, 0, 2], a * math.cos(0.3) - b * math.sin(0.3)) and torch.allclose(y[3, 0, 3], b * math.cos(0.3) + a * math.sin(0.3))


def test_oracle_scaled_frequencies():
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 128, "fast": 16.0, "slow": 1.0}}
    f, c = og.rotary_frequencies(rot)
    plain = 10000.0 ** (-torch.arange(8, dtype=og.DT) / 8)
    assert abs(c - (1 + 0.1 * math.log(4.0))) < 1e-12
    assert torch.allclose(f[0], plain[0]) and torch.allclose(f[-1], plain[-1] / 4.0)     # fast pairs untouched, slow pairs divided
    assert all(plain[i] / 4.0 - 1e-15 <= f[i] <= plain[i] + 1e-15 for i in range(8))


def test_oracle_sink_and_cap():
    """One token: the only key has probability e^s / (e^s + e^sink), s capped."""
    cfg = og.make_config(n_layers=1, heads=1, kv_heads=1, dim=4, rot_dims=0, scaling=None, scale=50.0, softcap=2.0, mlps=(False,))
    W = og.make_weights(cfg, seed=1)
    P = og.sub(W, "l0.mix.")
    h = torch.randn(1, cfg["width"], dtype=og.DT)
    k0 = h @ P["k"].T
    q = og.rms_all(h @ P["q"].T, P["q.norm"], 1e-5)
    k = og.rms_all(k0, P["k.norm"], 1e-5)
    s = 2.0 * torch.tanh(50.0 * (q @ k.T) / 2.0)
    p = torch.exp(s) / (torch.exp(s) + torch.exp(P["sink"][0]))
    want = (p * k0) @ P["o"].T
    assert torch.allclose(og.sink_attention(h, P, cfg["layers"][0]["mixer"], 1e-5), want)


def test_oracle_router_weights():
    h = torch.randn(3, 8, dtype=og.DT)
    R, b = torch.randn(5, 8, dtype=og.DT), torch.randn(5, dtype=og.DT)
    for order, w in og.route(h, R, b, 1):
        assert len(order) == 1 and float(w[0]) == 1.0
    z = h @ R.T + b
    for t, (order, w) in enumerate(og.route(h, R, b, 5)):
        assert torch.allclose(w, torch.softmax(z[t], 0)[order]) and order[0] == int(torch.argmax(z[t]))
