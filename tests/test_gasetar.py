"""Gasetar without a GPU: the configuration reader, the model's description, the rotary tables with slowed-down long
wavelengths, the head's scale before the cap, and the plain implementation's own invariants."""
import copy
import math

import numpy as np
import pytest

import plain_gasetar as plain
import tiny_gasetar
from rust_deeplearning_b200.config.base import ConfigError, architecture_for
from rust_deeplearning_b200.parts.position import Rotary, rotary_frequencies


def test_configuration_becomes_parts():
    cfg, _ = tiny_gasetar.config("GA")
    arch = architecture_for(cfg)
    assert arch.name == "Gasetar"
    spec = arch.build_spec(arch.parse_config(cfg))
    assert [layer.block for layer in spec.layers] == ["parallel"] * 4
    assert [layer.mixer.kind for layer in spec.layers] == ["latent_attention", "attention", "attention", "latent_attention"]
    assert all(layer.params["branch_scale"] == 0.6 and set(layer.norms) == {"pre"} for layer in spec.layers)
    assert spec.layers[2].feed_forward is None and spec.layers[1].feed_forward.kind == "gated_mlp"
    a = spec.layers[1].mixer.params
    assert (a["n_heads"], a["n_kv_heads"], a["head_dim"], a["value_dim"], a["window"], a["softcap"]) == (6, 2, 12, 20, 5, 8.0)
    assert a["proj_norm_eps"] == 1e-5 and a["position"].params["scaling"]["kind"] == "llama3" and a["position"].params["rotary_dim"] == 6
    assert spec.layers[2].mixer.params["position"].params["scaling"] is None
    la = spec.layers[0].mixer.params
    assert la["window"] is None and la["gate_per_value"] and la["position"].params["pairing"] == "half"
    f = spec.layers[0].feed_forward
    assert f.params["scoring"] == "softmax_chosen" and f.params["form"] == "silu" and f.params["top"] == 2
    names = spec.tensor_specs()
    assert names["l1.mix.q.norm"].shape == (72,) and names["l1.mix.k.norm"].shape == (24,) and names["l1.mix.o"].shape == (72, 120)
    assert names["l0.mix.sink"].shape == (3,) and names["l0.mix.g"].shape == (60, 72) and names["l0.mix.dkv"].shape == (34, 72)
    assert names["l0.mlp.router.b"].shape == (5,) and names["l0.mlp.shared.down"].shape == (72, 12) and "l3.mlp.shared.up" not in names
    assert "l2.mlp.gate" not in names and names["l1.mlp.gate"].shape == (44, 72)
    assert spec.embedding.params["scale"] == 3.0 and spec.head.params["pre_scale"] == 0.8 and spec.head.params["softcap"] == 12.0
    assert spec.head.tensors["weight"].name == "embed"


def test_optional_keys_have_their_meaning():
    """No mask: all keys; no soft-cap: none; kv_heads missing: one key head a query head; no rot: no rotation."""
    cfg, _ = tiny_gasetar.config("GB")
    m = cfg["layers"][2]["mixer"]
    del m["kv_heads"], m["rot"], m["softcap"]
    del cfg["logit_scale"], cfg["residual_mult"], cfg["embedding"]
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    a = spec.layers[2].mixer.params
    assert a["n_kv_heads"] == 2 and a["window"] is None and a["softcap"] is None and a["position"] is None
    assert spec.head.params["pre_scale"] == 1.0 and spec.head.params["softcap"] is None and spec.layers[0].params["branch_scale"] == 1.0


def test_configuration_errors_are_listed_together():
    cfg, _ = tiny_gasetar.config("GA")
    bad = copy.deepcopy(cfg)
    del bad["width"]
    bad["layers"][1]["mixer"]["rot"]["dims"] = 7
    bad["layers"][1]["mixer"]["kv_heads"] = 4
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    bad["layers"][3]["mixer"]["rot"]["dims"] = 12
    bad["layers"][2]["type"] = "convolution"
    with pytest.raises(ConfigError) as e:
        architecture_for(bad).parse_config(bad)
    text = str(e.value)
    for word in ("width", "dims (7)", "kv_heads", "top (9)", "rot_dim", "convolution"):
        assert word in text, word
    bad = copy.deepcopy(cfg)
    bad["layers"][1]["mlp"] = {"kind": "sparse"}
    with pytest.raises(ConfigError, match="sparse"):
        architecture_for(bad).parse_config(bad)


@pytest.mark.parametrize("scaling", [None, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64},
                                     {"factor": 3.0, "low": 2.0, "high": 16.0, "original": 500}])
def test_rotary_tables_against_the_plain_rotation(scaling):
    rot = {"base": 3000.0, "dims": 12, **({"scaling": scaling} if scaling else {})}
    f = plain.rotary_frequencies(rot)
    inv, mag = rotary_frequencies(rot["base"], rot["dims"], dict(scaling, kind="llama3") if scaling else None)
    assert np.allclose(inv.numpy(), f, rtol=1e-14) and mag == 1.0
    if scaling:      # the three ranges are all there: kept, slowed down, blended
        plainf = np.array([rot["base"] ** (-2.0 * i / 12) for i in range(6)])
        ratio = np.array(f) / plainf
        assert np.isclose(ratio[0], 1.0) and np.isclose(ratio[-1], 1.0 / scaling["factor"])
        assert ((ratio > 1.0 / scaling["factor"] + 1e-9) & (ratio < 1.0 - 1e-9)).any()
    part = Rotary(rot["base"], 16, 12, 50, "cpu", pairing="half", scaling=dict(scaling, kind="llama3") if scaling else None)
    v = np.random.default_rng(0).normal(size=16)
    for p in (0, 1, 17, 49):
        want = plain.rotate(v, p, rot)
        c, s = part.cos[p].double().numpy(), part.sin[p].double().numpy()
        got = v.copy()
        got[0:6], got[6:12] = v[0:6] * c - v[6:12] * s, v[6:12] * c + v[0:6] * s
        assert np.allclose(got, want, atol=1e-6)
        assert np.array_equal(want[12:], v[12:])


def test_head_scales_before_the_cap():
    """cap tanh(p z / cap) is run as a cap of cap / p followed by a factor p."""
    from rust_deeplearning_b200.parts.model import LinearHead
    head = LinearHead(None, 30.0, 1.0, 0.4)
    z = np.linspace(-300, 300, 41)
    assert np.allclose(head.softcap * np.tanh(z / head.softcap) * head.scale, 30.0 * np.tanh(0.4 * z / 30.0))
    plainhead = LinearHead(None, None, 1.0, 0.4)
    assert plainhead.softcap is None and plainhead.scale == 0.4


def test_plain_model_invariants(tmp_path):
    """What the plain implementation must satisfy by construction: a token's logits do not depend on later tokens; a key
    just outside an attention layer's window does not count, one just inside does; a sink takes weight from the keys;
    the absorbed form of latent attention equals the expanded one; the chosen experts' weights sum to one."""
    from rust_deeplearning_b200 import write_random_model
    cfg, seed = tiny_gasetar.config("GA")
    write_random_model(str(tmp_path), cfg, seed, "bfloat16")
    pcfg, w = plain.load_folder(str(tmp_path))
    ids = [int(v) for v in np.random.default_rng(1).integers(0, cfg["vocab"], size=24)]
    full = plain.forward(pcfg, w, ids)
    assert np.allclose(plain.forward(pcfg, w, ids[:11]), full[:11], atol=1e-12)
    assert np.abs(full).max() <= pcfg["logit_softcap"]
    # window: layer 1 sees the token itself and the 4 before it
    m = pcfg["layers"][1]["mixer"]
    h = np.random.default_rng(2).normal(size=(9, cfg["width"]))
    base = plain.attention(h, w, "l1.mix.", m, 1e-5)
    moved = h.copy()
    moved[3] += 1.0                               # key 3 is outside the window of query 8 (keys 4..8), inside that of query 7
    out = plain.attention(moved, w, "l1.mix.", m, 1e-5)
    assert np.allclose(out[8], base[8], atol=1e-12) and np.abs(out[7] - base[7]).max() > 1e-6
    # sinks and the absorbed form
    m = pcfg["layers"][0]["mixer"]
    want = plain.latent_attention(h, w, "l0.mix.", m, 1e-5)
    H, d, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w["l0.mix.q"].T).reshape(9, H, d + rd)
    dk = h @ w["l0.mix.dkv"].T
    c = plain.rms_norm(dk[:, :r], w["l0.mix.dkv.norm"], 1e-5)
    kr = np.stack([plain.rotate(dk[t, r:], t, m["rot"]) for t in range(9)])
    uk, uv = w["l0.mix.uk"].reshape(H, d, r), w["l0.mix.uv"].reshape(H, vd, r)
    gate = (1 / (1 + np.exp(-(h @ w["l0.mix.g"].T)))).reshape(9, H, vd)
    out = np.zeros((9, H, vd))
    for i in range(9):
        for a in range(H):
            qa = np.concatenate([uk[a].T @ q[i, a, :d], plain.rotate(q[i, a, d:], i, m["rot"])])
            s = np.array([qa @ np.concatenate([c[j], kr[j]]) * m["scale"] for j in range(i + 1)])
            e = np.exp(s)
            p = e / (e.sum() + math.exp(w["l0.mix.sink"][a]))
            out[i, a] = uv[a] @ (p[:, None] * c[:i + 1]).sum(axis=0) * gate[i, a]
    assert np.allclose(out.reshape(9, -1) @ w["l0.mix.o"].T, want, atol=1e-10)
    no_sink = dict(w)
    no_sink["l0.mix.sink"] = np.full(H, -1e9)
    assert np.abs(plain.latent_attention(h, no_sink, "l0.mix.", m, 1e-5) - want).max() > 1e-4
    chosen, weight, margin = plain.router(h, w, "l0.mlp.", pcfg["layers"][0]["mlp"])
    assert chosen.shape == (9, 2) and np.allclose(weight.sum(axis=-1), 1.0) and (weight[:, 0] >= weight[:, 1]).all() and (margin >= 0).all()
