"""Revepel without a GPU: the configuration reader, the model's description as parts, what the cache is asked for, and the
plain implementation's own invariants (causality, the edge of a window, what a shifted row reads, the recurrences in
another form)."""
import copy

import numpy as np
import pytest

import plain_revepel as plain
import tiny_revepel
from rust_deeplearning_b200.cache.cache import Cache, KVRequirement, RunNeeds, StateRequirement
from rust_deeplearning_b200.config.base import ConfigError, architecture_for
from rust_deeplearning_b200.parts.spec import shape_fits


def _spec(name):
    cfg, _ = tiny_revepel.config(name)
    arch = architecture_for(cfg)
    assert arch.name == "Revepel"
    return cfg, arch.build_spec(arch.parse_config(cfg))


def test_configuration_becomes_parts():
    cfg, spec = _spec("RA")
    assert [l.block for l in spec.layers] == ["parallel"] * 4
    assert all(l.params["token_shift"] and l.params["gated_residual"] for l in spec.layers)
    attn, delta, ssm, reader = (l.mixer for l in spec.layers)
    assert attn.kind == "attention" and attn.params["window"] == 8 and attn.params["cache_window"] == 12      # the reader looks further back
    assert reader.params["window"] == 12 and "k" not in reader.tensors and "v" not in reader.tensors and "score_bias" in reader.tensors
    assert [s.reads_cache_of for s in spec.schedule] == [None, None, None, 0]
    rot = attn.params["position"].params
    assert rot["rotary_dim"] == 8 and rot["pairing"] == "half" and rot["scaling"]["kind"] == "yarn" and rot["scaling"]["factor"] == 4.0
    assert delta.kind == "delta_rule" and delta.params["n_key_heads"] == 2 and delta.params["taps"] == 4 and delta.params["q_scale"] == 0.25
    assert ssm.kind == "state_space" and ssm.params["n_groups"] == 2 and ssm.params["norm_groups"] == 2
    ff = spec.layers[0].feed_forward
    assert ff.kind == "routed_experts" and ff.params["scoring"] == "sigmoid" and ff.params["weights_on_input"] and ff.params["form"] == "relu2"
    assert ff.params["top"] == 2 and "shared_up" in ff.tensors and "gate0" not in ff.tensors
    assert spec.layers[2].feed_forward is None and "gate_ff" not in spec.layers[2].tensors
    assert "shared_up" not in spec.layers[3].feed_forward.tensors
    names = spec.tensor_specs()
    assert names["l2.mix.in"].shape == (2 * 64 + 2 * 16 + 4, 64) and names["l2.mix.conv"].shape == (64 + 32, 4)
    assert names["l1.mix.a1"].shape == (8, 64) and names["l1.mix.g2"].shape == (96, 16) and names["l1.mix.norm"].shape == (24,)
    assert names["l1.mix.dt_bias"].shape == (64,) and names["l1.mix.b"].shape == (4, 64)
    assert names["l0.shift"].shape == (64,) and names["l0.rg2.b"].shape == (64,) and "l2.rg2" not in names
    assert names["head"].shape == (210, 64) and spec.head.params["scale"] == 0.5 and spec.embedding.params["scale"] == 6.0


def test_ranks_that_only_the_file_gives():
    cfg, _ = tiny_revepel.config("RA")
    del cfg["layers"][1]["mixer"]["decay_rank"], cfg["layers"][1]["mixer"]["gate_rank"]
    arch = architecture_for(cfg)
    names = arch.build_spec(arch.parse_config(cfg)).tensor_specs()
    assert names["l1.mix.a1"].shape == (None, 64) and names["l1.mix.a2"].shape == (64, None)
    assert shape_fits((24, 64), names["l1.mix.a1"].shape) and not shape_fits((24, 65), names["l1.mix.a1"].shape)
    from rust_deeplearning_b200.weights.loader import random_tensor
    with pytest.raises(ValueError, match="only a weight file gives"):
        random_tensor(names["l1.mix.a1"], 0, None)


def test_configuration_errors_are_listed_together():
    cfg, _ = tiny_revepel.config("RB")
    bad = copy.deepcopy(cfg)
    del bad["logit_scale"]
    bad["layers"][0]["mixer"]["groups"] = 2
    bad["layers"][1]["mixer"]["rot"]["dims"] = 14
    bad["layers"][2]["mixer"]["kv_heads"] = 2
    bad["layers"][3]["mlp"]["router"]["top"] = 3
    bad["layers"][4]["mixer"]["norm_groups"] = 5
    with pytest.raises(ConfigError) as e:
        architecture_for(bad).parse_config(bad)
    text = str(e.value)
    for piece in ("logit_scale", "3 heads cannot share 2 groups", "dims (14)", "3 heads cannot share 2 key heads", "3 of 2 experts", "5 norm groups"):
        assert piece in text, piece
    for change, message in ((lambda c: c["layers"][0].update(type="convolution"), "convolution"),
                            (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "attention layer with keys"),
                            (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
                            (lambda c: c["layers"][3]["mixer"].update(dim=16), "differ"),
                            (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "dense")):
        bad = copy.deepcopy(cfg)
        change(bad)
        with pytest.raises(ConfigError, match=message):
            architecture_for(bad).parse_config(bad)


def test_cache_needs_from_the_descriptions():
    """What the cache is asked for, from the descriptions alone (no device): every layer keeps the row before a step's
    first row; a recurrent mixer its state and, with more than one tap, the convolution's last inputs; attention layers
    that own keys a page group (a ring as wide as the widest reader's window), readers nothing."""
    cfg, spec = _spec("RB")
    W = cfg["width"]
    needs = []
    for layer, entry in zip(spec.layers, spec.schedule):
        p = layer.mixer.params
        own = (StateRequirement((W,)),)
        if layer.mixer.kind == "state_space":
            st = (StateRequirement((p["n_heads"], p["state_dim"], p["vdim"])),
                  StateRequirement((p["taps"] - 1, p["n_heads"] * p["vdim"] + 2 * p["n_groups"] * p["state_dim"])))
            needs.append(RunNeeds(None, own + st))
        elif layer.mixer.kind == "delta_rule":
            assert p["taps"] == 1                       # one tap: nothing of the convolution is kept
            needs.append(RunNeeds(None, own + (StateRequirement((p["n_heads"], p["dim"], p["vdim"])),)))
        else:
            window = None if p["cache_window"] in (None, "all") else p["cache_window"]
            needs.append(RunNeeds(KVRequirement(p["n_kv_heads"], max(p["head_dim"], p["value_dim"]), window), own, entry.reads_cache_of))
    cache = Cache(needs, max_tokens=64, max_seqs=2, page_size=16, device="cpu", allocate=False)
    assert len(cache.kv_groups) == 1 and cache.kv_groups[0].requirement.window is None      # layer 1 has no window: every key is kept
    shapes = sorted(g.requirement.shape for g in cache.state_groups)
    assert (W,) in shapes and (3, 12, 20) in shapes and (1, 60 + 72) in shapes and (3, 12, 24) in shapes and (2, 72 + 10) in shapes
    assert [g for g in cache.state_groups if g.requirement.shape == (W,)][0].runs == [0, 1, 2, 3, 4]


@pytest.fixture(scope="module")
def small():
    """A model of the plain implementation with weights drawn here (no file, no device)."""
    cfg, _ = tiny_revepel.config("RA")
    arch = architecture_for(cfg)
    rng = np.random.default_rng(5)
    w = {}
    for name, t in arch.build_spec(arch.parse_config(cfg)).tensor_specs().items():
        w[name] = rng.normal(t.init_mean, t.init_std, size=t.shape)
    return cfg, w


def test_plain_model_is_causal_and_its_first_token_reads_zeros(small):
    cfg, w = small
    ids = [int(v) for v in np.random.default_rng(1).integers(0, cfg["vocab"], size=40)]
    whole = plain.forward(cfg, w, ids)
    assert np.allclose(plain.forward(cfg, w, ids[:17]), whole[:17], atol=1e-12)
    other = ids[:25] + [(ids[25] + 1) % cfg["vocab"]] + ids[26:]
    changed = plain.forward(cfg, w, other)
    assert np.allclose(changed[:25], whole[:25], atol=1e-12) and np.abs(changed[25:] - whole[25:]).max() > 1e-6
    n = np.random.default_rng(2).normal(size=(5, 8))
    s = np.linspace(0.0, 1.0, 8)
    m = plain.shifted(n, s)
    assert np.allclose(m[0], n[0] * (1.0 - s)) and np.allclose(m[3][:, None][0], n[3][0]) and np.allclose(m[3][-1], n[2][-1])


def test_plain_window_edge_and_unnormalised_weights():
    """One key's score stands out: it counts while 0 <= i - j < size and not one token later; weights are plain sigmoids
    (two equal keys weigh twice one)."""
    d = 4
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 1.0, "mask": {"size": 3}}
    w = {"q": np.eye(d), "o": np.eye(d), "pb": np.array([-20.0])}
    T = 6
    h = np.zeros((T, d))
    h[:, 0] = 40.0                                  # every query
    k = np.zeros((T, 1, d))
    v = np.zeros((T, 1, d))
    k[1, 0, 0], v[1, 0] = 1.0, [1.0, 2.0, 3.0, 4.0]    # score 40 - 20: weight 1; all other keys: sigmoid(-20)
    out = plain.sigmoid_attention(w, "", m, h, k, v)
    assert np.allclose(out[1], v[1, 0], atol=1e-6) and np.allclose(out[3], v[1, 0], atol=1e-6)      # i - j = 0 and 2
    assert np.abs(out[4]).max() < 1e-6 and np.abs(out[0]).max() < 1e-6                               # i - j = 3; j > i
    k[2, 0, 0], v[2, 0] = 1.0, v[1, 0]
    assert np.allclose(plain.sigmoid_attention(w, "", m, h, k, v)[3], 2 * v[1, 0], atol=1e-6)


def test_plain_recurrences_against_their_unrolled_sums():
    rng = np.random.default_rng(3)
    T, N, P = 9, 5, 4
    x, B, C = rng.normal(size=(T, P)), rng.normal(size=(T, N)), rng.normal(size=(T, N))
    dt = rng.uniform(0.1, 1.0, size=T)
    y = plain.state_space_head(x, B, C, dt, 0.7, 0.3)
    for t in range(T):          # y_t = sum_s prod_(s < r <= t) exp(-a dt_r) dt_s (C_t . B_s) x_s + D x_t
        want = 0.3 * x[t] + sum(np.exp(-0.7 * dt[s + 1:t + 1].sum()) * dt[s] * (C[t] @ B[s]) * x[s] for s in range(t + 1))
        assert np.allclose(y[t], want)
    # the delta rule with beta 1, no decay and orthonormal keys stores each value exactly; a key written twice is overwritten
    k = np.eye(N)[[0, 1, 2, 1]]
    v = rng.normal(size=(4, P))
    o = plain.delta_head(k, k, v, np.ones(4), np.ones((4, N)))
    assert np.allclose(o, v)
    S_read = plain.delta_head(np.eye(N)[[1, 1, 1, 1]], k, v, np.ones(4), np.ones((4, N)))
    assert np.allclose(S_read[3], v[3]) and np.allclose(S_read[2], v[1])
    # a decay on one key channel fades what that channel holds and nothing else
    g = np.ones((4, N))
    g[2:, 0] = 0.5
    o = plain.delta_head(np.eye(N)[[0, 0, 0, 0]], k, v, np.ones(4), g)
    assert np.allclose(o[1], v[0]) and np.allclose(o[2], 0.5 * v[0]) and np.allclose(o[3], 0.25 * v[0])


def test_plain_experts_scale_their_inputs(small):
    cfg, w = small
    f = cfg["layers"][0]["mlp"]
    h = np.random.default_rng(4).normal(size=(3, cfg["width"]))
    margins = []
    got = plain.routed(w, "l0.mlp.", f, h, margins)
    assert margins[0].shape == (3,) and (margins[0] > 0).all()
    for t in range(3):
        s = plain.sigmoid(w["l0.mlp.router"] @ h[t])
        best = sorted(range(len(s)), key=lambda e: -s[e])[:f["router"]["top"]]
        want = sum(plain.relu2((s[e] * h[t]) @ w[f"l0.mlp.e{e}.up"].T) @ w[f"l0.mlp.e{e}.down"].T for e in best)
        want = want + plain.relu2(h[t] @ w["l0.mlp.shared.up"].T) @ w["l0.mlp.shared.down"].T
        assert np.allclose(got[t], want)
