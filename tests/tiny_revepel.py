"""Tiny Revepel configurations for the tests.  They differ from each other in every size, constant and in the order of
their layers:
  RA  attention first (window 8, YaRN-blended rotation on half of a head), a delta layer whose 4 heads share 2 key
      heads with values wider than keys and 4 taps, a state space with 2 groups and a norm in 2 parts, then an
      attention layer that reads layer 0's keys through a WIDER window (12) with other query heads; top 2 of 5 experts
  RB  sizes no fast kernel takes (heads of 12, 20 and 24 values, 6 rotated dimensions of 12, width 72), a state space
      first with 2 taps and one head per group, an attention layer without window and without feed-forward, read again
      by a later layer through a window of 5; a delta layer with one tap (no convolution state) and one key head for
      all heads; a layer without shared expert; every expert chosen in one layer
  RC  sizes the tensor-core kernels take (heads of 64, width 128), windows of 40 and 33 on shared keys (the reader's
      narrower), 3 taps, one expert of one
"""
import copy


def _rot(base, dims, scaling=None):
    return {"base": base, "dims": dims, **({"scaling": scaling} if scaling else {})}


def _ssm(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def _delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank, "gate_rank": gate_rank}


def _attn(heads, kv_heads, dim, vdim, scale, rot, window=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, shared_ff=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff is not None:
        m["shared"] = {"ff": shared_ff}
    return m


_ROT_A = _rot(5000.0, 8, {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0})
RA = {
    "architecture": "Revepel", "width": 64, "vocab": 210, "norm": {"eps": 1e-5}, "embedding": {"scale": 6.0}, "logit_scale": 0.5,
    "max_positions": 1024,
    "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 16, 16, 0.3, _ROT_A, window=8), "mlp": _moe(5, 2, 24, 40)},
        {"type": "channel_delta", "mixer": _delta(4, 2, 16, 24, 4, 8, 16), "mlp": _moe(3, 1, 32, 16)},
        {"type": "mamba2", "mixer": _ssm(4, 16, 8, 2, 2, 4), "mlp": None},
        {"type": "attention", "mixer": _attn(2, 2, 16, 16, 0.5, _ROT_A, window=12, kv_from=0), "mlp": _moe(4, 2, 16)},
    ],
}
_ROT_B = _rot(300.0, 6)
RB = {
    "architecture": "Revepel", "width": 72, "vocab": 131, "norm": {"eps": 1e-4}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "max_positions": 700,
    "layers": [
        {"type": "mamba2", "mixer": _ssm(3, 20, 12, 3, 1, 2), "mlp": _moe(3, 3, 20, 24)},
        {"type": "attention", "mixer": _attn(3, 3, 12, 20, 0.4, _ROT_B), "mlp": None},
        {"type": "channel_delta", "mixer": _delta(3, 1, 12, 24, 1, 5, 7), "mlp": _moe(4, 1, 40)},
        {"type": "attention", "mixer": _attn(6, 3, 12, 20, 0.25, _ROT_B, window=5, kv_from=1), "mlp": _moe(2, 1, 8, 8)},
        {"type": "mamba2", "mixer": _ssm(2, 36, 5, 1, 3, 3), "mlp": None},
    ],
}
_ROT_C = _rot(20000.0, 32, {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 2.0})
RC = {
    "architecture": "Revepel", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.0}, "logit_scale": 0.125,
    "max_positions": 2048,
    "layers": [
        {"type": "channel_delta", "mixer": _delta(2, 2, 64, 64, 3, 16, 16), "mlp": _moe(1, 1, 64, 64)},
        {"type": "attention", "mixer": _attn(4, 1, 64, 64, 0.11, _ROT_C, window=40), "mlp": _moe(8, 2, 32, 64)},
        {"type": "mamba2", "mixer": _ssm(2, 64, 64, 1, 1, 3), "mlp": _moe(4, 1, 48)},
        {"type": "attention", "mixer": _attn(2, 1, 64, 64, 0.2, _ROT_C, window=33, kv_from=1), "mlp": None},
    ],
}

CONFIGS = {"RA": (RA, 41), "RB": (RB, 42), "RC": (RC, 43)}

# after the random weights are made: heads that forget nothing (a token far back stays in their state), so that a lost
# state shows at the end of a long sequence; (tensor, index, value)
ADJUST = {
    "RA": [("l1.mix.A_log", 0, -9.0), ("l2.mix.A_log", 1, -9.0), ("l2.mix.dt_bias", 1, 1.0)],
    "RB": [("l0.mix.A_log", 0, -9.0), ("l2.mix.A_log", 2, -9.0)],
    "RC": [("l0.mix.A_log", 1, -9.0), ("l2.mix.A_log", 0, -9.0)],
}


def config(name):
    """A name with an x at its end: the same model (sizes, seed, weights) with every expert chosen in every layer, so
    that no choice can flip between number formats."""
    cfg, seed = CONFIGS[name.rstrip("x")]
    cfg = copy.deepcopy(cfg)
    if name.endswith("x"):
        for layer in cfg["layers"]:
            if layer["mlp"] is not None:
                layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return cfg, seed
