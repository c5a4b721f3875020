"""Tiny Gasetar configurations for the tests.  They differ from each other in every size and option:
  GA  four layers in an order of its own: latent attention first, a dense layer without rotation scaling, a layer
      without feed-forward, routed layers with and without a shared expert; windows of 5 and 9 keys; values narrower
      and wider than keys; sizes that are no multiples of 8 (the kernels' plain forms)
  GB  sizes the fast kernels take (heads of 64, cached rows of 64 values, a window of 33), three query heads a key head,
      multipliers and scales of 1, no caps, every head its own key head in one layer
  GC  as GB's shapes with every expert chosen (no choice can flip between number formats), for long runs in bfloat16
"""
import copy


def _rot(base, dims, scaling=None):
    return {"base": base, "dims": dims, **({"scaling": scaling} if scaling else {})}


def _attn(heads, kv_heads, dim, vdim, scale, softcap, window, rot):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, rot):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}


def _moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


_SCALED = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
GA = {
    "architecture": "Gasetar", "width": 72, "vocab": 210, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "residual_mult": 0.6, "logit_scale": 0.8, "logit_softcap": 12.0, "max_positions": 512,
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 12, 6, 20, 28, 0.2, _rot(200.0, 6)), "mlp": _moe(5, 2, 20, shared=12)},
        {"type": "attention", "mixer": _attn(6, 2, 12, 20, 0.3, 8.0, 5, _rot(3000.0, 6, _SCALED)), "mlp": {"kind": "dense", "ff": 44}},
        {"type": "attention", "mixer": _attn(4, 4, 20, 12, 0.2, 15.0, 9, _rot(100.0, 20)), "mlp": None},
        {"type": "latent_attention", "mixer": _latent(5, 4, 10, 6, 14, 0.35, _rot(50.0, 10)), "mlp": _moe(3, 1, 28)},
    ],
}
_ROT_B = _rot(20000.0, 32, {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 128})
GB = {
    "architecture": "Gasetar", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "residual_mult": 1.0, "logit_scale": 1.0, "max_positions": 1024,
    "layers": [
        {"type": "attention", "mixer": _attn(6, 2, 64, 64, 1.0 / 8.0, None, 33, _ROT_B), "mlp": _moe(8, 2, 64, shared=32)},
        {"type": "latent_attention", "mixer": _latent(4, 40, 24, 24, 40, 0.14, _rot(10000.0, 24)), "mlp": {"kind": "dense", "ff": 96}},
        {"type": "attention", "mixer": _attn(2, 2, 64, 64, 1.0 / 8.0, 30.0, None, _rot(500.0, 64)), "mlp": _moe(8, 2, 64)},
    ],
}
GC = copy.deepcopy(GB)
GC["layers"][0]["mlp"] = _moe(3, 3, 32, shared=32)
GC["layers"][2]["mlp"] = _moe(2, 2, 48)
GC["embedding"]["scale"] = 2.0
GC["logit_softcap"] = 20.0

CONFIGS = {"GA": (GA, 31), "GB": (GB, 32), "GC": (GC, 33)}


def config(name):
    cfg, seed = CONFIGS[name]
    return copy.deepcopy(cfg), seed
