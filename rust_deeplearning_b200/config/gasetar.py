"""Gasetar: typed configuration and its description as parts.

A decoder-only model of layers listed one by one in config.json.  Every layer is a parallel block: ONE scale-only
root-mean-square norm whose output both sublayers read, and one sum with a constant on the branches,
    n = norm1(x);   x <- x + m * (mixer(n) + ff(n)),   m = `residual_mult`.
`type` names the layer's mixer, `mixer` holds its sizes, `mlp` its feed-forward (null: none):

  attention          grouped-query attention (`parts/attention.py`): a norm over the whole query projection and over the
                     whole key projection (all heads at once, a learned weight per column) before the rotation; rotary
                     positions in half-split pairs on the first `rot.dims` dimensions of every head, with optional
                     `rot.scaling` (factor, low, high, original: long wavelengths slowed down, `parts/position.py`
                     kind "llama3"); scores times `scale`, soft-capped by `softcap`; a sliding window of `mask.size` keys
                     (the token itself and the mask.size - 1 before it); softmax; values of `vdim`.
  latent_attention   one cached latent row per token for all heads (`parts/latent_attention.py`): queries laid out per head
                     as [dim unrotated | rot_dim rotated], the latent normed, one rotated key part shared by the heads,
                     causal without a window, a learned sink per head in the softmax's denominator, and an output gate
                     with one row of W_g per value.
  mlp kind "dense"   W_down (silu(W_gate n) * (W_up n)) (`parts/feed_forward.py`).
  mlp kind "moe"     `router.experts` such feed-forwards of `expert.ff`, of which a token takes `router.top`: logits
                     W_r n + b in float, the largest chosen, weights the softmax over the chosen logits alone; plus an
                     optional shared expert of `shared.ff` that every token takes (`parts/routed_experts.py`).

The embedding rows are multiplied by `embedding.scale`; the embedding table is also the output matrix, and the logits are
cap * tanh(logit_scale * (E n) / cap) with cap = `logit_softcap` (null: no cap).

What the design fixes stands here (the arrangement, SiLU, half-split pairs, plain norm weights, which norms exist);
every size and every other constant is read from config.json.  The design names no longest context; tables of the
position encoding are built for `max_positions` (an optional key of this library, default 32,768).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

from .base import Architecture, ConfigReader, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

ARCHITECTURE_NAME = "Gasetar"
MODEL_TYPE = "gasetar"
DEFAULT_MAX_POSITIONS = 32768


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]]     # factor, low, high, original; None: plain frequencies


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    rot: Optional[RotaryConfig]


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class GasetarLayer:
    type: str
    mixer: Union[AttentionConfig, LatentConfig]
    mlp: Union[None, DenseConfig, MoEConfig]


def _sub(raw, key, reader: ConfigReader, required=True):
    """The object under `key` as a reader of its own, or None (a problem is noted if it is required or ill-typed)."""
    v = raw.get(key)
    if v is None:
        if required:
            reader.problems.append(f"missing key '{key}' (an object)")
        return None
    if not isinstance(v, dict):
        reader.problems.append(f"key '{key}' must be an object")
        return None
    return ConfigReader(v, key)


def _fold(parent: ConfigReader, child: Optional[ConfigReader]):
    if child is not None:
        parent.problems += [f"{child.what}: {p}" for p in child.problems]


def _parse_rot(m: Dict[str, Any], rm: ConfigReader, limit: Optional[int], limit_name: str, required: bool) -> Optional[RotaryConfig]:
    rr = _sub(m, "rot", rm, required)
    if rr is None:
        return None
    base = rr.number("base", positive=True)
    dims = rr.integer("dims", minimum=2)
    scaling = None
    rs = _sub(rr.raw, "scaling", rr, required=False)
    if rs is not None:
        vals = [(k, rs.number(k, positive=True)) for k in ("factor", "high", "low", "original")]
        if not rs.problems:
            rs.check(dict(vals)["high"] != dict(vals)["low"], "low and high must differ")
        _fold(rr, rs)
        scaling = tuple(vals)
    if dims is not None and limit is not None:
        rr.check(dims % 2 == 0 and dims <= limit, f"dims ({dims}) must be even and at most {limit_name} ({limit})")
    if base is not None:
        rr.check(base != 1.0, "base must not be 1")
    bad = bool(rr.problems)
    _fold(rm, rr)
    return None if bad else RotaryConfig(base, dims, scaling)


def _parse_attention(m: Dict[str, Any]):
    rm = ConfigReader(m, "mixer")
    heads = rm.integer("heads", minimum=1)
    kv_heads = rm.integer("kv_heads", default=heads, minimum=1)
    dim = rm.integer("dim", minimum=1)
    vdim = rm.integer("vdim", default=dim, minimum=1)
    scale = rm.number("scale")
    softcap = rm.number("softcap", default=None, positive=True)
    if heads is not None and kv_heads is not None:
        rm.check(heads % kv_heads == 0, f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    window = None
    rk = _sub(m, "mask", rm, required=False)
    if rk is not None:
        window = rk.integer("size", minimum=1)
        _fold(rm, rk)
    rot = _parse_rot(m, rm, dim, "dim", required=False)
    if rm.problems:
        return None, rm.problems
    return AttentionConfig(heads, kv_heads, dim, vdim, scale, softcap, window, rot), []


def _parse_latent(m: Dict[str, Any]):
    rm = ConfigReader(m, "mixer")
    heads = rm.integer("heads", minimum=1)
    dim = rm.integer("dim", minimum=1)
    rot_dim = rm.integer("rot_dim", minimum=2)
    vdim = rm.integer("vdim", minimum=1)
    kv_rank = rm.integer("kv_rank", minimum=1)
    scale = rm.number("scale")
    rot = _parse_rot(m, rm, rot_dim, "rot_dim", required=True)
    if rm.problems:
        return None, rm.problems
    return LatentConfig(heads, dim, rot_dim, vdim, kv_rank, scale, rot), []


_MIXERS = {"attention": _parse_attention, "latent_attention": _parse_latent}


def _parse_mlp(f):
    if not isinstance(f, dict):
        return None, ["key 'mlp' must be an object or null"]
    rf = ConfigReader(f, "mlp")
    kind = rf.string("kind")
    out = None
    if kind == "dense":
        ff = rf.integer("ff", minimum=1)
        out = DenseConfig(ff)
    elif kind == "moe":
        ff = experts = top = shared = None
        re_ = _sub(f, "expert", rf)
        if re_ is not None:
            ff = re_.integer("ff", minimum=1)
            _fold(rf, re_)
        rr = _sub(f, "router", rf)
        if rr is not None:
            experts = rr.integer("experts", minimum=1)
            top = rr.integer("top", minimum=1)
            if experts is not None and top is not None:
                rr.check(top <= experts, f"top ({top}) of {experts} experts cannot be chosen")
            _fold(rf, rr)
        rs = _sub(f, "shared", rf, required=False)
        if rs is not None:
            shared = rs.integer("ff", minimum=1)
            _fold(rf, rs)
        out = MoEConfig(experts, top, ff, shared)
    elif kind is not None:
        rf.problems.append(f"kind '{kind}' is not known (known: 'dense', 'moe')")
    if rf.problems:
        return None, [f"mlp: {p}" for p in rf.problems]
    return out, []


def _parse_layer(entry):
    if not isinstance(entry, dict):
        return None, ["must be an object"]
    r = ConfigReader(entry, "layer")
    kind = r.string("type")
    mixer = None
    if kind is not None and kind not in _MIXERS:
        r.problems.append(f"type '{kind}' is not known (known: {sorted(_MIXERS)})")
    elif kind is not None:
        if not isinstance(entry.get("mixer"), dict):
            r.problems.append("missing key 'mixer' (an object)")
        else:
            mixer, problems = _MIXERS[kind](entry["mixer"])
            r.problems += [f"mixer: {p}" for p in problems]
    mlp = None
    if entry.get("mlp") is not None:
        mlp, problems = _parse_mlp(entry["mlp"])
        r.problems += problems
    if r.problems:
        return None, r.problems
    return GasetarLayer(kind, mixer, mlp), []


@dataclass(frozen=True)
class GasetarConfig:
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    residual_mult: float
    logit_scale: float
    logit_softcap: Optional[float]
    max_positions: int
    layers: Tuple[GasetarLayer, ...]

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "GasetarConfig":
        r = ConfigReader(raw, "Gasetar config")
        width = r.integer("width", minimum=1)
        vocab = r.integer("vocab", minimum=1)
        mult = r.number("residual_mult", default=1.0)
        logit_scale = r.number("logit_scale", default=1.0, positive=True)
        logit_softcap = r.number("logit_softcap", default=None, positive=True)
        maxpos = r.integer("max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1)
        eps = emb_scale = None
        rn = _sub(raw, "norm", r)
        if rn is not None:
            eps = rn.number("eps", positive=True)
            _fold(r, rn)
        emb_scale = 1.0
        re_ = _sub(raw, "embedding", r, required=False)
        if re_ is not None:
            emb_scale = re_.number("scale", default=1.0)
            _fold(r, re_)
        layers: List[GasetarLayer] = []
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            r.problems.append("key 'layers' must list at least one layer")
            listed = []
        for i, entry in enumerate(listed):
            layer, problems = _parse_layer(entry)
            r.problems += [f"layers[{i}]: {p}" for p in problems]
            if layer is not None:
                layers.append(layer)
        r.finish()
        return GasetarConfig(width, vocab, eps, emb_scale, mult, logit_scale, logit_softcap, maxpos, tuple(layers))


# ---- the description as parts ----

def _mat(name: str, out_features: int, in_features: int) -> TensorSpec:
    """A matrix [out, in]; random weights are drawn with a standard deviation of in^(-1/2), so that a product keeps the
    size of what it reads and every mechanism of a random model weighs in the logits."""
    return TensorSpec(name, (out_features, in_features), init_std=float(in_features) ** -0.5)


def _plain_weight(name: str, n: int) -> TensorSpec:
    return TensorSpec(name, (n,), "vector", init_std=0.1, init_mean=1.0)


def _rotary(rot: RotaryConfig, head_dim: int, max_positions: int) -> PartSpec:
    scaling = dict(rot.scaling, kind="llama3") if rot.scaling is not None else None
    return PartSpec("rotary", {"theta": rot.base, "head_dim": head_dim, "rotary_dim": rot.dims, "max_positions": max_positions,
                               "pairing": "half", "scaling": scaling})


def _attention_part(cfg: GasetarConfig, m: AttentionConfig, p: str) -> PartSpec:
    W, H, G = cfg.width, m.heads, m.kv_heads
    tensors = {"q": _mat(p + "q", H * m.dim, W), "k": _mat(p + "k", G * m.dim, W), "v": _mat(p + "v", G * m.vdim, W),
               "q_norm": _plain_weight(p + "q.norm", H * m.dim), "k_norm": _plain_weight(p + "k.norm", G * m.dim),
               "o": _mat(p + "o", W, H * m.vdim)}
    position = _rotary(m.rot, max(m.dim, m.vdim), cfg.max_positions) if m.rot is not None else None
    return PartSpec("attention", {"hidden_size": W, "n_heads": H, "n_kv_heads": G, "head_dim": m.dim, "value_dim": m.vdim,
                                  "score_scale": m.scale, "softcap": m.softcap, "window": m.window, "proj_norm_eps": cfg.eps,
                                  "position": position}, tensors)


def _latent_part(cfg: GasetarConfig, m: LatentConfig, p: str) -> PartSpec:
    W, H, d, rd, vd, r = cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
    tensors = {"q": _mat(p + "q", H * (d + rd), W), "dkv": _mat(p + "dkv", r + rd, W),
               "dkv_norm": _plain_weight(p + "dkv.norm", r),
               "uk": _mat(p + "uk", H * d, r), "uv": _mat(p + "uv", H * vd, r),
               "sinks": TensorSpec(p + "sink", (H,), "vector", init_std=1.0),
               "g": _mat(p + "g", H * vd, W), "o": _mat(p + "o", W, H * vd)}
    return PartSpec("latent_attention", {"hidden_size": W, "n_heads": H, "dim": d, "rot_dim": rd, "vdim": vd, "kv_rank": r,
                                         "score_scale": m.scale, "window": None, "cache_window": None, "eps": cfg.eps,
                                         "gate_per_value": True, "position": _rotary(m.rot, rd, cfg.max_positions)}, tensors)


def _dense_part(cfg: GasetarConfig, f: DenseConfig, p: str) -> PartSpec:
    W = cfg.width
    return PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": f.ff, "activation": "silu"},
                    {"gate": _mat(p + "gate", f.ff, W), "up": _mat(p + "up", f.ff, W), "down": _mat(p + "down", W, f.ff)})


def _moe_part(cfg: GasetarConfig, f: MoEConfig, p: str) -> PartSpec:
    W = cfg.width
    tensors = {"router": _mat(p + "router", f.experts, W),
               "router_bias": TensorSpec(p + "router.b", (f.experts,), "vector", init_std=0.5)}
    for e in range(f.experts):
        tensors[f"gate{e}"] = _mat(p + f"e{e}.gate", f.ff, W)
        tensors[f"up{e}"] = _mat(p + f"e{e}.up", f.ff, W)
        tensors[f"down{e}"] = _mat(p + f"e{e}.down", W, f.ff)
    if f.shared_ff is not None:
        tensors["shared_gate"] = _mat(p + "shared.gate", f.shared_ff, W)
        tensors["shared_up"] = _mat(p + "shared.up", f.shared_ff, W)
        tensors["shared_down"] = _mat(p + "shared.down", W, f.shared_ff)
    return PartSpec("routed_experts", {"hidden_size": W, "expert_size": f.ff, "n_experts": f.experts, "n_identity": 0, "top": f.top,
                                       "form": "silu", "scoring": "softmax_chosen"}, tensors)


def build_spec(cfg: GasetarConfig) -> ModelSpec:
    """The model as parts; tensor names are the checkpoint's own ('l<i>.' + 'norm1', 'mix.q', 'mix.q.norm', 'mlp.e<k>.gate', ...)."""
    W, V = cfg.width, cfg.vocab

    def norm(name):
        return PartSpec("rms_norm", {"size": W, "eps": cfg.eps, "offset": 0.0}, {"weight": _plain_weight(name, W)})

    layers: List[LayerSpec] = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        if layer.type == "attention":
            mixer = _attention_part(cfg, layer.mixer, p + "mix.")
        else:
            mixer = _latent_part(cfg, layer.mixer, p + "mix.")
        ff = None
        if isinstance(layer.mlp, DenseConfig):
            ff = _dense_part(cfg, layer.mlp, p + "mlp.")
        elif isinstance(layer.mlp, MoEConfig):
            ff = _moe_part(cfg, layer.mlp, p + "mlp.")
        layers.append(LayerSpec("parallel", mixer, ff, {"pre": norm(p + "norm1")},
                                {"hidden_size": W, "branch_scale": cfg.residual_mult}))
    table = TensorSpec("embed", (V, W), init_std=W ** -0.5)
    spec = ModelSpec(
        architecture=ARCHITECTURE_NAME, hidden_size=W, vocab_size=V, max_positions=cfg.max_positions,
        embedding=PartSpec("scaled_embedding", {"vocab_size": V, "hidden_size": W, "scale": cfg.embedding_scale}, {"table": table}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i, None) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": W, "softcap": cfg.logit_softcap, "pre_scale": cfg.logit_scale},
                      {"weight": table}))
    spec.validate()
    return spec


register_architecture(Architecture(ARCHITECTURE_NAME, MODEL_TYPE, GasetarConfig.from_dict, build_spec), replace=True)
