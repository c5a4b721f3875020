"""Revepel: typed configuration and its description as parts.

A decoder-only model whose layers are listed one by one in config.json.  Every layer is a parallel block
(`parts/model.py:ParallelBlock`) with one norm n = rms_norm(x), a token shift on what the mixer reads and a gate on
each branch:
    m_t = n_t + (n_(t-1) - n_t) * shift;    x <- x + sigmoid(R1 n + b1) * mixer(m) + sigmoid(R2 n + b2) * ff(n).
A layer's `type` names its mixer:

  "mamba2"         a selective state space with a scalar decay per head and token (`parts/state_space.py`);
  "channel_delta"  a delta rule with a decay per key channel (`parts/delta_rule.py`); the ranks of its two low-rank
                   products are the shapes of their tensors (optional keys `decay_rank`, `gate_rank` name them where
                   there is no file, as for random weights);
  "attention"      attention over a sliding window whose weights are sigmoid(score + a bias per head), not normalised
                   over the keys (`parts/attention.py` with `score_bias`), grouped key/value heads, rotary positions on
                   the first `rot.dims` dimensions (half-split pairs) with YaRN-blended frequencies.  With `kv_from: j`
                   the layer has no key and value projections and reads the keys and values layer j cached.

The feed-forward (`mlp`, or null) is a routed mixture of two-matrix experts W_down relu(W_up h)^2
(`parts/routed_experts.py`): sigmoid scores, the `top` largest chosen, the score multiplying the expert's input, plus an
optional expert every token takes.  The embedding is multiplied by `embedding.scale`; logits are
head(rms_norm(x)) * logit_scale with a head matrix of its own.

What the design fixes stands here (the activations, which gate comes before which norm, 1e-6 under the unit vectors'
root, dim^(-1/2) on q); every size and every other constant is read from config.json.  The design names no longest
context; tables of the position encoding are built for `max_positions` (an optional key of this library, default 32,768).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import Architecture, ConfigReader, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

ARCHITECTURE_NAME = "Revepel"
MODEL_TYPE = "revepel"
DEFAULT_MAX_POSITIONS = 32768
UNIT_EPS = 1e-6


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int]
    gate_rank: Optional[int]


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]]     # YaRN: factor, original, fast, slow; None: plain frequencies


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot: Optional[RotaryConfig]
    kv_from: Optional[int]


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class RevepelLayer:
    type: str
    mixer: Any
    mlp: Optional[MoEConfig]


@dataclass(frozen=True)
class RevepelConfig:
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    logit_scale: float
    max_positions: int
    layers: Tuple[RevepelLayer, ...]

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "RevepelConfig":
        r = ConfigReader(raw, "Revepel config")
        width = r.integer("width", minimum=1)
        vocab = r.integer("vocab", minimum=1)
        logit_scale = r.number("logit_scale")
        maxpos = r.integer("max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1)
        eps = _sub_number(r, raw, "norm", "eps", positive=True)
        scale = _sub_number(r, raw, "embedding", "scale")
        layers: List[RevepelLayer] = []
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            r.problems.append("key 'layers' must list at least one layer")
            listed = []
        for i, entry in enumerate(listed):
            layer, problems = _parse_layer(entry)
            r.problems += [f"layers[{i}]: {p}" for p in problems]
            if layer is not None:
                layers.append(layer)
        if len(layers) == len(listed):
            for i, layer in enumerate(layers):
                r.problems += [f"layers[{i}]: {p}" for p in _check_kv_from(i, layer, layers)]
        r.finish()
        return RevepelConfig(width, vocab, eps, scale, logit_scale, maxpos, tuple(layers))


def _sub_number(r: ConfigReader, raw, outer: str, key: str, positive: bool = False):
    if isinstance(raw.get(outer), dict):
        rr = ConfigReader(raw[outer], outer)
        v = rr.number(key, positive=positive)
        r.problems += [f"{outer}: {p}" for p in rr.problems]
        return v
    r.problems.append(f"missing key '{outer}' (an object with '{key}')")
    return None


def _parse_state_space(m):
    rm = ConfigReader(m, "mixer")
    heads = rm.integer("heads", minimum=1)
    vdim = rm.integer("vdim", minimum=1)
    state = rm.integer("state", minimum=1)
    groups = rm.integer("groups", minimum=1)
    norm_groups = rm.integer("norm_groups", minimum=1)
    conv = rm.integer("conv", minimum=1)
    if None not in (heads, groups):
        rm.check(heads % groups == 0, f"{heads} heads cannot share {groups} groups")
    if None not in (heads, vdim, norm_groups):
        rm.check((heads * vdim) % norm_groups == 0, f"{norm_groups} norm groups do not divide {heads * vdim} values")
    return (None if rm.problems else StateSpaceConfig(heads, vdim, state, groups, norm_groups, conv)), rm.problems


def _parse_delta(m):
    rm = ConfigReader(m, "mixer")
    heads = rm.integer("heads", minimum=1)
    kv_heads = rm.integer("kv_heads", minimum=1)
    dim = rm.integer("dim", minimum=1)
    vdim = rm.integer("vdim", minimum=1)
    conv = rm.integer("conv", minimum=1)
    decay_rank = rm.integer("decay_rank", default=0, minimum=0) or None
    gate_rank = rm.integer("gate_rank", default=0, minimum=0) or None
    if None not in (heads, kv_heads):
        rm.check(heads % kv_heads == 0, f"{heads} heads cannot share {kv_heads} key heads")
    return (None if rm.problems else DeltaConfig(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank)), rm.problems


def _parse_rot(m, rm: ConfigReader, dim) -> Optional[RotaryConfig]:
    if m.get("rot") is None:
        return None
    if not isinstance(m["rot"], dict):
        rm.problems.append("key 'rot' must be an object with 'base' and 'dims'")
        return None
    rr = ConfigReader(m["rot"], "rot")
    base = rr.number("base", positive=True)
    dims = rr.integer("dims", minimum=2)
    if dims is not None and dim is not None:
        rr.check(dims % 2 == 0 and dims <= dim, f"dims ({dims}) must be even and at most dim ({dim})")
    scaling = None
    sc = m["rot"].get("scaling")
    if sc is not None:
        if not isinstance(sc, dict):
            rr.problems.append("key 'scaling' must be an object or null")
        else:
            rs = ConfigReader(sc, "scaling")
            vals = {k: rs.number(k, positive=True) for k in ("factor", "original", "fast", "slow")}
            rr.problems += [f"scaling: {p}" for p in rs.problems]
            if not rs.problems:
                scaling = tuple(sorted(vals.items()))
    rm.problems += [f"rot: {p}" for p in rr.problems]
    return None if rr.problems else RotaryConfig(base, dims, scaling)


def _parse_attention(m):
    rm = ConfigReader(m, "mixer")
    heads = rm.integer("heads", minimum=1)
    kv_heads = rm.integer("kv_heads", minimum=1)
    dim = rm.integer("dim", minimum=1)
    vdim = rm.integer("vdim", minimum=1)
    scale = rm.number("scale")
    kv_from = rm.integer("kv_from", default=-1, minimum=-1)
    window = None
    if m.get("mask") is not None:
        if not isinstance(m["mask"], dict):
            rm.problems.append("key 'mask' must be an object with 'size'")
        else:
            rk = ConfigReader(m["mask"], "mask")
            window = rk.integer("size", minimum=1)
            rm.problems += [f"mask: {p}" for p in rk.problems]
    if None not in (heads, kv_heads):
        rm.check(heads % kv_heads == 0, f"{heads} heads cannot share {kv_heads} key/value heads")
    rot = _parse_rot(m, rm, dim)
    if rm.problems:
        return None, rm.problems
    return AttentionConfig(heads, kv_heads, dim, vdim, scale, window, rot, None if kv_from < 0 else kv_from), []


_MIXERS = {"mamba2": _parse_state_space, "channel_delta": _parse_delta, "attention": _parse_attention}


def _parse_mlp(f):
    if not isinstance(f, dict):
        return None, ["key 'mlp' must be an object or null"]
    rf = ConfigReader(f, "mlp")
    kind = rf.string("kind", default="moe")
    if kind is not None and kind != "moe":
        rf.problems.append(f"kind '{kind}' is not known (known: 'moe')")
    experts = top = ff = shared_ff = None
    if isinstance(f.get("router"), dict):
        rr = ConfigReader(f["router"], "router")
        experts = rr.integer("experts", minimum=1)
        top = rr.integer("top", minimum=1)
        if None not in (experts, top):
            rr.check(top <= experts, f"{top} of {experts} experts cannot be chosen")
        rf.problems += [f"router: {p}" for p in rr.problems]
    else:
        rf.problems.append("missing key 'router' (an object with 'experts' and 'top')")
    if isinstance(f.get("expert"), dict):
        re_ = ConfigReader(f["expert"], "expert")
        ff = re_.integer("ff", minimum=1)
        rf.problems += [f"expert: {p}" for p in re_.problems]
    else:
        rf.problems.append("missing key 'expert' (an object with 'ff')")
    if f.get("shared") is not None:
        if isinstance(f["shared"], dict):
            rs = ConfigReader(f["shared"], "shared")
            shared_ff = rs.integer("ff", minimum=1)
            rf.problems += [f"shared: {p}" for p in rs.problems]
        else:
            rf.problems.append("key 'shared' must be an object with 'ff' or null")
    if rf.problems:
        return None, [f"mlp: {p}" for p in rf.problems]
    return MoEConfig(experts, top, ff, shared_ff), []


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
            r.problems.append("missing key 'mixer' (an object with the mixer's sizes)")
        else:
            mixer, problems = _MIXERS[kind](entry["mixer"])
            r.problems += [f"mixer: {p}" for p in problems]
    mlp = None
    if entry.get("mlp") is not None:
        mlp, problems = _parse_mlp(entry["mlp"])
        r.problems += problems
    if r.problems:
        return None, r.problems
    return RevepelLayer(kind, mixer, mlp), []


def _check_kv_from(i: int, layer: RevepelLayer, layers) -> List[str]:
    if layer.type != "attention" or layer.mixer.kv_from is None:
        return []
    j, m = layer.mixer.kv_from, layer.mixer
    if not 0 <= j < i:
        return [f"kv_from {j} must name an earlier layer"]
    src = layers[j]
    if src.type != "attention" or src.mixer.kv_from is not None:
        return [f"kv_from {j} must name an attention layer with keys and values of its own"]
    s = src.mixer
    if (s.kv_heads, s.dim, s.vdim, s.rot) != (m.kv_heads, m.dim, m.vdim, m.rot):
        return [f"layer {j}'s key/value heads, sizes and rotation differ from this layer's"]
    return []


# ---- the description as parts ----

def _mat(name: str, out_features, in_features) -> TensorSpec:
    """A matrix [out, in]; random weights are drawn with a standard deviation of in^(-1/2), so that a product keeps the
    size of what it reads and every mechanism of a random model weighs in the logits."""
    return TensorSpec(name, (out_features, in_features), init_std=float(in_features or 16) ** -0.5)


def _state_space_part(cfg: RevepelConfig, m: StateSpaceConfig, p: str) -> PartSpec:
    W, inner, gn = cfg.width, m.heads * m.vdim, m.groups * m.state
    channels = inner + 2 * gn
    vec = lambda name, n, std, mean=0.0: TensorSpec(p + name, (n,), "vector", init_std=std, init_mean=mean)
    tensors = {"in": _mat(p + "in", 2 * inner + 2 * gn + m.heads, W),
               "conv": TensorSpec(p + "conv", (channels, m.conv), init_std=0.4), "conv_bias": vec("conv.b", channels, 0.1),
               "dt_bias": vec("dt_bias", m.heads, 0.5), "a_log": vec("A_log", m.heads, 0.5), "d_skip": vec("D", m.heads, 0.2, 1.0),
               "norm": vec("norm", inner, 0.1, 1.0), "o": _mat(p + "o", W, inner)}
    return PartSpec("state_space", {"hidden_size": W, "n_heads": m.heads, "vdim": m.vdim, "state_dim": m.state, "n_groups": m.groups,
                                    "taps": m.conv, "norm_groups": m.norm_groups, "eps": cfg.eps}, tensors)


def _delta_part(cfg: RevepelConfig, m: DeltaConfig, p: str) -> PartSpec:
    W, H, J, d, e = cfg.width, m.heads, m.kv_heads, m.dim, m.vdim
    conv = lambda name, n: TensorSpec(p + name, (n, m.conv), init_std=0.4)
    tensors = {"q": _mat(p + "q", J * d, W), "k": _mat(p + "k", J * d, W), "v": _mat(p + "v", H * e, W),
               "conv_q": conv("q.conv", J * d), "conv_k": conv("k.conv", J * d), "conv_v": conv("v.conv", H * e),
               "beta": _mat(p + "b", H, W),
               "a_log": TensorSpec(p + "A_log", (H,), "vector", init_std=0.5),
               "norm": TensorSpec(p + "norm", (e,), "vector", init_std=0.1, init_mean=1.0),
               "decay_down": _mat(p + "a1", m.decay_rank, W), "decay_up": TensorSpec(p + "a2", (H * d, m.decay_rank), init_std=0.1),
               "dt_bias": TensorSpec(p + "dt_bias", (H * d,), "vector", init_std=0.5),
               "gate_down": _mat(p + "g1", m.gate_rank, W), "gate_up": TensorSpec(p + "g2", (H * e, m.gate_rank), init_std=0.1),
               "o": _mat(p + "o", W, H * e)}
    return PartSpec("delta_rule", {"hidden_size": W, "n_heads": H, "n_key_heads": J, "dim": d, "vdim": e, "taps": m.conv, "eps": cfg.eps,
                                   "unit_eps": UNIT_EPS, "q_scale": d ** -0.5}, tensors)


def _attention_part(cfg: RevepelConfig, m: AttentionConfig, p: str, cache_window) -> PartSpec:
    W, H, G = cfg.width, m.heads, m.kv_heads
    tensors = {"q": _mat(p + "q", H * m.dim, W), "o": _mat(p + "o", W, H * m.vdim),
               "score_bias": TensorSpec(p + "pb", (H,), "vector", init_std=1.0, init_mean=-3.0)}
    if m.kv_from is None:
        tensors["k"] = _mat(p + "k", G * m.dim, W)
        tensors["v"] = _mat(p + "v", G * m.vdim, W)
    position = None
    if m.rot is not None:
        scaling = dict(m.rot.scaling, kind="yarn") if m.rot.scaling is not None else None
        position = PartSpec("rotary", {"theta": m.rot.base, "head_dim": max(m.dim, m.vdim), "rotary_dim": m.rot.dims,
                                       "max_positions": cfg.max_positions, "pairing": "half", "scaling": scaling})
    return PartSpec("attention", {"hidden_size": W, "n_heads": H, "n_kv_heads": G, "head_dim": m.dim, "value_dim": m.vdim,
                                  "score_scale": m.scale, "softcap": None, "window": m.window, "cache_window": cache_window,
                                  "position": position}, tensors)


def _moe_part(cfg: RevepelConfig, f: MoEConfig, p: str) -> PartSpec:
    W = cfg.width
    tensors = {"router": _mat(p + "router", f.experts, W)}
    for e in range(f.experts):
        tensors[f"up{e}"] = _mat(p + f"e{e}.up", f.ff, W)
        tensors[f"down{e}"] = _mat(p + f"e{e}.down", W, f.ff)
    if f.shared_ff is not None:
        tensors["shared_up"] = _mat(p + "shared.up", f.shared_ff, W)
        tensors["shared_down"] = _mat(p + "shared.down", W, f.shared_ff)
    return PartSpec("routed_experts", {"hidden_size": W, "expert_size": f.ff, "n_experts": f.experts, "n_identity": 0, "top": f.top,
                                       "form": "relu2", "scoring": "sigmoid", "weights_on_input": True}, tensors)


def build_spec(cfg: RevepelConfig) -> ModelSpec:
    """The model as parts; tensor names are the checkpoint's own ('l<i>.' + 'norm1', 'shift', 'rg1', 'mix.in', 'mlp.e0.up', ...)."""
    W, V = cfg.width, cfg.vocab
    # the keys an attention layer's cache keeps: its own window, or the widest window among the layers that read its keys
    keeps: Dict[int, Any] = {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "attention":
            owner = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            w = layer.mixer.window
            if owner not in keeps:
                keeps[owner] = w
            elif keeps[owner] is not None:
                keeps[owner] = None if w is None else max(keeps[owner], w)

    def norm(name):
        return PartSpec("rms_norm", {"size": W, "eps": cfg.eps, "offset": 0.0},
                        {"weight": TensorSpec(name, (W,), "vector", init_std=0.1, init_mean=1.0)})

    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        reads = None
        if layer.type == "mamba2":
            mixer = _state_space_part(cfg, layer.mixer, p + "mix.")
        elif layer.type == "channel_delta":
            mixer = _delta_part(cfg, layer.mixer, p + "mix.")
        else:
            keep = keeps[i] if layer.mixer.kv_from is None else layer.mixer.window
            mixer = _attention_part(cfg, layer.mixer, p + "mix.", "all" if (keep is None and layer.mixer.window is not None) else keep)
            reads = layer.mixer.kv_from
        tensors = {"shift": TensorSpec(p + "shift", (W,), "vector", init_std=0.2, init_mean=0.5),
                   "gate_mixer": _mat(p + "rg1", W, W), "gate_mixer_bias": TensorSpec(p + "rg1.b", (W,), "vector", init_std=0.5)}
        ff = None
        if layer.mlp is not None:
            ff = _moe_part(cfg, layer.mlp, p + "mlp.")
            tensors["gate_ff"] = _mat(p + "rg2", W, W)
            tensors["gate_ff_bias"] = TensorSpec(p + "rg2.b", (W,), "vector", init_std=0.5)
        layers.append(LayerSpec("parallel", mixer, ff, {"pre": norm(p + "norm1")},
                                {"hidden_size": W, "token_shift": True, "gated_residual": True}, tensors))
        schedule.append(ScheduleEntry(i, reads))

    spec = ModelSpec(
        architecture=ARCHITECTURE_NAME, hidden_size=W, vocab_size=V, max_positions=cfg.max_positions,
        embedding=PartSpec("scaled_embedding", {"vocab_size": V, "hidden_size": W, "scale": cfg.embedding_scale},
                           {"table": TensorSpec("embed", (V, W), init_std=0.05)}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": W, "softcap": None, "scale": cfg.logit_scale},
                      {"weight": _mat("head", V, W)}),
        ignored_tensors=tuple(f"l{i}.rg2*" for i, layer in enumerate(cfg.layers) if layer.mlp is None))
    spec.validate()
    return spec


register_architecture(Architecture(ARCHITECTURE_NAME, MODEL_TYPE, RevepelConfig.from_dict, build_spec), replace=True)
