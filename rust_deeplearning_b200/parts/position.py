"""Position encodings.

`Rotary`: inv_i = theta^(-2i/d), angle = position * inv_i, half-split pairing
(`rustml/nn/main/src/core/rope.rs:93-108, :188-191`).  theta, the head size, how
many of its dimensions rotate and the number of positions are parameters.  The
reference forms theta^(...), the angle and cos/sin in float32; here the angle is
formed in float64 on the host and cos/sin are stored as float32 tables, which
keeps positions in the thousands exact to float32 rounding.

Two further parameters of `Rotary`.  `pairing`: "half" pairs dimension i with i + n/2 (above); "interleaved"
pairs 2i with 2i + 1, (u, v) -> (u cos a - v sin a, v cos a + u sin a).  `scaling`: None, or a dictionary
{"kind": "yarn", "factor", "original", "fast", "slow"} that blends each frequency f_i between itself and
f_i / factor:
    d(t)   = n ln(original / (2 pi t)) / (2 ln theta)        the pair index whose wavelength makes t turns in `original` positions
    lo, hi = max(floor(d(fast)), 0), min(ceil(d(slow)), n - 1)
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    f_i   <- f_i / factor * ramp_i + f_i (1 - ramp_i)
and multiplies cos and sin by 0.1 ln(factor) + 1.  A second kind, {"kind": "llama3", "factor", "low", "high",
"original"}, slows the long wavelengths down and leaves the short ones alone: with l_i = 2 pi / f_i,
    l_i < original / high:  f_i stays;      l_i > original / low:  f_i <- f_i / factor;
    between:  s = (original / l_i - low) / (high - low),   f_i <- (1 - s) f_i / factor + s f_i
(cos and sin keep their size).  All of it is in the tables, so kernels need not know of it.

Interface of a position encoding, as an attention mixer uses it:
`rotate(rows, n_heads, n_kv_heads, head_dim, batch)` rotates, in place, the query and
key heads of packed rows [tokens, (n_heads + 2 n_kv_heads) * head_dim] at the rows'
positions.  A part that also offers `tables(device)` and `rotary_dim` lets the
mixer fuse the rotation with the cache write in one kernel.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .registry import BuildContext, register_part
from .spec import PartSpec


def rotary_frequencies(theta: float, n: int, scaling: Optional[dict] = None):
    """float64 frequencies [n / 2] and the factor on cos and sin, for the parameters above."""
    half = n // 2
    i = torch.arange(half, dtype=torch.float64)
    inv = torch.tensor(float(theta), dtype=torch.float64) ** (-2.0 * i / n)
    if scaling is None:
        return inv, 1.0
    if scaling.get("kind") == "llama3":
        factor, original = float(scaling["factor"]), float(scaling["original"])
        low, high = float(scaling["low"]), float(scaling["high"])
        if high == low:
            raise ValueError("rotary scaling 'llama3': low and high must differ")
        wavelength = 2.0 * math.pi / inv
        s = (original / wavelength - low) / (high - low)
        blended = (1.0 - s) * inv / factor + s * inv
        out = torch.where(wavelength < original / high, inv, torch.where(wavelength > original / low, inv / factor, blended))
        return out, 1.0
    if scaling.get("kind") != "yarn":
        raise ValueError(f"rotary scaling of kind {scaling.get('kind')!r} is not known (known: 'yarn', 'llama3')")
    factor, original = float(scaling["factor"]), float(scaling["original"])
    d = lambda turns: n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))
    lo = max(math.floor(d(float(scaling["fast"]))), 0)
    hi = min(math.ceil(d(float(scaling["slow"]))), n - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return inv / factor * ramp + inv * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class Rotary:
    def __init__(self, theta: float, head_dim: int, rotary_dim: int, max_positions: int, device,
                 pairing: str = "half", scaling: Optional[dict] = None):
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing '{pairing}' is not one of 'half', 'interleaved'")
        self.theta, self.head_dim, self.rotary_dim, self.max_positions = float(theta), head_dim, rotary_dim, max_positions
        self.pairing, self.interleaved = pairing, pairing == "interleaved"
        inv, magnitude = rotary_frequencies(self.theta, rotary_dim, scaling)
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos = (torch.cos(ang) * magnitude).to(torch.float32).contiguous().to(device)
        self.sin = (torch.sin(ang) * magnitude).to(torch.float32).contiguous().to(device)

    def tables(self):
        return self.cos, self.sin

    def rotate(self, rows, n_heads, n_kv_heads, head_dim, batch):
        if self.interleaved:
            raise ValueError("the interleaved pairing is applied by the kernels of the mixers that use it, from tables()")
        ops.rope_cache(rows, n_heads, n_kv_heads, head_dim, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                       cos=self.cos, sin=self.sin, rotary_dim=self.rotary_dim)


def _build_rotary(spec: PartSpec, ctx: BuildContext) -> Rotary:
    p = spec.params
    scaling = p.get("scaling")
    key = ("rotary", p["theta"], p["head_dim"], p["rotary_dim"], p["max_positions"], p.get("pairing", "half"),
           tuple(sorted(scaling.items())) if scaling else None)
    if key not in ctx.shared:     # one table for all layers that share the parameters
        ctx.shared[key] = Rotary(p["theta"], p["head_dim"], p["rotary_dim"], p["max_positions"], ctx.device,
                                 pairing=p.get("pairing", "half"), scaling=scaling)
    return ctx.shared[key]


register_part("position", "rotary", _build_rotary, replace=True)
