"""The state-space mixer: a selective state space with a scalar decay per head and token (the "state-space duality" form).

One product makes, from the mixer's input x, the row [z | u | B | C | dt] with inner = heads * vdim values of z and
of u, groups * state values of B and of C, and one raw step size per head.  Then, along each sequence,
    (u, B, C) <- silu(conv(u, B, C))         a short causal convolution per channel with a bias, zeros before the start
    dt_h      = softplus(dt_h + dt_bias_h)    float32 from here on
    S_h,t     = exp(-exp(A_log_h) dt_h) S_h,t-1 + dt_h B_g(h),t u_h,t^T        S [state, vdim], zero before the first token
    y_h,t     = S_h,t^T C_g(h),t + D_h u_h,t
    out       = W_o (norm_parts(y * silu(z)) * w_norm)
where head h reads B and C of group g(h) = h // (heads / groups), and the gated y is divided by its root mean square in
`norm_groups` equal parts (the gate comes before the norm).

Per sequence the cache keeps two things of fixed size (`needs()` declares both): S in float32 and the last taps - 1
inputs of the convolution, so that a sequence's tokens may arrive whole, in portions or one by one.  Every constant
(sizes, taps, groups, how many parts the norm has, eps) is a parameter.
"""
from __future__ import annotations

import torch

from ..cache.cache import RunCache, StateRequirement
from ..kernels import ops
from .registry import BuildContext, register_part
from .spec import PartSpec


def _f32(t):
    return t.to(torch.float32).contiguous()


class StateSpace:
    def __init__(self, *, hidden_size, n_heads, vdim, state_dim, n_groups, taps, norm_groups, eps, w_in, conv_w, conv_b,
                 dt_bias, a_log, d_skip, norm_weight, w_o):
        if n_heads % n_groups:
            raise ValueError(f"state_space: {n_heads} heads cannot share {n_groups} groups of B and C")
        inner = n_heads * vdim
        if inner % norm_groups:
            raise ValueError(f"state_space: {norm_groups} norm parts do not divide {inner} values")
        if not 1 <= taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"state_space: {taps} taps, the convolution kernel takes 1 to {ops.SHORT_CONV_MAX_TAPS}")
        self.hidden_size, self.n_heads, self.vdim, self.state_dim, self.n_groups = hidden_size, n_heads, vdim, state_dim, n_groups
        self.taps, self.norm_groups, self.eps, self.inner = taps, norm_groups, float(eps), inner
        self.conv_channels = inner + 2 * n_groups * state_dim
        width = 2 * inner + 2 * n_groups * state_dim + n_heads
        if tuple(w_in.shape) != (width, hidden_size) or tuple(conv_w.shape) != (self.conv_channels, taps):
            raise ValueError("state_space: the input product or the convolution does not fit the sizes")
        self.w_in, self.w_o = w_in, w_o
        self.conv_w, self.conv_b = conv_w.contiguous(), conv_b
        self.dt_bias, self.a_log = _f32(dt_bias), _f32(a_log)
        self.d_skip = _f32(d_skip) if d_skip is not None else None
        self.norm_weight = norm_weight
        self.dt_col = width - n_heads

    def needs(self):
        state = [StateRequirement((self.n_heads, self.state_dim, self.vdim), "float32")]
        if self.taps > 1:
            state.append(StateRequirement((self.taps - 1, self.conv_channels), "float32"))
        return None, tuple(state)

    def forward(self, x, batch, cache: RunCache, run: int):
        inner, gn = self.inner, self.n_groups * self.state_dim
        where = dict(tok_pos=batch.tok_pos, seq_start=batch.seq_start, slots=batch.slots)
        rows = ops.linear(x, self.w_in)
        ubc = ops.short_conv(rows[:, inner:inner + self.conv_channels], self.conv_w, self.conv_b,
                             cache.state[1] if self.taps > 1 else None, tok_seq=batch.tok_seq, silu=True, **where)
        y = ops.state_space_scan(ubc, rows[:, self.dt_col:], x_col=0, b_col=inner, c_col=inner + gn, n_heads=self.n_heads,
                                 n_groups=self.n_groups, state_dim=self.state_dim, vdim=self.vdim, dt_bias=self.dt_bias,
                                 a_log=self.a_log, d_skip=self.d_skip, state=cache.state[0], n_seqs=batch.n_seqs, **where)
        y = ops.group_norm_gate(y, self.norm_groups, eps=self.eps, weight=self.norm_weight, gate=rows[:, :inner], gate_kind="silu",
                                out_dtype=x.dtype, gate_first=True)
        return ops.linear(y, self.w_o)


def _build_state_space(spec: PartSpec, ctx: BuildContext) -> StateSpace:
    p, t = spec.params, spec.tensors
    return StateSpace(hidden_size=p["hidden_size"], n_heads=p["n_heads"], vdim=p["vdim"], state_dim=p["state_dim"],
                      n_groups=p["n_groups"], taps=p["taps"], norm_groups=p.get("norm_groups", 1), eps=p["eps"],
                      w_in=ctx.tensor(t["in"]), conv_w=ctx.tensor(t["conv"]), conv_b=ctx.tensor(t["conv_bias"]) if "conv_bias" in t else None,
                      dt_bias=ctx.tensor(t["dt_bias"]), a_log=ctx.tensor(t["a_log"]), d_skip=ctx.tensor(t["d_skip"]) if "d_skip" in t else None,
                      norm_weight=ctx.tensor(t["norm"]) if "norm" in t else None, w_o=ctx.tensor(t["o"]))


register_part("mixer", "state_space", _build_state_space, replace=True)
