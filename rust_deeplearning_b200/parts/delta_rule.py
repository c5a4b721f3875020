"""The delta-rule mixer: a recurrent state that is corrected towards each token's value, with a decay per key channel.

From the mixer's input x: q and k (key heads x dim), v (heads x vdim), a write strength per head, and two low-rank
products for the decays (heads x dim) and the output gate (heads x vdim).  Along each sequence,
    (q, k, v) <- silu(conv(q, k, v))              a short causal convolution per channel, no bias, zeros before the start
    q, k      <- unit vectors per head, t / sqrt(sum(t^2) + unit_eps);  q times dim^(-1/2)          float32 from here on
    beta_h    = sigmoid(W_b x)_h
    g_h       = exp(-exp(A_log_h) softplus(W_a2 (W_a1 x) + dt_bias)_h)                  a decay per head and key channel
    S_h       <- g_h (.) S_h  (row i times g_h[i]);   u = beta_h (v_h - S_h^T k);   S_h <- S_h + k u^T;   o_h = S_h^T q
    out       = W_o (o_h / rms(o_h) * w_norm * sigmoid(W_g2 (W_g1 x))_h)
where head h reads q and k of key head h // (heads / key heads), S is [dim, vdim] and zero before the first token, and
the read-out sees the token's own write.  The norm's weight has vdim values and is shared by the heads.

Per sequence the cache keeps S in float32 and the last taps - 1 inputs of the convolution (`needs()` declares both).
Products: [W_q; W_k; W_v; W_b] in one, [W_a1; W_g1] in one, and the two second factors as one block-diagonal matrix on
the low-rank rows (its zero blocks cost less than a launch).  Every size, the taps and the constants are parameters.
"""
from __future__ import annotations

import torch

from ..cache.cache import RunCache, StateRequirement
from ..kernels import ops
from .registry import BuildContext, register_part
from .spec import PartSpec


class DeltaRule:
    def __init__(self, *, hidden_size, n_heads, n_key_heads, dim, vdim, taps, eps, unit_eps, q_scale, wq, wk, wv, wb, conv_q, conv_k,
                 conv_v, wa1, wa2, wg1, wg2, dt_bias, a_log, norm_weight, wo):
        if n_heads % n_key_heads:
            raise ValueError(f"delta_rule: {n_heads} heads cannot share {n_key_heads} key heads")
        if not 1 <= taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"delta_rule: {taps} taps, the convolution kernel takes 1 to {ops.SHORT_CONV_MAX_TAPS}")
        H, J = n_heads, n_key_heads
        self.hidden_size, self.n_heads, self.n_key_heads, self.dim, self.vdim = hidden_size, H, J, dim, vdim
        self.taps, self.eps, self.unit_eps, self.q_scale = taps, float(eps), float(unit_eps), float(q_scale)
        self.conv_channels = 2 * J * dim + H * vdim
        self.w_in = torch.cat([wq, wk, wv, wb], dim=0).contiguous()
        self.conv_w = torch.cat([conv_q, conv_k, conv_v], dim=0).contiguous()
        if tuple(self.conv_w.shape) != (self.conv_channels, taps):
            raise ValueError("delta_rule: the convolutions do not fit the sizes")
        ra, rg = wa1.shape[0], wg1.shape[0]
        self.w_low = torch.cat([wa1, wg1], dim=0).contiguous()
        up = torch.zeros((H * dim + H * vdim, ra + rg), dtype=wa2.dtype, device=wa2.device)
        up[:H * dim, :ra] = wa2
        up[H * dim:, ra:] = wg2
        self.w_up = up
        self.dt_bias = dt_bias.contiguous()
        self.a_log = a_log.to(torch.float32).contiguous()
        self.norm_weight = norm_weight.repeat(H).contiguous()      # a weight per column: the heads share vdim values
        self.w_o = wo
        self.b_col = self.conv_channels

    def needs(self):
        state = [StateRequirement((self.n_heads, self.dim, self.vdim), "float32")]
        if self.taps > 1:
            state.append(StateRequirement((self.taps - 1, self.conv_channels), "float32"))
        return None, tuple(state)

    def forward(self, x, batch, cache: RunCache, run: int):
        H, J, d, e = self.n_heads, self.n_key_heads, self.dim, self.vdim
        where = dict(tok_pos=batch.tok_pos, seq_start=batch.seq_start, slots=batch.slots)
        rows = ops.linear(x, self.w_in)
        wide = ops.linear(ops.linear(x, self.w_low), self.w_up)         # [decay logits heads x dim | gate logits heads x vdim]
        qkv = ops.short_conv(rows[:, :self.conv_channels], self.conv_w, None, cache.state[1] if self.taps > 1 else None,
                             tok_seq=batch.tok_seq, silu=True, **where)
        q_f, k_f, g_f, beta_f = ops.delta_prepare(qkv, q_col=0, k_col=J * d, n_heads=H, n_key_heads=J, dim=d,
                                                  decay_rows=wide[:, :H * d], beta_rows=rows[:, self.b_col:self.b_col + H],
                                                  dt_bias=self.dt_bias, a_log=self.a_log, q_scale=self.q_scale, unit_eps=self.unit_eps)
        o = ops.delta_rule_scan(qkv, v_col=2 * J * d, q_f=q_f, k_f=k_f, g_f=g_f, beta_f=beta_f, n_heads=H, n_key_heads=J, dim=d,
                                vdim=e, state=cache.state[0], n_seqs=batch.n_seqs, **where)
        y = ops.group_norm_gate(o, H, eps=self.eps, weight=self.norm_weight, gate=wide[:, H * d:], gate_kind="sigmoid", out_dtype=x.dtype)
        return ops.linear(y, self.w_o)


def _build_delta_rule(spec: PartSpec, ctx: BuildContext) -> DeltaRule:
    p, t = spec.params, spec.tensors
    g = lambda role: ctx.tensor(t[role])
    return DeltaRule(hidden_size=p["hidden_size"], n_heads=p["n_heads"], n_key_heads=p["n_key_heads"], dim=p["dim"], vdim=p["vdim"],
                     taps=p["taps"], eps=p["eps"], unit_eps=p.get("unit_eps", 1e-6), q_scale=p.get("q_scale", p["dim"] ** -0.5),
                     wq=g("q"), wk=g("k"), wv=g("v"), wb=g("beta"), conv_q=g("conv_q"), conv_k=g("conv_k"), conv_v=g("conv_v"),
                     wa1=g("decay_down"), wa2=g("decay_up"), wg1=g("gate_down"), wg2=g("gate_up"), dt_bias=g("dt_bias"),
                     a_log=g("a_log"), norm_weight=g("norm"), wo=g("o"))


register_part("mixer", "delta_rule", _build_delta_rule, replace=True)
