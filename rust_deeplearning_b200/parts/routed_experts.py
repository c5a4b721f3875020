"""A routed feed-forward: a router chooses, per token, a few of many small gated feed-forwards.

Per row x (`csrc/moe.cu`):
    z = W_r x                      float32 logits over all experts, identity experts included
    s = softmax(z)
    the `top` experts with the largest s + correction are taken; their weights are s itself, not renormalised
    y = sum_k s[e_k] * expert_{e_k}(x)
A real expert is W_down gated(W_gate x, W_up x) without biases, with the gated form and its parameter as
parameters (`ops.GATED_FORMS`); the last `n_identity` outputs of the router are identity experts, whose
output is x itself.  Rows are independent of each other, so packing and batching never concern the part.
Interface: `forward(x [rows, hidden] normed) -> [rows, hidden]`.

Further parameters, for designs that have them:
  scoring           "softmax" (above), "sigmoid": s = sigmoid(z), every expert's score by itself, or "softmax_chosen": the
                    `top` largest logits are taken and their weights are the softmax over those logits alone
  router_bias       a learned number per expert added to the logits, z = W_r x + b (tensor role "router_bias")
  form              a name of `ops.UNARY_FORMS` ("relu2", ...): experts of two matrices, W_down act(W_up x), built from
                    `up<e>` and `down<e>` alone
  weights_on_input  y = sum_k expert_{e_k}(s[e_k] * x): the score multiplies what the expert reads, not what it returns
  shared            an expert of the same form and a size of its own that every row takes; its result is kept apart
                    (`forward_parts` returns both), so that whoever adds them up can do so in float32
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .registry import BuildContext, register_part
from .spec import PartSpec


class RoutedExperts:
    def __init__(self, *, hidden_size, expert_size, n_experts, n_identity, top, form, form_param, w_router, correction,
                 gates, ups, downs, scoring="softmax", weights_on_input=False, shared=None, router_bias=None):
        if form not in ops.EXPERT_FORMS:
            raise ValueError(f"routed_experts: unknown expert form '{form}', known: {sorted(ops.EXPERT_FORMS)}")
        if scoring not in ops.ROUTE_SCORING:
            raise ValueError(f"routed_experts: unknown scoring '{scoring}', known: {sorted(ops.ROUTE_SCORING)}")
        if not 1 <= top <= n_experts + n_identity:
            raise ValueError(f"routed_experts: {top} of {n_experts + n_identity} experts cannot be chosen")
        self.hidden_size, self.expert_size = hidden_size, expert_size
        self.n_experts, self.n_identity, self.top = n_experts, n_identity, top
        self.form, self.form_param, self.unary = form, float(form_param), form in ops.UNARY_FORMS
        self.scoring, self.weights_on_input = scoring, bool(weights_on_input)
        self.w_router = w_router.to(torch.float32).contiguous()
        self.correction = correction.to(torch.float32).contiguous() if correction is not None else None
        self.router_bias = router_bias.to(torch.float32).contiguous() if router_bias is not None else None
        # [experts, 2 ff, hidden]: an expert's gate rows, then its up rows ([experts, ff, hidden] for experts of two
        # matrices); [experts, hidden, ff]
        if not n_experts:
            self.w_gate_up = self.w_down = None
        elif self.unary:
            self.w_gate_up = torch.stack(list(ups)).contiguous()
        else:
            self.w_gate_up = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]).contiguous()
        if n_experts:
            self.w_down = torch.stack(list(downs)).contiguous()
        # the expert every row takes: (gate or None, up, down)
        self.shared = None
        if shared is not None:
            g, u, d = shared
            self.shared = (u.contiguous() if self.unary else torch.cat([g, u], dim=0).contiguous(), d)

    def forward_parts(self, x):
        """(the routed experts' sum, the shared expert's result or None), each [rows, hidden]."""
        sel, sel_w = ops.moe_route(x, self.w_router, self.correction, self.top, self.scoring, bias=self.router_bias)
        routed = ops.moe_experts(x, sel, sel_w, self.w_gate_up, self.w_down, self.n_experts, self.form, self.form_param,
                                 weights_on_input=self.weights_on_input)
        if self.shared is None:
            return routed, None
        w_in, w_down = self.shared
        if self.unary:
            mid = ops.linear(x, w_in, activation=self.form)
        else:
            if self.form not in ops.ACTIVATIONS:
                raise ValueError(f"routed_experts: the shared expert takes the gated forms {sorted(ops.ACTIVATIONS)}, not '{self.form}'")
            mid = ops.linear_gated(x, w_in, self.form)
        return routed, ops.linear(mid, w_down)

    def forward(self, x):
        routed, shared = self.forward_parts(x)
        if shared is None:
            return routed
        out = routed.to(torch.float32) if routed.dtype is not torch.float32 else routed
        return ops.residual_add_(out, shared)


def _build_routed_experts(spec: PartSpec, ctx: BuildContext) -> RoutedExperts:
    p, t = spec.params, spec.tensors
    E = p["n_experts"]
    unary = p["form"] in ops.UNARY_FORMS
    shared = None
    if "shared_up" in t:
        shared = (None if unary else ctx.tensor(t["shared_gate"]), ctx.tensor(t["shared_up"]), ctx.tensor(t["shared_down"]))
    return RoutedExperts(hidden_size=p["hidden_size"], expert_size=p["expert_size"], n_experts=E, n_identity=p.get("n_identity", 0),
                         top=p["top"], form=p["form"], form_param=p.get("form_param", 0.0),
                         w_router=ctx.tensor(t["router"]), correction=ctx.tensor(t["correction"]) if "correction" in t else None,
                         gates=[] if unary else [ctx.tensor(t[f"gate{e}"]) for e in range(E)],
                         ups=[ctx.tensor(t[f"up{e}"]) for e in range(E)], downs=[ctx.tensor(t[f"down{e}"]) for e in range(E)],
                         scoring=p.get("scoring", "softmax"), weights_on_input=p.get("weights_on_input", False), shared=shared,
                         router_bias=ctx.tensor(t["router_bias"]) if "router_bias" in t else None)


register_part("feed_forward", "routed_experts", _build_routed_experts, replace=True)
