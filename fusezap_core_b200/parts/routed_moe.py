"""Mixture of small gated feed-forwards chosen by a softmax router, with groups of experts and a shared expert.

Router logits `z = W_router h` leave the product in float32; scores `s = softmax(z)` over all experts. The experts form
`groups` equal groups of neighbours; a group's score is its largest score, and only experts of the best `keep_groups`
groups can be chosen. Of those the `top` with the largest scores are taken (the lower index first among equals); their
weights are their scores (divided by their sum if `renormalize`). Expert e: `W_down,e (silu(W_gate,e h) * (W_up,e h))`,
no biases. A shared expert of the same form (`shared_size` > 0) runs for every token and is added times
`sigmoid(W_sg h)`, one number per token. The step sorts its (row, choice) pairs by expert on the device and runs each
expert's products over its own rows only; a row's result does not depend on the other rows. Router, softmax, weights
and the weighted sum are 32-bit; the activation is computed from unrounded 32-bit sums.

Options: `router_bias`: the logits are `W_router h + b` (tensor `<router_bias>`); `shared_gate=False`: the shared expert
is added as it is, without a gate. With one group and `renormalize`, the weights are the softmax over the chosen logits
alone (softmax over all, divided by the chosen ones' sum, is the same number). The part takes a block's other term and
multiplier into its last kernel: `forward(ctx, h, add=a, scale=m)` returns `m * (a + ff(h))`.
"""
from __future__ import annotations
import math

import torch

from ..weights import ParamSpec
from .base import FeedForward, register_feed_forward
from .feed_forward import SwiGLU

_NAMES = {"router": "router", "expert": "experts.{}", "gate": "gate_proj", "up": "up_proj", "down": "down_proj",
          "shared": "shared_expert", "shared_gate": "shared_gate", "router_bias": "router.bias"}


@register_feed_forward("routed_moe")
class RoutedMoE(FeedForward):
    takes_sum = True      # forward(ctx, h, add=, scale=): see `ParallelSharedBlock`

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, groups: int = 1,
                 keep_groups: int = 1, shared_size: int = 0, renormalize: bool = False, names: dict | None = None,
                 router_bias: bool = False, shared_gate: bool = True):
        if not 0 < top <= num_experts:
            raise ValueError(f"top {top} must lie in 1..{num_experts}")
        if groups <= 0 or num_experts % groups or not 0 < keep_groups <= groups or top > keep_groups * (num_experts // groups):
            raise ValueError(f"{num_experts} experts in {groups} groups of which {keep_groups} are kept cannot give {top} choices")
        self.D, self.I, self.E, self.top = hidden_size, intermediate_size, num_experts, top
        self.groups, self.keep, self.renormalize = int(groups), int(keep_groups), bool(renormalize)
        self.names = {**_NAMES, **(names or {})}
        self.router_bias, self.shared_gate = bool(router_bias), bool(shared_gate) and shared_size > 0
        self.b_router = None
        self.shared = None
        if shared_size:
            n = self.names
            self.shared = SwiGLU(hidden_size, shared_size, names=(n["gate"], n["up"], n["down"]), suffix="")
        self.w_router = self.w_gate_up = self.w_down = None

    def children(self):
        return ((self.names["shared"], self.shared),) if self.shared is not None else ()

    def _expert(self, e: int, which: str) -> str:
        return f"{self.names['expert'].format(e)}.{self.names[which]}"

    def tensors(self) -> dict[str, ParamSpec]:
        n, out = self.names, {}
        for e in range(self.E):
            out[self._expert(e, "gate")] = ParamSpec((self.I, self.D))
            out[self._expert(e, "up")] = ParamSpec((self.I, self.D))
            out[self._expert(e, "down")] = ParamSpec((self.D, self.I))
        out[n["router"]] = ParamSpec((self.E, self.D))
        if self.router_bias:
            out[n["router_bias"]] = ParamSpec((self.E,), role="vector")
        if self.shared is not None:
            out.update({f"{n['shared']}.{k}": v for k, v in self.shared.tensors().items() if v.group is None})
            if self.shared_gate:
                out[f"{n['shared']}.{n['shared_gate']}"] = ParamSpec((1, self.D))
        return out

    def bind(self, tensors, ops) -> None:
        n, E = self.names, self.E
        self.w_gate_up = torch.stack([torch.cat([tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]], 0)
                                      for e in range(E)]).contiguous()                  # (E, 2 I, D)
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in range(E)]).contiguous()      # (E, D, I)
        router = tensors[n["router"]]
        if self.shared is not None:
            pre = n["shared"] + "."
            self.shared.bind({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)}, ops)
            if self.shared_gate:
                router = torch.cat([router, tensors[pre + n["shared_gate"]]], 0)        # one product: [router; shared gate]
        self.w_router = router.contiguous()
        if self.router_bias:
            b = tensors[n["router_bias"]].float()
            self.b_router = torch.cat([b, b.new_zeros(router.shape[0] - self.E)]).contiguous()

    def weight_tensors(self) -> list:
        return [self.w_router, self.w_gate_up, self.w_down]

    def forward(self, ctx, h: torch.Tensor, add: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        z = ws.get("router_logits", (n, self.w_router.shape[0]), torch.float32)
        ops.linear(h, self.w_router, self.b_router, z)
        weights = ws.get("router_weights", (n, self.top), torch.float32)
        route = ops.route_by_scores(z, self.E, self.top, self.groups, self.keep, self.renormalize, ctx.meta, weights,
                                    math.gcd(self.D, self.I))
        y = ws.get("moe_act", (n * self.top, self.I), ops.dtype)             # rows in the sorted order of the pairs
        ops.grouped_linear_glu(h, self.w_gate_up, route, y, 1.0, math.inf, 0.0)      # silu(gate) * up
        terms = ws.get("moe_terms", (n * self.top, self.D), torch.float32)   # row n * top + k: the k-th expert of row n
        ops.grouped_linear_scatter(y, self.w_down, route, terms)
        shared = self.shared.forward(ctx, h, tag="shared_") if self.shared is not None else None
        out = ws.get("moe_delta", (n, self.D), torch.float32)
        gate = z if self.shared_gate else None
        if add is None and scale == 1.0:
            ops.moe_combine(terms, weights, shared, gate, self.E, out)
        else:
            ops.moe_combine(terms, weights, shared, gate, self.E, out, add=add, scale=scale)
        return out
