"""Generalized delta rule: a recurrent mixer whose state decays per key channel and forgets along the token's unit key.

`r = W_r h`, `k = W_k h` (num_heads x key_dim), `v = W_v h` (num_heads x value_dim). Per head, with S (key_dim x
value_dim) and the unit key `u = k / sqrt(sum(k^2) + unit_eps)`:

    d = exp(-decay_rate * sigmoid(W_d2 tanh(W_d1 h) + d0))        a decay per head and key channel (rows of S)
    a = sigmoid(W_a h + a0)                                       a removal rate per head and key channel
    S <- diag(d) S - (a * u) (u^T S) + k v^T                      both products read the state before the token
    o  = S^T r                                                    the read-out sees the token's write

Each head's o is divided by its root mean square over value_dim (`eps` inside the root), the heads are concatenated and
multiplied by the weight `norm` (num_heads x value_dim) and by `sigmoid(W_g h)`, then the output product. S (float32,
zero at a request's start) is request state. One product with the rows [r; k; v; g; a; d1] leaves float32 and enters the
recurrence unrounded; the unit key, both rates with their sigmoids and the exponential, the recurrence and the output norm
are 32-bit in both dtypes; tanh(W_d1 h) is rounded once to the activation dtype as the operand of the second product.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import LayerCache, Mixer, register_mixer

_NAMES = {"r": "r_proj", "k": "k_proj", "v": "v_proj", "gate": "g_proj", "remove": "a_proj", "remove_bias": "a_bias",
          "decay_in": "d_down", "decay_out": "d_up", "decay_bias": "d_bias", "norm": "norm", "out": "o_proj"}


@register_mixer("general_delta")
class GeneralDelta(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay_rate: float = 1.0,
                 unit_eps: float = 1e-6, eps: float = 1e-6, names: dict | None = None, low_rank: int = 0):
        """low_rank: the inner size of the two-step decay projection for writers of random weights (0: a sixteenth of the
        hidden size, at least 8); a checkpoint's own size is read from its tensors."""
        self.D, self.H, self.dk, self.dv = hidden_size, num_heads, key_dim, value_dim
        self.decay_rate, self.unit_eps, self.eps = float(decay_rate), float(unit_eps), float(eps)
        self.names = {**_NAMES, **(names or {})}
        self.low_rank = int(low_rank) or max(8, hidden_size // 16)
        self.rank = 0
        self.w_in = self.w_decay = self.wo = self.decay_bias = self.remove_bias = self.norm_w = None

    def tensors(self) -> dict[str, ParamSpec]:
        n, H, dk, dv, D, r = self.names, self.H, self.dk, self.dv, self.D, self.low_rank
        return {n["r"]: ParamSpec((H * dk, D)), n["k"]: ParamSpec((H * dk, D)), n["v"]: ParamSpec((H * dv, D)),
                n["gate"]: ParamSpec((H * dv, D)), n["remove"]: ParamSpec((H * dk, D)),
                n["remove_bias"]: ParamSpec((H * dk,), role="vector"),
                n["decay_in"]: ParamSpec((-1, D), open=r), n["decay_out"]: ParamSpec((H * dk, -1), open=r),
                n["decay_bias"]: ParamSpec((H * dk,), role="vector"),
                n["norm"]: ParamSpec((H * dv,), role="vector", init="ones"), n["out"]: ParamSpec((D, H * dv))}

    def bind(self, tensors, ops) -> None:
        n, H, dk, dv = self.names, self.H, self.dk, self.dv
        d1, d2 = tensors[n["decay_in"]], tensors[n["decay_out"]]
        self.rank = d1.shape[0]
        if d2.shape[1] != self.rank:
            raise ValueError(f"the two steps of the decay projection do not fit: {tuple(d1.shape)} -> {tuple(d2.shape)}")
        # one product for everything that reads h: columns [r | k | v | gate | remove | decay step one]
        self.w_in = torch.cat([tensors[n[x]] for x in ("r", "k", "v", "gate", "remove")] + [d1], 0).contiguous()
        self.off_gate = 2 * H * dk + H * dv
        self.off_remove = self.off_gate + H * dv
        self.off_low = self.off_remove + H * dk
        self.w_decay = d2.contiguous()
        self.decay_bias = tensors[n["decay_bias"]].float().contiguous()
        self.remove_bias = tensors[n["remove_bias"]].float().contiguous()
        self.norm_w = tensors[n["norm"]].float().contiguous()
        self.wo = tensors[n["out"]]
        self.state_shape = ops.recurrent_state_shape(H, dk, dv)

    def state_need(self) -> dict:
        return {"S": self.state_shape}

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        H, dk, dv = self.H, self.dk, self.dv
        proj = ws.get("gdelta_proj", (n, self.off_low + self.rank), torch.float32)
        ops.linear(h, self.w_in, None, proj)
        low = ws.get("gdelta_low", (n, self.rank), ops.dtype)
        ops.activate(proj, self.off_low, "tanh", low)
        decay_in = ws.get("gdelta_decay", (n, H * dk), torch.float32)
        ops.linear(low, self.w_decay, None, decay_in)
        o = ws.get("gdelta_o", (n, H * dv), torch.float32)
        ops.general_delta_scan(proj, H, dk, dv, self.off_remove, decay_in, self.decay_bias, self.remove_bias,
                               self.decay_rate, self.unit_eps, cache.state["S"], ctx.meta, o)
        y = ws.get("gdelta_y", (n, H * dv), ops.dtype)
        ops.head_norm_gate(o, H, dv, self.norm_w, self.eps, proj, self.off_gate, "sigmoid", y)
        delta = ws.get("gdelta_delta", (n, self.D), torch.float32)
        ops.linear(y, self.wo, None, delta)
        return delta
