"""The kernel table: every device operation a part may ask for, with its exact meaning.

The product has one implementation, `CudaOps` (hand-written sm_100a kernels; it refuses tensors that are not on a
GPU and raises if its library cannot be built or loaded). The interface exists so that parts depend on meanings, not on
launch details, and so that a test can hand the same engine a plain PyTorch table to check the host-side logic without
a GPU.

Conventions. N: token rows of the step. T: the activation dtype (`ops.dtype`: float32 or bfloat16). The residual stream
and every sublayer output are float32. Rows whose `meta.seq_row` is negative are padding: kernels write zeros for them
and store nothing in the cache. All sums over a row, a head or a key range are in 32-bit and their order depends only
on the row's own data, never on the other rows of the step.
"""
from __future__ import annotations
from typing import Any

import torch


class Ops:
    dtype: torch.dtype

    def step_extra_ints(self, needs: tuple, max_rows: int, max_segments: int) -> int:
        """How many int32 of the step's metadata block this table wants for itself, given the kinds of step data the
        model's parts need (`Part.step_needs()`), for steps of at most max_rows rows of at most max_segments requests."""
        return 0

    def plan_step(self, meta: Any, needs: tuple) -> None:
        """Called once per step, after the metadata is packed on the host and before its copy to the device: the table
        may fill `meta.extra_host` (its int32 in the block) and keep launch sizes in `meta.plan`."""

    def step_signature(self, meta: Any) -> tuple:
        """What, beside the numbers of rows and wanted rows, fixes the kernel launches of the step just planned; two
        steps with equal signatures may replay one captured graph."""
        return ()

    def check_attention(self, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        """Raise ValueError if the attention kernels cannot take these sizes (nothing is ever computed wrongly)."""
        raise NotImplementedError

    def embed(self, table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, src: torch.Tensor | None = None,
              prev_ids: torch.Tensor | None = None, scale: float = 1.0) -> None:
        """x[n, :] = float32(table[tokens[n], :]) * scale. tokens: int32 (N,). A token outside the table is an error.
        With src (int32 (N,)) and prev_ids (int32): a row with src[n] >= 0 uses token prev_ids[src[n]] instead."""
        raise NotImplementedError

    def add_rmsnorm(self, x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                    h: torch.Tensor, rows: torch.Tensor | None = None, groups: int = 1) -> None:
        """rows None: x += delta (if given), in place; h[n] = T(weight * x[n] / sqrt(mean(x[n]^2) + eps)).
        rows (int32 (R,), -1 = none): h[r] is computed from x[rows[r]] + delta[rows[r]]; x is not written.
        groups > 1: the row is split into that many equal consecutive parts and the mean is taken over each part alone."""
        raise NotImplementedError

    def select_tokens(self, tokens: torch.Tensor, src: torch.Tensor, prev_ids: torch.Tensor, out: torch.Tensor) -> None:
        """out[n] = prev_ids[src[n]] if src[n] >= 0 else tokens[n] (all int32): the ids `embed` reads, as one tensor."""
        raise NotImplementedError

    def short_conv(self, h: torch.Tensor, w: torch.Tensor, state: torch.Tensor | None, meta: Any, out: torch.Tensor,
                   residual: bool = True, activation: str | None = None, bias: torch.Tensor | None = None) -> None:
        """Causal convolution over time within each portion of the step (meta.seg: first row, rows, first position,
        state slot). h, out: (N, C) T; w: (C, taps) T; state: (slots, taps - 1, C) float32, the last taps - 1 inputs of
        each request so far, oldest first. For the row at place i of its portion:
        out = (h if residual) + sum_j w[:, j] * in(i - taps + 1 + j), in(k) = h[first row + k] for k >= 0, else
        state[slot, taps - 1 + k]. The sum is float32, j rising, rounded once. Afterwards state[slot] holds the portion's
        request's last taps - 1 inputs. Padding rows give zeros. activation "silu": out = z * sigmoid(z) of
        the float32 sum z (residual included), rounded once. bias (C,) float32: added to the sum after the taps, before
        the residual and the activation."""
        raise NotImplementedError

    def gated_sum(self, a: torch.Tensor, gate_a: torch.Tensor | None, f: torch.Tensor | None, gate_f: torch.Tensor | None,
                  out: torch.Tensor, f_terms: int = 1, f_weight: float = 1.0) -> None:
        """out[n] = a[n] * sigmoid(gate_a[n]) + (f_weight * sum_k f[n * f_terms + k]) * sigmoid(gate_f[n]); all float32,
        (N, D), f (N * f_terms, D), the terms added in rising k. A gate that is None counts as 1, f None as no second
        term. sigmoid(z) = 1 / (1 + exp(-z))."""
        raise NotImplementedError

    def scale_(self, x: torch.Tensor, factor: float) -> None:
        """x *= factor, float32, in place."""
        raise NotImplementedError

    def check_latent_attention(self, num_heads: int, key_width: int, value_width: int) -> None:
        """Raise ValueError if `latent_attention` cannot take these sizes."""
        raise NotImplementedError

    def latent_cache_write(self, down: torch.Tensor, norm_weight: torch.Tensor, eps: float, cos: torch.Tensor,
                           sin: torch.Tensor, rotated: int, meta: Any, cache: Any, pairing: int = 0) -> None:
        """down: (N, L + R) float32, cache.keys: (pages, page_size, L + R) T. For every live row: the first L values
        are divided by their root mean square (eps inside the root) and multiplied by norm_weight (L,); of the last R,
        the first `rotated` are turned by the row's position (pairs i, i + rotated/2, tables (max_len, rotated/2)), the
        rest pass; the L + R values are rounded once and stored at the row's place in its request's pages. pairing 1:
        pairs 2i, 2i + 1 instead."""
        raise NotImplementedError

    def rotate_heads(self, q: torch.Tensor, offset: int, cos: torch.Tensor, sin: torch.Tensor, rotated: int, meta: Any,
                     out: torch.Tensor, out_offset: int, pairing: int = 0) -> None:
        """q: (N, H, W) T, out: (N, H, Wo) T. out[n, h, out_offset : out_offset + W - offset] = q[n, h, offset:] with its
        first `rotated` values turned by the row's position (as in `latent_cache_write`); float32 arithmetic."""
        raise NotImplementedError

    def linear_heads(self, a: torch.Tensor, a_offset: int, k: int, w: torch.Tensor, out: torch.Tensor,
                     out_offset: int) -> None:
        """One product per head: out[n, h, out_offset : out_offset + M] = w[h] . a[n, h, a_offset : a_offset + k];
        a: (N, H, Wa) T, w: (H, M, k) T, out: (N, H, Wo) T or float32; float32 accumulation over k in rising order."""
        raise NotImplementedError

    def latent_attention(self, q: torch.Tensor, cache: Any, meta: Any, out: torch.Tensor, value_width: int, scale: float,
                         window: int, sink: torch.Tensor | None = None) -> None:
        """q: (N, H, W) T; cache.keys: (pages, page_size, W) T, one vector e_j per cached token, shared by all heads.
        out[n, h] = sum_j softmax_j((q[n, h] . e_j) * scale) e_j[:value_width] over the keys j of the row's own request
        with max(0, p - window + 1) <= j <= p (window 0: 0 <= j <= p), p = meta.pos[n]; out: (N, H, value_width) T.
        sink (H,) float32: the softmax's denominator of head h also holds exp(sink[h]) (not scaled, no value)."""
        raise NotImplementedError

    def route_by_table(self, token_ids: torch.Tensor, meta: Any, table: torch.Tensor, num_experts: int, align: int = 1) -> Any:
        """table: (V, top) int32. Groups the step's (row, choice) pairs by expert table[token_ids[row], choice] (padding
        rows have none). Returns what `grouped_linear_glu` / `grouped_linear_scatter` need, valid until the next call.
        align: a common divisor of the sizes of the products that will use the route (a hint for the choice of tiles)."""
        raise NotImplementedError

    def grouped_linear_glu(self, h: torch.Tensor, w: torch.Tensor, route: Any, y: torch.Tensor, alpha: float,
                           limit: float, up_shift: float = 1.0) -> None:
        """w: (E, 2 I, K): expert e's gate rows, then its up rows. For every pair (row n, expert e) of the route:
        g = min(w[e, :I] . h[n], limit), u = clamp(w[e, I:] . h[n], -limit, limit), y[pair] = T(g * sigmoid(alpha * g) *
        (u + up_shift)); y: (N * top, I) T in the route's own order of pairs; products and activation in float32.
        (alpha 1, an infinite limit and up_shift 0 give silu(g) * u.)"""
        raise NotImplementedError

    def grouped_linear_scatter(self, y: torch.Tensor, w: torch.Tensor, route: Any, out: torch.Tensor) -> None:
        """w: (E, D, I). out[n * top + k] = w[e] . y[pair], float32 (N * top, D), for the pair of row n's k-th choice;
        rows of padding are zero."""
        raise NotImplementedError

    # ---- recurrent mixers, windowed attention with a sink, routed experts
    def recurrent_state_shape(self, heads: int, key_dim: int, value_dim: int) -> tuple:
        """The shape of one request's float32 state for `retention_scan` / `gated_delta_scan`: `heads` matrices of
        key_dim x value_dim in whatever layout and padding this table's kernels keep them (only they read it; a zeroed
        slot is the zero state)."""
        raise NotImplementedError

    def retention_scan(self, proj: torch.Tensor, heads: int, key_dim: int, value_dim: int, decay: torch.Tensor,
                       key_scale: float, cos: torch.Tensor | None, sin: torch.Tensor | None, rotated: int, pairing: int,
                       state: torch.Tensor, meta: Any, out: torch.Tensor) -> None:
        """proj: (N, >= H (2 dk + dv)) float32, a row = [q heads | k heads | v heads | ...]. For every portion of the step
        (meta.seg), token by token in order, per head h from the state of the portion's slot:
        S = decay[h] * S + k' v^T, out[n, h] = S^T q' with q' = rot(q), k' = rot(k) * key_scale, where rot turns the
        first `rotated` dimensions by the row's position (tables (max_len, rotated/2); pairing 0: i with i + rotated/2,
        1: 2i with 2i+1). out: (N, H dv) float32; everything float32. The slot's state is that after the portion's last
        token. Padding rows give zeros."""
        raise NotImplementedError

    def gated_delta_scan(self, qkv: torch.Tensor, heads: int, key_heads: int, key_dim: int, value_dim: int,
                         high: torch.Tensor, beta: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                         unit_eps: float, query_scale: float, state: torch.Tensor, meta: Any, out: torch.Tensor) -> None:
        """qkv: (N, 2 Hk dk + H dv) T = [q | k | v]; high: (N, >= H dk) float32 whose first H dk columns are the decay
        inputs a; beta: (N, H) float32 (before the sigmoid); a_log (H,), dt_bias (H dk,) float32. Per portion, token by
        token, per head h (key head h // (H / Hk)): q^ = q / sqrt(sum q^2 + unit_eps) * query_scale, k^ likewise without
        the scale, b = sigmoid(beta), g = exp(-exp(a_log[h]) * softplus(a[h] + dt_bias[h])) per key channel;
        S = g * S (rows), u = b * (v - S^T k^), S = S + k^ u^T, out[n, h] = S^T q^. float32 throughout; out (N, H dv)."""
        raise NotImplementedError

    def head_norm_gate(self, o: torch.Tensor, heads: int, value_dim: int, weight: torch.Tensor | None, eps: float,
                       gate: torch.Tensor | None, gate_offset: int, activation: str | None, out: torch.Tensor) -> None:
        """o: (N, H dv) float32. out[n, h, c] = T(o / sqrt(mean_c(o[n, h]^2) + eps) * weight[c] * act(gate[n, gate_offset +
        h dv + c])); weight (dv,) float32, shared by the heads, or (H dv,), one per head and channel (weight[h dv + c]),
        or None (1); gate float32 (N, any width) or None (1); act "silu", "sigmoid"."""
        raise NotImplementedError

    def general_delta_scan(self, proj: torch.Tensor, heads: int, key_dim: int, value_dim: int, remove_offset: int,
                           decay_in: torch.Tensor, decay_bias: torch.Tensor, remove_bias: torch.Tensor, decay_rate: float,
                           unit_eps: float, state: torch.Tensor, meta: Any, out: torch.Tensor) -> None:
        """proj: (N, ld) float32, a row = [r (H dk) | k (H dk) | v (H dv) | ...] with the removal inputs (H dk) from
        column remove_offset on; decay_in (N, H dk) float32; decay_bias, remove_bias (H dk,) float32. Per portion, token
        by token, per head: u = k / sqrt(sum k^2 + unit_eps), d = exp(-decay_rate * sigmoid(decay_in + decay_bias)),
        a = sigmoid(remove + remove_bias) per key channel; with b = S^T u of the state before the token,
        S = diag(d) S - (a * u) b^T + k v^T, out[n, h] = S^T r. float32 throughout; out (N, H dv); the state
        (`recurrent_state_shape`) is that after the portion's last token. Rows of padding are left as they are."""
        raise NotImplementedError

    def activate(self, src: torch.Tensor, offset: int, kind: str, out: torch.Tensor) -> None:
        """out[n, j] = T(act(src[n, offset + j])) for the columns of out; src float32 (N, any width); kind "tanh",
        "sigmoid", "silu", "gelu_tanh", "identity", computed in float32 and rounded once. Padding rows need not be zero."""
        raise NotImplementedError

    def gate_multiply(self, x: torch.Tensor, gate: torch.Tensor, gate_offset: int, kind: str, out: torch.Tensor) -> None:
        """out[n, j] = T(x[n, j] * act(gate[n, gate_offset + j])); x, out (N, W) T (out may be x), gate float32 (N, any
        width), act as in `activate`; the activation and the product in float32, rounded once."""
        raise NotImplementedError

    def blend_columns(self, dst: torch.Tensor, dst_offset: int, src: torch.Tensor, src_offset: int, width: int,
                      weight: torch.Tensor) -> None:
        """dst[n, dst_offset + j] = (1 - w) * dst[n, dst_offset + j] + w * src[n, src_offset + j] for j < width, in place;
        dst, src float32 (N, any width), w = weight[0] (float32, on the device). float32: the two products rounded, then
        their sum."""
        raise NotImplementedError

    def rglru_scan(self, u: torch.Tensor, gates: torch.Tensor, gate_bias: torch.Tensor, lam: torch.Tensor, y: torch.Tensor,
                   sharpness: float, state: torch.Tensor, meta: Any, out: torch.Tensor) -> None:
        """u, y, out: (N, W) T; gates: (N, B, 2 W/B) float32, part b = [recurrence gate | input gate] before bias and
        sigmoid; gate_bias (B, 2 W/B), lam (W,) float32; state (slots, W) float32. Per portion (meta.seg), token by token,
        per channel c of part b: r = sigmoid(gates[n, b, j] + bias), i = sigmoid(gates[n, b, W/B + j] + bias), a =
        exp(-sharpness * r * softplus(lam[c])), S = a * S + sqrt(1 - a^2) * (i * u[n, c]) from the slot's state,
        out[n, c] = T(S * y[n, c]). float32 throughout; the slot's state is that after the portion's last token.
        Padding rows give zeros. softplus(z) = max(z, 0) + log1p(exp(-|z|))."""
        raise NotImplementedError

    def hashed_pair_embed(self, table: torch.Tensor, token_ids: torch.Tensor, meta: Any, state: torch.Tensor,
                          buckets: int, mul_prev: int, mul_cur: int, x: torch.Tensor) -> None:
        """table: (buckets + 1, D) T; token_ids int32 (N,); state int32 (slots, 1); x (N, D) float32. For the row at
        place i of its portion (meta.seg), at position p: x += float32(table[r]) with r = buckets if p = 0, else
        (u * mul_prev + t * mul_cur) mod buckets in 64-bit integers, t the row's token and u the token of the row before
        (i > 0) or state[slot] (i = 0). Afterwards state[slot] holds the portion's last token. Padding rows are left."""
        raise NotImplementedError

    def depth_average(self, streams: torch.Tensor, depth: int, coef: torch.Tensor | None, x: torch.Tensor,
                      delta: torch.Tensor | None) -> None:
        """streams: (N, L + 1, D) float32; x, delta (N, D) float32 (delta None: zero). streams[:, depth + 1] = x + delta;
        then x = sum_j coef[j] * streams[:, j] over j = 0 .. depth + 1 in rising j (coef float32, depth + 2 numbers),
        by fused multiply-adds from zero, in float32. depth -1 with coef None: streams[:, 0] = x + delta and x = x + delta."""
        raise NotImplementedError

    def depth_average_rmsnorm(self, streams: torch.Tensor, depth: int, coef: torch.Tensor, x: torch.Tensor,
                              delta: torch.Tensor | None, weight: torch.Tensor, eps: float, h: torch.Tensor,
                              rows: torch.Tensor | None = None) -> bool:
        """`depth_average` followed by `add_rmsnorm(x, None, weight, eps, h, rows)` as one operation. rows None: streams and
        x are written as `depth_average` writes them and h[n] is the norm of the averaged row. rows (int32 (R,), -1 =
        none): only h[r], from row rows[r], is written. Optional: returns False, having done nothing, if this table has
        no such kernel for these sizes; the caller then runs the two operations."""
        return False

    def check_sink_attention(self, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int) -> None:
        """Raise ValueError if `sink_attention` cannot take these sizes."""
        raise NotImplementedError

    def rotate_kv_write(self, qkv: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None, rotated: int,
                        pairing: int, meta: Any, cache: Any, q_out: torch.Tensor, num_heads: int, num_kv_heads: int,
                        key_dim: int, value_dim: int, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                        norm_eps: float = 0.0, query_temperature: tuple | None = None) -> None:
        """qkv: (N, >= Hq dk + Hkv dk + Hkv dv) float32 = [q | k | v | anything] (with cache.write False only the q
        columns are read and the row may be as short as Hq dk). The first `rotated` dimensions of every q and k head
        are turned by the row's position (pairing as in `retention_scan`), the rest pass; q goes to q_out (N, Hq dk) T,
        k and v, rounded once, to the row's place in its request's pages (cache.keys (pages, Hkv, page, dk),
        cache.values (pages, Hkv, page, dv), any strides with a unit last one). q_norm / k_norm (dk,) float32: before the
        rotation every q / k head becomes x / sqrt(mean(x^2) + norm_eps) * weight. query_temperature (coef, every): after
        the rotation q at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1). All in float32."""
        raise NotImplementedError

    def sink_attention(self, q: torch.Tensor, cache: Any, meta: Any, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                       key_dim: int, value_dim: int, scale: float, window: int, keep_first: int,
                       sink: torch.Tensor | None, softcap: float = 0.0, gate: tuple | None = None, span: int = 0) -> None:
        """out[n, h] = sum_j e_j v_j / (sum_j e_j + exp(sink[h] - m)), e_j = exp(s_j - m), s_j = (q[n, h] . k_j) * scale,
        over the keys j <= p of the row's own request with p - j < window or j < keep_first (window 0: all), p =
        meta.pos[n], m the largest of the scores and sink[h]; sink None: no such term. kv head h // (Hq / Hkv).
        out: (N, Hq dv) T. softcap c > 0: s_j = c * tanh((q . k_j) * scale / c). gate (g, offset), g float32 (N, any
        width): out[n, h] is multiplied by sigmoid(g[n, offset + h]) before it is rounded. span s > 0: key j is seen
        only if also floor(j / s) = floor(p / s) (keep_first must then be 0)."""
        raise NotImplementedError

    def weighted_sum(self, terms: list, weights: list, out: torch.Tensor) -> None:
        """out = sum_i weights[i] * terms[i], float32 (N, D), each product rounded, added in the order given."""
        raise NotImplementedError

    def route_by_scores(self, logits: torch.Tensor, num_experts: int, top: int, groups: int, keep_groups: int,
                        renormalize: bool, meta: Any, weights: torch.Tensor, align: int = 1) -> Any:
        """logits: (N, >= E) float32, the first E columns are router logits. s = softmax over them; the experts form
        `groups` equal groups of neighbours, a group's score is its largest s, only experts of the keep_groups best groups
        (lower index first among equals) can be chosen; of those the `top` with the largest s (lower index first among
        equals), in falling order. weights[n, k] = s of the k-th choice (divided by their sum if renormalize); float32.
        Returns the route of the (row, choice) pairs sorted by expert, as `route_by_table` does."""
        raise NotImplementedError

    def moe_combine(self, terms: torch.Tensor, weights: torch.Tensor, shared: torch.Tensor | None,
                    gate_logits: torch.Tensor | None, gate_column: int, out: torch.Tensor,
                    add: torch.Tensor | None = None, scale: float = 1.0) -> None:
        """out[n] = sum_k weights[n, k] * terms[n * top + k] (+ sigmoid(gate_logits[n, gate_column]) * shared[n]); all
        float32; terms (N top, D), weights (N, top), shared (N, D), the sum in rising k and the shared term last
        (gate_logits None: the shared term is added as it is). add (N, D) float32 and scale: out = scale * (add + the
        sum). Padding rows give zeros."""
        raise NotImplementedError

    def linear(self, a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> None:
        """out[m, n] = sum_k a[m, k] * w[n, k] (+ bias[n]); a: (M, K) T, w: (N, K) T, bias float32, out float32 or T;
        accumulation in float32, one rounding into out."""
        raise NotImplementedError

    def pack_gate_up(self, gate: torch.Tensor, up: torch.Tensor, gate_bias: torch.Tensor | None = None,
                     up_bias: torch.Tensor | None = None):
        """Prepares the gate and up matrices ((I, K) each) for `linear_swiglu` in whatever layout the kernels want, or
        returns None if this table has no fused kernel for these sizes (the part then runs `linear` + `swiglu`)."""
        return None

    def linear_swiglu(self, a: torch.Tensor, packed: Any, out: torch.Tensor, activation: str = "silu") -> None:
        """out[m, i] = T(act(a[m] . gate[i] + gate_bias[i]) * (a[m] . up[i] + up_bias[i])); `packed` from `pack_gate_up`;
        act as in `swiglu`.
        The products are accumulated in float32 and are not rounded before the activation."""
        raise NotImplementedError

    def rope_kv_write(self, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, meta: Any, cache: Any,
                      q_out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        """qkv: (N, (Hq + 2 Hkv) * hd) float32, heads [q | k | v]. Rotates q and k heads by the row's position
        (pairs j, j + hd/2, angles from the float32 tables cos/sin (max_len, hd/2)); writes q to q_out (N, Hq*hd) T
        and, if cache.write, k and v to the row's page slot of cache.keys / cache.values."""
        raise NotImplementedError

    def linear_rope_kv_write(self, a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, cos: torch.Tensor,
                             sin: torch.Tensor, meta: Any, cache: Any, q_out: torch.Tensor, num_heads: int,
                             num_kv_heads: int, head_dim: int) -> bool:
        """`linear` (a . w^T + bias, w rows = [q heads | k heads | v heads]) followed by `rope_kv_write` on its float32
        result, as one operation that never writes that result out. Returns False, having done nothing, if this table
        has no such kernel for these sizes; the caller then runs the two operations."""
        return False

    def paged_attention(self, q: torch.Tensor, cache: Any, meta: Any, out: torch.Tensor, num_heads: int,
                        num_kv_heads: int, head_dim: int, scale: float, window: int) -> None:
        """out[n, h] = softmax_j((q[n, h] . K[j]) * scale) V[j] over the keys j of the row's own request with
        max(0, p - window + 1) <= j <= p (window 0: 0 <= j <= p), p = meta.pos[n]; kv head h // (Hq / Hkv)."""
        raise NotImplementedError

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
        """gate_up: (N, 2 I) T = [gate | up]; out[n, i] = T(act(gate[n, i]) * up[n, i]), act in float32: "silu", or
        "gelu_tanh": 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))."""
        raise NotImplementedError

    def linear_argmax(self, a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> bool:
        """out[m] = argmax_n (a[m] . w[n] + bias[n]) (the order of `argmax` below) without writing the products out.
        Optional: returns False, having done nothing, if this table has no such kernel for these sizes."""
        return False

    def argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        """out[r] = first index of the row's maximum (a NaN counts as the maximum, the first one wins); int32."""
        raise NotImplementedError

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
        """out[r] = the token at which the running sum of softmax(logits[r] / temperature[r]) (float64, in index
        order) first exceeds uniform[r] * total; temperature[r] <= 0 means argmax. uniform: float64 in [0, 1)."""
        raise NotImplementedError

    def sample_filtered(self, logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                        uniform: torch.Tensor, out: torch.Tensor) -> None:
        """`sample` after the reference's filters on logits[r] / temperature[r] (fusezap/serve/sampling.py:25-45):
        top_k[r] (int32; <= 0 or >= V: off, 1: argmax) keeps what is not below the k-th largest value, ties included;
        top_p[r] (float32; >= 1: off) then keeps, in falling order of value and rising index among equals, every token
        before which less than top_p[r] of the probability lies."""
        raise NotImplementedError
