"""A plain PyTorch kernel table with the meanings of `fusezap_core_b200.kernels.interface.Ops`.

Two uses: (1) the plain reference of every CUDA kernel in the `-m gpu` kernel tests (called with CPU copies of the
same inputs); (2) the `-m "not gpu"` tests hand it to the engine in place of the CUDA table, so the host-side logic
(step metadata, block tables, page reuse, the scheduler) is exercised on the CPU. It is never on the product path.
"""
from __future__ import annotations
import numpy as np
import torch

import plain_model


class PlainOps:
    def __init__(self, dtype: torch.dtype = torch.float32):
        self.dtype = dtype
        self.launches = 0

    def check_attention(self, num_heads, num_kv_heads, head_dim) -> None:
        if num_heads % num_kv_heads or head_dim % 2:
            raise ValueError("bad attention sizes")

    def embed(self, table, tokens, x, src=None, prev_ids=None, scale=1.0) -> None:
        t = tokens.long()
        if src is not None:
            t = torch.where(src >= 0, prev_ids.long()[src.long().clamp(min=0)], t)
        if ((t < 0) | (t >= table.shape[0])).any():
            raise ValueError("token id outside the embedding table")
        x.copy_(table[t].float() * torch.tensor(scale, dtype=torch.float32))

    def add_rmsnorm(self, x, delta, weight, eps, h, rows=None) -> None:
        if rows is None:
            if delta is not None:
                x.add_(delta)
            src = x
        else:
            r = rows.long().clamp(min=0)
            src = x[r] + (delta[r] if delta is not None else 0)
        y = src * torch.rsqrt((src * src).mean(-1, keepdim=True) + eps)
        y = weight.float() * y
        if rows is not None:
            y = torch.where((rows < 0)[:, None], torch.zeros_like(y), y)
        h.copy_(y.to(h.dtype))

    def linear(self, a, w, bias, out) -> None:
        y = a.float() @ w.float().T
        if bias is not None:
            y = y + bias.float()
        out.copy_(y.to(out.dtype))

    def rope_kv_write(self, qkv, cos, sin, meta, cache, q_out, num_heads, num_kv_heads, head_dim) -> None:
        n, Hq, Hkv, hd = qkv.shape[0], num_heads, num_kv_heads, head_dim
        pos, row = meta.pos.long(), meta.seq_row.long()
        x = qkv.view(n, Hq + 2 * Hkv, hd)
        c, s = cos[pos][:, None, :], sin[pos][:, None, :]
        qk = x[:, :Hq + Hkv]
        x1, x2 = qk[..., :hd // 2], qk[..., hd // 2:]
        rot = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
        live = row >= 0
        q = torch.where(live[:, None, None], rot[:, :Hq], torch.zeros(()))
        q_out.copy_(q.reshape(n, Hq * hd).to(q_out.dtype))
        if not cache.write:
            return
        table = meta.table(cache.group)
        bs = cache.page_size
        for i in range(n):
            if row[i] < 0:
                continue
            page = int(table[row[i], pos[i] // bs])
            assert page >= 0, f"row {i} at position {int(pos[i])} has no page"
            cache.keys[page, :, pos[i] % bs, :] = rot[i, Hq:].to(cache.keys.dtype)
            cache.values[page, :, pos[i] % bs, :] = x[i, Hq + Hkv:].to(cache.values.dtype)

    def paged_attention(self, q, cache, meta, out, num_heads, num_kv_heads, head_dim, scale, window) -> None:
        n, Hq, Hkv, hd = q.shape[0], num_heads, num_kv_heads, head_dim
        G = Hq // Hkv
        pos, row = meta.pos.long(), meta.seq_row.long()
        table = meta.table(cache.group)
        bs = cache.page_size
        o = torch.zeros(n, Hq, hd)
        for i in range(n):
            if row[i] < 0:
                continue
            p = int(pos[i])
            lo = max(0, p - window + 1) if window else 0
            js = torch.arange(lo, p + 1)
            pages = table[row[i], js // bs].long()
            assert (pages >= 0).all(), f"row {i}: a visible key's page was given back"
            K = cache.keys[pages, :, js % bs, :].float()       # (keys, Hkv, hd)
            V = cache.values[pages, :, js % bs, :].float()
            qi = q[i].float().view(Hq, hd)
            for h in range(Hq):
                s = (K[:, h // G, :] @ qi[h]) * scale
                o[i, h] = torch.softmax(s, 0) @ V[:, h // G, :]
        out.copy_(o.reshape(n, Hq * hd).to(out.dtype))

    def pack_gate_up(self, gate, up, gate_bias=None, up_bias=None):
        return None

    def swiglu(self, gate_up, out) -> None:
        I = out.shape[1]
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def argmax(self, logits, out) -> None:
        a = logits.detach().cpu().numpy()
        out.copy_(torch.from_numpy(np.argmax(a, axis=-1).astype(np.int32)))

    def sample(self, logits, temperature, uniform, out) -> None:
        a = logits.detach().cpu().numpy()
        res = np.zeros(a.shape[0], np.int32)
        for r in range(a.shape[0]):
            t = float(temperature[r])
            if t <= 0:
                res[r] = int(np.argmax(a[r]))
                continue
            x = a[r].astype(np.float64) / t
            e = np.exp(x - x.max())
            c = np.cumsum(e)
            res[r] = int(np.searchsorted(c, float(uniform[r]) * c[-1], side="right").clip(0, len(c) - 1))
        out.copy_(torch.from_numpy(res))

    def sample_filtered(self, logits, temperature, top_k, top_p, uniform, out) -> None:
        a = logits.detach().cpu().numpy()
        res = np.zeros(a.shape[0], np.int32)
        for r in range(a.shape[0]):
            t, k, p = float(temperature[r]), int(top_k[r]), float(top_p[r])
            if t <= 0 or k == 1:
                res[r] = int(np.argmax(a[r]))
                continue
            x = plain_model.top_p_filter(plain_model.top_k_filter(a[r].astype(np.float64) / t, k), p)
            c = np.cumsum(np.exp(x - x.max()))
            res[r] = int(np.searchsorted(c, float(uniform[r]) * c[-1], side="right").clip(0, len(c) - 1))
        out.copy_(torch.from_numpy(res))

    def errors_to_host(self) -> None:
        pass

    def check_errors(self, copied: bool = False) -> None:
        pass


class PlainOpsWide(PlainOps):
    """The plain table with the operations of the gated parallel block, the latent attention and the table-routed
    experts, written from their meanings in `kernels/interface.py`."""

    def add_rmsnorm(self, x, delta, weight, eps, h, rows=None, groups=1) -> None:
        if groups == 1:
            return super().add_rmsnorm(x, delta, weight, eps, h, rows)
        if rows is None:
            if delta is not None:
                x.add_(delta)
            src = x
        else:
            r = rows.long().clamp(min=0)
            src = x[r] + (delta[r] if delta is not None else 0)
        parts = src.view(src.shape[0], groups, -1)
        y = (parts * torch.rsqrt((parts * parts).mean(-1, keepdim=True) + eps)).reshape(src.shape) * weight.float()
        if rows is not None:
            y = torch.where((rows < 0)[:, None], torch.zeros_like(y), y)
        h.copy_(y.to(h.dtype))

    def select_tokens(self, tokens, src, prev_ids, out) -> None:
        out.copy_(torch.where(src >= 0, prev_ids[src.long().clamp(min=0)], tokens))

    def short_conv(self, h, w, state, meta, out, residual=True, activation=None) -> None:
        taps = w.shape[1]
        out.zero_()
        wf = w.float()
        for sg in meta.segments:
            rows = h[sg.row0: sg.row0 + sg.n].float()
            before = state[sg.state_slot] if taps > 1 else rows[:0]
            line = torch.cat([before, rows], 0)                      # inputs taps-1 back from the portion's start
            acc = rows.clone() if residual else torch.zeros_like(rows)
            y = torch.zeros_like(rows)
            for j in range(taps):
                y = y + wf[:, j] * line[j: j + sg.n]
            z = acc + y
            if activation == "silu":
                z = z * torch.sigmoid(z)
            out[sg.row0: sg.row0 + sg.n] = z.to(out.dtype)
            if taps > 1:
                state[sg.state_slot] = line[line.shape[0] - (taps - 1):]

    def gated_sum(self, a, gate_a, f, gate_f, out, f_terms=1, f_weight=1.0) -> None:
        sig = lambda z: 1.0 / (1.0 + torch.exp(-z))
        y = a * sig(gate_a) if gate_a is not None else a.clone()
        if f is not None:
            t = f.view(a.shape[0], f_terms, -1).sum(1) * torch.tensor(f_weight, dtype=torch.float32)
            y = y + (t * sig(gate_f) if gate_f is not None else t)
        out.copy_(y)

    def scale_(self, x, factor) -> None:
        x.mul_(factor)

    def check_latent_attention(self, num_heads, key_width, value_width) -> None:
        if value_width > key_width:
            raise ValueError("the value part cannot be wider than the cached vector")

    def _turn(self, v, cos, sin, rotated, pos):
        half = rotated // 2
        c, s = cos[pos], sin[pos]
        while c.dim() < v.dim():
            c, s = c.unsqueeze(1), s.unsqueeze(1)
        a, b = v[..., :half], v[..., half:rotated]
        return torch.cat([a * c - b * s, b * c + a * s, v[..., rotated:]], -1)

    def latent_cache_write(self, down, norm_weight, eps, cos, sin, rotated, meta, cache) -> None:
        L = norm_weight.shape[0]
        pos, row = meta.pos.long(), meta.seq_row.long()
        c = down[:, :L]
        c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * norm_weight.float()
        e = torch.cat([c, self._turn(down[:, L:], cos, sin, rotated, pos)], -1).to(cache.keys.dtype)
        table, bs = meta.table(cache.group), cache.page_size
        for i in range(down.shape[0]):
            if row[i] < 0:
                continue
            page = int(table[row[i], pos[i] // bs])
            assert page >= 0, f"row {i} at position {int(pos[i])} has no page"
            cache.keys[page, pos[i] % bs] = e[i]

    def rotate_heads(self, q, offset, cos, sin, rotated, meta, out, out_offset) -> None:
        v = self._turn(q[..., offset:].float(), cos, sin, rotated, meta.pos.long())
        v = torch.where((meta.seq_row >= 0)[:, None, None], v, torch.zeros(()))
        out[..., out_offset: out_offset + v.shape[-1]] = v.to(out.dtype)

    def linear_heads(self, a, a_offset, k, w, out, out_offset) -> None:
        y = torch.einsum("nhk,hmk->nhm", a[..., a_offset: a_offset + k].float(), w.float())
        out[..., out_offset: out_offset + w.shape[1]] = y.to(out.dtype)

    def latent_attention(self, q, cache, meta, out, value_width, scale, window) -> None:
        pos, row = meta.pos.long(), meta.seq_row.long()
        table, bs = meta.table(cache.group), cache.page_size
        out.zero_()
        for i in range(q.shape[0]):
            if row[i] < 0:
                continue
            p = int(pos[i])
            js = torch.arange(max(0, p - window + 1) if window else 0, p + 1)
            pages = table[row[i], js // bs].long()
            assert (pages >= 0).all(), f"row {i}: a visible key's page was given back"
            e = cache.keys[pages, js % bs].float()                 # (keys, W)
            w = torch.softmax((q[i].float() @ e.T) * scale, -1)    # (H, keys)
            out[i] = (w @ e[:, :value_width]).to(out.dtype)

    def route_by_table(self, token_ids, meta, table, num_experts, align=1):
        ex = table[token_ids.long().clamp(0, table.shape[0] - 1)].long()
        assert ((ex >= 0) & (ex < num_experts)).all()
        return ex, meta.seq_row >= 0

    def grouped_linear_glu(self, h, w, route, y, alpha, limit, up_shift=1.0) -> None:
        ex, live = route
        I = w.shape[1] // 2
        wf = w.float()[ex]                                           # (N, top, 2I, K)
        gu = torch.einsum("ntik,nk->nti", wf, h.float())
        g, u = gu[..., :I].clamp(max=limit), gu[..., I:].clamp(-limit, limit)
        act = g * (1.0 / (1.0 + torch.exp(-alpha * g))) * (u + up_shift)
        y.copy_(torch.where(live[:, None, None], act, torch.zeros(())).reshape(y.shape).to(y.dtype))

    def grouped_linear_scatter(self, y, w, route, out) -> None:
        ex, live = route
        t = torch.einsum("ntdi,nti->ntd", w.float()[ex], y.view(ex.shape[0], ex.shape[1], -1).float())
        out.copy_(torch.where(live[:, None, None], t, torch.zeros(())).reshape(out.shape))


class PlainOpsSeq(PlainOpsWide):
    """The operations of the recurrent mixers, the windowed attention with a sink and the routed experts."""

    def recurrent_state_shape(self, heads, key_dim, value_dim):
        return (heads, key_dim, value_dim)

    def _rot(self, x, cos, sin, rotated, pairing, pos):
        """x: (N, heads, d) float; the first `rotated` dimensions turned by pos."""
        if not rotated:
            return x
        c, s = cos[pos][:, None, :].to(x.dtype), sin[pos][:, None, :].to(x.dtype)
        out = x.clone()
        if pairing == 1:
            u, v = x[..., 0:rotated:2], x[..., 1:rotated:2]
            out[..., 0:rotated:2], out[..., 1:rotated:2] = u * c - v * s, v * c + u * s
        else:
            half = rotated // 2
            u, v = x[..., :half], x[..., half:rotated]
            out[..., :half], out[..., half:rotated] = u * c - v * s, v * c + u * s
        return out

    def retention_scan(self, proj, heads, key_dim, value_dim, decay, key_scale, cos, sin, rotated, pairing, state, meta, out):
        H, dk, dv = heads, key_dim, value_dim
        out.zero_()
        pos = meta.pos.long()
        for sg in meta.segments:
            r = slice(sg.row0, sg.row0 + sg.n)
            x = proj[r].double()
            q = self._rot(x[:, :H * dk].reshape(-1, H, dk), cos, sin, rotated, pairing, pos[r])
            k = self._rot(x[:, H * dk: 2 * H * dk].reshape(-1, H, dk), cos, sin, rotated, pairing, pos[r]) * key_scale
            v = x[:, 2 * H * dk: 2 * H * dk + H * dv].reshape(-1, H, dv)
            S = state[sg.state_slot].double()
            for t in range(sg.n):
                S = decay.double()[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
                out[sg.row0 + t] = torch.einsum("hkv,hk->hv", S, q[t]).reshape(-1).float()
            state[sg.state_slot] = S.float()

    def gated_delta_scan(self, qkv, heads, key_heads, key_dim, value_dim, high, beta, a_log, dt_bias, unit_eps, query_scale,
                         state, meta, out):
        H, Hk, dk, dv = heads, key_heads, key_dim, value_dim
        out.zero_()
        rep = H // Hk
        for sg in meta.segments:
            r = slice(sg.row0, sg.row0 + sg.n)
            x = qkv[r].double()
            q = x[:, :Hk * dk].reshape(-1, Hk, dk)
            k = x[:, Hk * dk: 2 * Hk * dk].reshape(-1, Hk, dk)
            v = x[:, 2 * Hk * dk:].reshape(-1, H, dv)
            q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * query_scale).repeat_interleave(rep, 1)
            k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)).repeat_interleave(rep, 1)
            b = torch.sigmoid(beta[r].double())
            a = high[r, :H * dk].double() + dt_bias.double()
            g = torch.exp(-torch.exp(a_log.double())[None, :, None] * torch.nn.functional.softplus(a).reshape(-1, H, dk))
            S = state[sg.state_slot].double()
            for t in range(sg.n):
                S = g[t][:, :, None] * S
                u = b[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
                S = S + k[t][:, :, None] * u[:, None, :]
                out[sg.row0 + t] = torch.einsum("hkv,hk->hv", S, q[t]).reshape(-1).float()
            state[sg.state_slot] = S.float()

    def head_norm_gate(self, o, heads, value_dim, weight, eps, gate, gate_offset, activation, out):
        n = o.shape[0]
        x = o.view(n, heads, value_dim)
        y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
        if weight is not None:
            y = y * weight.float()
        if gate is not None:
            z = gate[:, gate_offset: gate_offset + heads * value_dim].reshape(n, heads, value_dim)
            y = y * (torch.sigmoid(z) if activation == "sigmoid" else z * torch.sigmoid(z))
        out.copy_(y.reshape(n, -1).to(out.dtype))

    def check_sink_attention(self, num_heads, num_kv_heads, key_dim, value_dim) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("bad attention sizes")

    def rotate_kv_write(self, qkv, cos, sin, rotated, pairing, meta, cache, q_out, num_heads, num_kv_heads, key_dim, value_dim):
        n, Hq, Hkv, dk, dv = qkv.shape[0], num_heads, num_kv_heads, key_dim, value_dim
        pos, row = meta.pos.long(), meta.seq_row.long()
        q = self._rot(qkv[:, :Hq * dk].reshape(n, Hq, dk), cos, sin, rotated, pairing, pos)
        k = self._rot(qkv[:, Hq * dk: (Hq + Hkv) * dk].reshape(n, Hkv, dk), cos, sin, rotated, pairing, pos)
        v = qkv[:, (Hq + Hkv) * dk:].reshape(n, Hkv, dv)
        live = row >= 0
        q_out.copy_(torch.where(live[:, None, None], q, torch.zeros(())).reshape(n, -1).to(q_out.dtype))
        table, bs = meta.table(cache.group), cache.page_size
        for i in range(n):
            if not live[i] or not cache.write:
                continue
            page = int(table[row[i], pos[i] // bs])
            assert page >= 0, "a position has no page"
            cache.keys[page, :, pos[i] % bs] = k[i].to(cache.keys.dtype)
            cache.values[page, :, pos[i] % bs] = v[i].to(cache.values.dtype)

    def sink_attention(self, q, cache, meta, out, num_heads, num_kv_heads, key_dim, value_dim, scale, window, keep_first, sink):
        n, Hq, Hkv, dk, dv = q.shape[0], num_heads, num_kv_heads, key_dim, value_dim
        pos, row = meta.pos.long(), meta.seq_row.long()
        table, bs = meta.table(cache.group), cache.page_size
        out.zero_()
        for i in range(n):
            if row[i] < 0:
                continue
            p = int(pos[i])
            js = [j for j in range(p + 1) if not window or p - j < window or j < keep_first]
            pages = [int(table[row[i], j // bs]) for j in js]
            assert min(pages) >= 0, "a visible key has no page"
            K = torch.stack([cache.keys[pg, :, j % bs] for pg, j in zip(pages, js)]).float()      # (J, Hkv, dk)
            V = torch.stack([cache.values[pg, :, j % bs] for pg, j in zip(pages, js)]).float()
            qi = q[i].float().view(Hkv, Hq // Hkv, dk)
            s = torch.einsum("gak,jgk->gaj", qi, K) * scale
            if sink is not None:
                s = torch.cat([s, sink.float().view(Hkv, Hq // Hkv, 1)], -1)
            w = torch.softmax(s, -1)[..., :len(js)]
            out[i] = torch.einsum("gaj,jgv->gav", w, V).reshape(-1).to(out.dtype)

    def weighted_sum(self, terms, weights, out) -> None:
        acc = torch.zeros_like(out)
        for t, w in zip(terms, weights):
            acc = acc + torch.tensor(w, dtype=torch.float32) * t
        out.copy_(acc)

    def route_by_scores(self, logits, num_experts, top, groups, keep_groups, renormalize, meta, weights, align=1):
        E = num_experts
        s = torch.softmax(logits[:, :E].float(), -1)
        per = E // groups
        gs = s.view(-1, groups, per).max(-1).values
        best = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :keep_groups]
        allowed = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, 1)
        masked = torch.where(allowed, s, torch.full_like(s, -1.0))
        order = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :top]
        w = torch.gather(s, 1, order)
        if renormalize:
            w = w / w.sum(-1, keepdim=True)
        weights.copy_(w)
        return order, meta.seq_row >= 0

    def moe_combine(self, terms, weights, shared, gate_logits, gate_column, out) -> None:
        n, top = weights.shape
        acc = (terms.view(n, top, -1) * weights[:, :, None]).sum(1)
        if shared is not None:
            acc = acc + torch.sigmoid(gate_logits[:, gate_column: gate_column + 1]) * shared
        out.copy_(acc)


class PlainOpsDeep(PlainOpsSeq):
    """The operations of depth-averaged layers, the hashed pair embedding, the generalized delta rule and the attention
    with head gates, capped scores, normed queries and keys and a query temperature."""

    @staticmethod
    def _act(z, kind):
        if kind == "tanh":
            return torch.tanh(z)
        if kind == "sigmoid":
            return torch.sigmoid(z)
        if kind == "silu":
            return z * torch.sigmoid(z)
        if kind == "gelu_tanh":
            return 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
        raise ValueError(kind)

    def swiglu(self, gate_up, out, activation="silu") -> None:
        I = out.shape[1]
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
        out.copy_((self._act(g, activation) * u).to(out.dtype))

    def activate(self, src, offset, kind, out) -> None:
        out.copy_(self._act(src[:, offset: offset + out.shape[1]].float(), kind).to(out.dtype))

    def head_norm_gate(self, o, heads, value_dim, weight, eps, gate, gate_offset, activation, out):
        if weight is not None and weight.shape[0] == heads * value_dim:
            n = o.shape[0]
            x = o.view(n, heads, value_dim)
            y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight.float().view(heads, value_dim)
            z = gate[:, gate_offset: gate_offset + heads * value_dim].reshape(n, heads, value_dim)
            out.copy_((y * self._act(z, activation)).reshape(n, -1).to(out.dtype))
        else:
            super().head_norm_gate(o, heads, value_dim, weight, eps, gate, gate_offset, activation, out)

    def hashed_pair_embed(self, table, token_ids, meta, state, buckets, mul_prev, mul_cur, x) -> None:
        ids = token_ids.long()
        for sg in meta.segments:
            for i in range(sg.n):
                n = sg.row0 + i
                if sg.pos0 + i == 0:
                    r = buckets
                else:
                    prev = int(ids[n - 1]) if i > 0 else int(state[sg.state_slot, 0])
                    r = (prev * mul_prev + int(ids[n]) * mul_cur) % buckets
                x[n] += table[r].float()
            state[sg.state_slot, 0] = ids[sg.row0 + sg.n - 1].to(state.dtype)

    def depth_average(self, streams, depth, coef, x, delta) -> None:
        if delta is not None:
            x += delta
        streams[:, depth + 1] = x
        if coef is not None:
            acc = torch.zeros_like(x)
            for j in range(depth + 2):
                acc = acc + coef[j] * streams[:, j]
            x.copy_(acc)

    def general_delta_scan(self, proj, heads, key_dim, value_dim, remove_offset, decay_in, decay_bias, remove_bias, decay_rate,
                           unit_eps, state, meta, out) -> None:
        H, dk, dv = heads, key_dim, value_dim
        out.zero_()
        for sg in meta.segments:
            rows = slice(sg.row0, sg.row0 + sg.n)
            x = proj[rows].double()
            r = x[:, :H * dk].reshape(-1, H, dk)
            k = x[:, H * dk: 2 * H * dk].reshape(-1, H, dk)
            v = x[:, 2 * H * dk: 2 * H * dk + H * dv].reshape(-1, H, dv)
            a = torch.sigmoid(x[:, remove_offset: remove_offset + H * dk] + remove_bias.double()).reshape(-1, H, dk)
            d = torch.exp(-decay_rate * torch.sigmoid(decay_in[rows].double() + decay_bias.double())).reshape(-1, H, dk)
            u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
            S = state[sg.state_slot].double()
            for t in range(sg.n):
                back = torch.einsum("hk,hkv->hv", u[t], S)
                S = d[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * back[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
                out[sg.row0 + t] = torch.einsum("hkv,hk->hv", S, r[t]).reshape(-1).float()
            state[sg.state_slot] = S.float()

    def rotate_kv_write(self, qkv, cos, sin, rotated, pairing, meta, cache, q_out, num_heads, num_kv_heads, key_dim, value_dim,
                        q_norm=None, k_norm=None, norm_eps=0.0, query_temperature=None):
        n, Hq, Hkv, dk, dv = qkv.shape[0], num_heads, num_kv_heads, key_dim, value_dim
        pos, row = meta.pos.long(), meta.seq_row.long()
        live = row >= 0
        q = qkv[:, :Hq * dk].reshape(n, Hq, dk).float()
        if q_norm is not None:
            q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + norm_eps) * q_norm.float()
        q = self._rot(q, cos, sin, rotated, pairing, pos)
        if query_temperature is not None:
            coef, every = query_temperature
            q = q * (1 + coef * torch.log(torch.floor((pos.float() + 1) / every) + 1))[:, None, None]
        q_out.copy_(torch.where(live[:, None, None], q, torch.zeros(())).reshape(n, -1).to(q_out.dtype))
        if not cache.write:
            return
        k = qkv[:, Hq * dk: (Hq + Hkv) * dk].reshape(n, Hkv, dk).float()
        if k_norm is not None:
            k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + norm_eps) * k_norm.float()
        k = self._rot(k, cos, sin, rotated, pairing, pos)
        v = qkv[:, (Hq + Hkv) * dk: (Hq + Hkv) * dk + Hkv * dv].reshape(n, Hkv, dv)
        table, bs = meta.table(cache.group), cache.page_size
        for i in range(n):
            if not live[i]:
                continue
            page = int(table[row[i], pos[i] // bs])
            assert page >= 0, "a position has no page"
            cache.keys[page, :, pos[i] % bs] = k[i].to(cache.keys.dtype)
            cache.values[page, :, pos[i] % bs] = v[i].to(cache.values.dtype)

    def sink_attention(self, q, cache, meta, out, num_heads, num_kv_heads, key_dim, value_dim, scale, window, keep_first, sink,
                       softcap=0.0, gate=None):
        n, Hq, Hkv, dk, dv = q.shape[0], num_heads, num_kv_heads, key_dim, value_dim
        pos, row = meta.pos.long(), meta.seq_row.long()
        table, bs = meta.table(cache.group), cache.page_size
        out.zero_()
        for i in range(n):
            if row[i] < 0:
                continue
            p = int(pos[i])
            js = [j for j in range(p + 1) if not window or p - j < window or j < keep_first]
            pages = [int(table[row[i], j // bs]) for j in js]
            assert min(pages) >= 0, "a visible key has no page"
            K = torch.stack([cache.keys[pg, :, j % bs] for pg, j in zip(pages, js)]).float()
            V = torch.stack([cache.values[pg, :, j % bs] for pg, j in zip(pages, js)]).float()
            s = torch.einsum("gak,jgk->gaj", q[i].float().view(Hkv, Hq // Hkv, dk), K) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if sink is not None:
                s = torch.cat([s, sink.float().view(Hkv, Hq // Hkv, 1)], -1)
            o = torch.einsum("gaj,jgv->gav", torch.softmax(s, -1)[..., :len(js)], V).reshape(Hq, dv)
            if gate is not None:
                g, off = gate
                o = o * torch.sigmoid(g[i, off: off + Hq].float())[:, None]
            out[i] = o.reshape(-1).to(out.dtype)

    def depth_average_rmsnorm(self, streams, depth, coef, x, delta, weight, eps, h, rows=None) -> bool:
        if not getattr(self, "fuse_depth_norm", True):
            return False
        if rows is None:
            self.depth_average(streams, depth, coef, x, delta)
            self.add_rmsnorm(x, None, weight, eps, h)
            return True
        full = x + delta if delta is not None else x.clone()
        acc = torch.zeros_like(full)
        for j in range(depth + 1):
            acc = acc + coef[j] * streams[:, j]
        acc = acc + coef[depth + 1] * full
        self.add_rmsnorm(acc, None, weight, eps, h, rows)
        return True


class PlainOpsGated(PlainOpsDeep):
    """The operations of the real-gated recurrent unit, of the latent attention with paired neighbours, a sink and an
    output gate, of the attention with a chunked mask and blended values, and of the feed-forward's sum with a block's
    other term."""

    def short_conv(self, h, w, state, meta, out, residual=True, activation=None, bias=None) -> None:
        if bias is None:
            return super().short_conv(h, w, state, meta, out, residual, activation)
        taps = w.shape[1]
        out.zero_()
        for sg in meta.segments:
            rows = h[sg.row0: sg.row0 + sg.n].float()
            line = torch.cat([state[sg.state_slot] if taps > 1 else rows[:0], rows], 0)
            z = torch.zeros_like(rows)
            for j in range(taps):
                z = z + w.float()[:, j] * line[j: j + sg.n]
            z = z + bias.float() + (rows if residual else 0)
            if activation == "silu":
                z = z * torch.sigmoid(z)
            out[sg.row0: sg.row0 + sg.n] = z.to(out.dtype)
            if taps > 1:
                state[sg.state_slot] = line[line.shape[0] - (taps - 1):]

    def _turn_pairs(self, v, cos, sin, rotated, pos, pairing):
        if pairing == 0:
            return self._turn(v, cos, sin, rotated, pos)
        c, s = cos[pos], sin[pos]
        while c.dim() < v.dim():
            c, s = c.unsqueeze(1), s.unsqueeze(1)
        out = v.clone()
        a, b = v[..., 0:rotated:2], v[..., 1:rotated:2]
        out[..., 0:rotated:2], out[..., 1:rotated:2] = a * c - b * s, b * c + a * s
        return out

    def latent_cache_write(self, down, norm_weight, eps, cos, sin, rotated, meta, cache, pairing=0) -> None:
        L = norm_weight.shape[0]
        pos, row = meta.pos.long(), meta.seq_row.long()
        c = down[:, :L]
        c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * norm_weight.float()
        e = torch.cat([c, self._turn_pairs(down[:, L:], cos, sin, rotated, pos, pairing)], -1).to(cache.keys.dtype)
        table, bs = meta.table(cache.group), cache.page_size
        for i in range(down.shape[0]):
            if row[i] >= 0:
                page = int(table[row[i], pos[i] // bs])
                assert page >= 0, f"row {i} at position {int(pos[i])} has no page"
                cache.keys[page, pos[i] % bs] = e[i]

    def rotate_heads(self, q, offset, cos, sin, rotated, meta, out, out_offset, pairing=0) -> None:
        v = self._turn_pairs(q[..., offset:].float(), cos, sin, rotated, meta.pos.long(), pairing)
        v = torch.where((meta.seq_row >= 0)[:, None, None], v, torch.zeros(()))
        out[..., out_offset: out_offset + v.shape[-1]] = v.to(out.dtype)

    def latent_attention(self, q, cache, meta, out, value_width, scale, window, sink=None) -> None:
        if sink is None:
            return super().latent_attention(q, cache, meta, out, value_width, scale, window)
        pos, row = meta.pos.long(), meta.seq_row.long()
        table, bs = meta.table(cache.group), cache.page_size
        out.zero_()
        for i in range(q.shape[0]):
            if row[i] < 0:
                continue
            p = int(pos[i])
            js = torch.arange(max(0, p - window + 1) if window else 0, p + 1)
            pages = table[row[i], js // bs].long()
            assert (pages >= 0).all(), f"row {i}: a visible key's page was given back"
            e = cache.keys[pages, js % bs].float()
            s = torch.cat([(q[i].float() @ e.T) * scale, sink.float()[:, None]], -1)
            out[i] = (torch.softmax(s, -1)[:, :-1] @ e[:, :value_width]).to(out.dtype)

    def activate(self, src, offset, kind, out) -> None:
        z = src[:, offset: offset + out.shape[1]].float()
        out.copy_((z if kind == "identity" else self._act(z, kind)).to(out.dtype))

    def gate_multiply(self, x, gate, gate_offset, kind, out) -> None:
        z = gate[:, gate_offset: gate_offset + x.shape[1]].float()
        out.copy_((x.float() * (z if kind == "identity" else self._act(z, kind))).to(out.dtype))

    def blend_columns(self, dst, dst_offset, src, src_offset, width, weight) -> None:
        w = weight.float()[0]
        d = dst[:, dst_offset: dst_offset + width]
        d.copy_((1.0 - w) * d + w * src[:, src_offset: src_offset + width])

    def rglru_scan(self, u, gates, gate_bias, lam, y, sharpness, state, meta, out) -> None:
        n, W = u.shape
        bw = W // gates.shape[1]
        g = gates.double() + gate_bias.double()
        r = torch.sigmoid(g[..., :bw]).reshape(n, W)
        i = torch.sigmoid(g[..., bw:]).reshape(n, W)
        la = -sharpness * r * torch.nn.functional.softplus(lam.double())
        a, b = torch.exp(la), torch.sqrt(-torch.expm1(2 * la)) * i * u.double()
        out.zero_()
        for sg in meta.segments:
            S = state[sg.state_slot].double()
            for t in range(sg.row0, sg.row0 + sg.n):
                S = a[t] * S + b[t]
                out[t] = (S * y[t].double()).to(out.dtype)
            state[sg.state_slot] = S.float()

    def sink_attention(self, q, cache, meta, out, num_heads, num_kv_heads, key_dim, value_dim, scale, window, keep_first, sink,
                       softcap=0.0, gate=None, span=0):
        if not span:
            return super().sink_attention(q, cache, meta, out, num_heads, num_kv_heads, key_dim, value_dim, scale, window,
                                          keep_first, sink, softcap, gate)
        n, Hq, Hkv, dk, dv = q.shape[0], num_heads, num_kv_heads, key_dim, value_dim
        pos, row = meta.pos.long(), meta.seq_row.long()
        table, bs = meta.table(cache.group), cache.page_size
        out.zero_()
        for i in range(n):
            if row[i] < 0:
                continue
            p = int(pos[i])
            js = [j for j in range(p - p % span, p + 1) if not window or p - j < window]
            pages = [int(table[row[i], j // bs]) for j in js]
            assert min(pages) >= 0, "a visible key has no page"
            K = torch.stack([cache.keys[pg, :, j % bs] for pg, j in zip(pages, js)]).float()
            V = torch.stack([cache.values[pg, :, j % bs] for pg, j in zip(pages, js)]).float()
            s = torch.einsum("gak,jgk->gaj", q[i].float().view(Hkv, Hq // Hkv, dk), K) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if sink is not None:
                s = torch.cat([s, sink.float().view(Hkv, Hq // Hkv, 1)], -1)
            o = torch.einsum("gaj,jgv->gav", torch.softmax(s, -1)[..., :len(js)], V).reshape(Hq, dv)
            if gate is not None:
                g, off = gate
                o = o * torch.sigmoid(g[i, off: off + Hq].float())[:, None]
            out[i] = o.reshape(-1).to(out.dtype)

    def moe_combine(self, terms, weights, shared, gate_logits, gate_column, out, add=None, scale=1.0) -> None:
        n, top = weights.shape
        acc = (terms.view(n, top, -1) * weights[:, :, None]).sum(1)
        if shared is not None:
            acc = acc + (torch.sigmoid(gate_logits[:, gate_column: gate_column + 1]) * shared if gate_logits is not None else shared)
        if add is not None:
            acc = acc + add
        out.copy_(acc * scale)
