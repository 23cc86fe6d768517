"""A stand-in for the CUDA extension, for tests that run without a GPU.

It has the extension's functions with the same arguments and writes the same outputs, computed
with plain tensor operations on whatever device the tensors are on.  Tests install it with
``monkeypatch.setattr(ops, "_EXT", FakeExt())`` to drive the engine's host logic (batch layout,
cache manager, step function, scheduler, replay) on the CPU.  The package itself never uses it:
without the real extension the product path raises.
"""

from __future__ import annotations

import math

import torch


class FakeExt:
    def smoke_add(self, a, b):
        return a + b

    def embedding(self, ids, table, hidden, status=None, sampled=None, scale=1.0, positions=None, position_rows=None):
        ids = ids.long()
        if sampled is not None:
            ids = torch.where(ids < 0, sampled.long()[(-ids - 1).clamp(min=0)], ids)
        rows = table[ids].float() * scale
        if position_rows is not None:
            rows = rows + position_rows[positions.long()].float()
        hidden.copy_(rows)

    def softcap(self, logits, cap):
        logits.copy_(cap * torch.tanh(logits / cap))

    @staticmethod
    def _layer_norm(x, weight, eps):
        mu = x.mean(-1, keepdim=True)
        var = (x - mu).square().mean(-1, keepdim=True)
        return (x - mu) * torch.rsqrt(var + eps) * weight

    def add_layernorm(self, hidden, delta, weight, out, rows, eps, status=None):
        if rows is None:
            if delta is not None:
                hidden += delta.float()
            x = hidden
        else:
            x = hidden[rows.long()]
            if delta is not None:
                x = x + delta[rows.long()].float()
        out.copy_(self._layer_norm(x, weight, eps).to(out.dtype))

    def branch_layernorm(self, hidden, branch, weight, copy, eps):
        hidden += self._layer_norm(branch.float(), weight, eps)
        if copy is not None:
            copy.copy_(hidden.to(copy.dtype))

    def branch_layernorm_parts(self, hidden, parts, shared, weight, copy, eps, top):
        branch = parts.view(-1, top, parts.shape[1]).sum(1)
        if shared is not None:
            branch = branch + shared.float()
        self.branch_layernorm(hidden, branch, weight, copy, eps)

    def stream_copy(self, hidden, out):
        out.copy_(hidden.to(out.dtype))

    def glu(self, gate_up, out, kind, block, limit, slope):
        inter = gate_up.shape[1] // 2
        block = block or inter
        pairs = gate_up.float().view(gate_up.shape[0], inter // block, 2, block)
        g, u = pairs[:, :, 0].reshape(-1, inter), pairs[:, :, 1].reshape(-1, inter)
        if kind == 0:
            y = g * torch.sigmoid(g) * u
        elif kind == 1:
            y = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))) * u
        else:
            g, u = g.clamp(max=limit), u.clamp(min=-limit, max=limit)
            y = g * torch.sigmoid(slope * g) * (u + 1)
        out.copy_(y.to(out.dtype))

    def add_rmsnorm(self, hidden, delta, weight, out, rows, eps, status=None):
        if delta is not None and delta.dim() == 3:
            delta = delta.sum(0)
        if rows is None:
            if delta is not None:
                hidden += delta.float()
            x = hidden
        else:
            x = hidden[rows.long()]
            if delta is not None:
                x = x + delta[rows.long()].float()
        inv = torch.rsqrt(x.square().mean(-1, keepdim=True) + eps)
        out.copy_((x * inv * weight).to(out.dtype))

    def silu_mul(self, gate_up, out, block=0):
        if gate_up.dim() == 3:
            gate_up = gate_up.sum(0)
        inter = gate_up.shape[1] // 2
        block = block or inter
        pairs = gate_up.float().view(gate_up.shape[0], inter // block, 2, block)
        g, u = pairs[:, :, 0].reshape(-1, inter), pairs[:, :, 1].reshape(-1, inter)
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def qk_norm_rope_write(self, qkv, positions, slots, q_weight, k_weight, inv_freq, q_out, k_out, v_out, k_cache,
                           v_cache, num_heads, num_kv_heads, head_dim, rotary_dim, eps, status=None):
        if qkv.dim() == 3:
            qkv = qkv.sum(0)
        n = qkv.shape[0]
        x = qkv.float().view(n, num_heads + 2 * num_kv_heads, head_dim)
        q, k, v = x[:, :num_heads], x[:, num_heads:num_heads + num_kv_heads], x[:, num_heads + num_kv_heads:]

        def norm(t, w):
            if w is None:
                return t
            return t * torch.rsqrt(t.square().mean(-1, keepdim=True) + eps) * w

        def rotate(t):
            if inv_freq is None or rotary_dim == 0:
                return t
            ang = positions.float()[:, None] * inv_freq[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            half = rotary_dim // 2
            a, b = t[..., :half], t[..., half:rotary_dim]
            return torch.cat((a * cos - b * sin, b * cos + a * sin, t[..., rotary_dim:]), dim=-1)

        q, k = rotate(norm(q, q_weight)), rotate(norm(k, k_weight))
        q_out.copy_(q.reshape(n, -1).to(q_out.dtype))
        if k_out is not None:
            k_out.copy_(k.reshape(n, -1).to(k_out.dtype))
        if v_out is not None:
            v_out.copy_(v.reshape(n, -1).to(v_out.dtype))
        if k_cache is not None and slots is not None:
            self._write(k.to(k_cache.dtype), v.to(v_cache.dtype), slots, k_cache, v_cache)

    @staticmethod
    def _write(k, v, slots, k_cache, v_cache):
        page_size = k_cache.shape[2]
        keep = slots >= 0
        s = slots[keep].long()
        k_cache[s // page_size, :, s % page_size] = k[keep]
        v_cache[s // page_size, :, s % page_size] = v[keep]

    def kv_write(self, k, v, slots, k_cache, v_cache, status=None):
        nkv, d = k_cache.shape[1], k_cache.shape[3]
        self._write(k.view(-1, nkv, d), v.view(-1, nkv, d), slots, k_cache, v_cache)

    def paged_attention(self, q, k_cache, v_cache, out, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq,
                        partials, num_tiles, q_tile, num_splits, num_heads, num_kv_heads, window, scale, status=None,
                        kernel=0):
        page_size, d = k_cache.shape[2], k_cache.shape[3]
        group = num_heads // num_kv_heads
        cu = cu_q.tolist()
        for s, ctx in enumerate(ctx_lens.tolist()):
            q0, q1 = cu[s], cu[s + 1]
            n = q1 - q0
            first_pos = ctx - n
            lo = max(0, first_pos - window + 1) if window else 0
            keys = torch.arange(lo, ctx)
            pages = block_table[s].long()[keys // page_size]
            assert (pages >= 0).all(), "attention would read a page that is not held"
            k = k_cache[pages, :, keys % page_size].float()     # [keys, nkv, d]
            v = v_cache[pages, :, keys % page_size].float()
            qs = q[q0:q1].float().view(n, num_heads, d)
            scores = torch.einsum("thd,shd->hts", qs, k.repeat_interleave(group, dim=1)) * scale
            pos = torch.arange(first_pos, ctx)[:, None]
            visible = keys[None, :] <= pos
            if window:
                visible &= keys[None, :] > pos - window
            scores = scores.masked_fill(~visible[None], -math.inf)
            o = torch.einsum("hts,shd->thd", torch.softmax(scores, -1), v.repeat_interleave(group, dim=1))
            out[q0:q1] = o.reshape(n, -1).to(out.dtype)

    def sample_slices(self):
        return 8

    def sample(self, logits, temperature, uniform, tokens, parts=None, tickets=None):
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t <= 0:
                tokens[r] = int(logits[r].argmax())
                continue
            p = torch.softmax(logits[r].double() / t, -1)
            cdf = torch.cumsum(p, -1)
            target = float(uniform[r]) * float(cdf[-1])
            tokens[r] = min(int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True)),
                            logits.shape[1] - 1)

    # ------------------------------------------------------------------ mixers with reshaped scores / latents

    def scored_attention(self, q, k_cache, v_cache, out, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq,
                         partials, num_tiles, q_tile, num_splits, num_heads, num_kv_heads, v_dim, window, chunk, scale,
                         softcap, slopes=None, gate=None, status=None, kernel=0, keep_first=0, sigmoid_weights=False,
                         head_bias=None, out_scale=1.0):
        page_size = k_cache.shape[2]
        d = q.shape[1] // num_heads
        group = num_heads // num_kv_heads
        cu = cu_q.tolist()
        seqs = sorted(set(tile_seq.tolist()[:num_tiles]))
        lens = ctx_lens.tolist()
        for s in seqs:
            ctx = lens[s]
            q0, q1 = cu[s], cu[s + 1]
            n = q1 - q0
            first_pos = ctx - n
            pos = torch.arange(first_pos, ctx)[:, None]
            lo = 0
            if window:
                lo = max(lo, first_pos - window + 1)
            if chunk:
                lo = max(lo, first_pos // chunk * chunk)
            keys = torch.arange(lo, ctx)
            if keep_first and lo > 0:
                keys = torch.cat((torch.arange(0, min(keep_first, lo)), keys))
            pages = block_table[s].long()[keys // page_size]
            assert (pages >= 0).all(), "attention would read a page that is not held"
            k = k_cache[pages, :, keys % page_size][..., :d].float()
            v = v_cache[pages, :, keys % page_size][..., :v_dim].float()
            qs = q[q0:q1].float().view(n, num_heads, d)
            scores = torch.einsum("thd,shd->hts", qs, k.repeat_interleave(group, dim=1)) * scale
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            if slopes is not None:
                scores = scores - slopes.float()[:, None, None] * (pos - keys[None, :]).float()[None]
            visible = keys[None, :] <= pos
            if window:
                visible &= (keys[None, :] > pos - window) | (keys[None, :] < keep_first)
            if chunk:
                visible &= (keys[None, :] // chunk) == (pos // chunk)
            if sigmoid_weights:
                if head_bias is not None:
                    scores = scores + head_bias.float()[:, None, None]
                weights = torch.sigmoid(scores) * visible[None]
            else:
                weights = torch.softmax(scores.masked_fill(~visible[None], -math.inf), -1)
            o = torch.einsum("hts,shd->thd", weights, v.repeat_interleave(group, dim=1))
            if gate is not None:
                o = o * gate[q0:q1].float()[:, :, None]
            out[q0:q1] = (o * out_scale).reshape(n, -1).to(out.dtype)

    def head_prep(self, x, slots, q_out, k_cache, v_cache, v_keep, v_other, blend_weight, gate_out, num_heads,
                  num_kv_heads, head_dim, v_dim, unit_norm, eps, status=None, q_weight=None, k_weight=None,
                  has_kv=True):
        n = x.shape[0]
        xf = x.float()
        a = num_heads * head_dim
        b, c = (num_kv_heads * head_dim, num_kv_heads * v_dim) if has_kv else (0, 0)
        q, k, v = xf[:, :a].view(n, num_heads, head_dim), xf[:, a:a + b].view(n, -1, head_dim), \
            xf[:, a + b:a + b + c].view(n, -1, v_dim)
        if unit_norm:
            q = q * torch.rsqrt(q.square().mean(-1, keepdim=True) + eps)
            k = k * torch.rsqrt(k.square().mean(-1, keepdim=True) + eps)
        if q_weight is not None:
            q = q * q_weight
        if k_weight is not None:
            k = k * k_weight
        q_out.copy_(q.reshape(n, -1).to(q_out.dtype))
        if v_keep is not None:
            v_keep.copy_(v.reshape(n, -1).to(v_keep.dtype))
        if v_other is not None:
            lam = blend_weight.float()
            v = (1 - lam) * v + lam * v_other.float().view(n, num_kv_heads, v_dim)
        if gate_out is not None:
            gate_out.copy_(torch.sigmoid(xf[:, a + b + c:]))
        if k_cache is not None and slots is not None:
            page_size = k_cache.shape[2]
            keep = slots >= 0
            s = slots[keep].long()
            k_cache[s // page_size, :, s % page_size] = k[keep].to(k_cache.dtype)
            v_cache[s // page_size, :, s % page_size] = v[keep].to(v_cache.dtype)

    @staticmethod
    def _turn_pairs(t, positions, inv_freq, rotary_dims):
        if rotary_dims == 0:
            return t
        ang = positions.float()[:, None] * inv_freq[None, :]
        shape = [t.shape[0]] + [1] * (t.dim() - 2) + [rotary_dims // 2]
        cos, sin = ang.cos().view(shape), ang.sin().view(shape)
        out = t.clone()
        u, v = t[..., 0:rotary_dims:2], t[..., 1:rotary_dims:2]
        out[..., 0:rotary_dims:2] = u * cos - v * sin
        out[..., 1:rotary_dims:2] = v * cos + u * sin
        return out

    def latent_prep(self, x, positions, slots, q_weight, kv_weight, inv_freq, q_latent, cache, q_rank, kv_rank,
                    rot_dim, rotary_dims, eps, status=None):
        xf = x.float()
        a, b, r = xf[:, :q_rank], xf[:, q_rank:q_rank + kv_rank], xf[:, q_rank + kv_rank:]
        q_latent.copy_((a * torch.rsqrt(a.square().mean(-1, keepdim=True) + eps) * q_weight).to(q_latent.dtype))
        if cache is None or slots is None:
            return
        c = b * torch.rsqrt(b.square().mean(-1, keepdim=True) + eps) * kv_weight
        row = torch.cat((c, self._turn_pairs(r, positions, inv_freq, rotary_dims)), dim=-1)
        page_size = cache.shape[2]
        keep = slots >= 0
        s = slots[keep].long()
        cache[s // page_size, 0, s % page_size, :row.shape[1]] = row[keep].to(cache.dtype)

    def rotate_pairs(self, x, out, positions, inv_freq, heads, cols, rotary_dims, in_offset, out_offset):
        n = x.shape[0]
        part = x.view(n, heads, -1)[:, :, in_offset:in_offset + cols].float()
        out.view(n, heads, -1)[:, :, out_offset:out_offset + cols] = \
            self._turn_pairs(part, positions, inv_freq, rotary_dims).to(out.dtype)

    def activation(self, x, out, kind):
        z = x.float()
        if kind == 0:
            y = torch.relu(z).square()
        elif kind == 1:
            y = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
        else:
            y = z / (1 + torch.exp(-z))
        out.copy_(y.to(out.dtype))

    # ------------------------------------------------------------------ the gated delta rule

    def delta_prep(self, x, conv, rate_log, step_bias, state, cu_q, state_slots, qkv, coef, num_heads, num_kv_heads,
                   head_dim, v_dim, taps, unit_eps):
        from ampere_kv_engine_b200.kernels import ops
        G, D, H, V = num_kv_heads, head_dim, num_heads, v_dim
        channels = 2 * G * D + H * V
        memory = ops.delta_state_floats(H, G, D, V, taps)[0]      # where the convolutions' inputs begin
        cu, slots = cu_q.tolist(), state_slots.tolist()
        xf = x.float()
        qkv.zero_()
        coef.zero_()
        for s, slot in enumerate(slots):
            q0, q1 = cu[s], cu[s + 1]
            if slot < 0 or q1 <= q0:
                continue
            before = state[slot, memory:memory + (taps - 1) * channels].view(taps - 1, channels)
            stream = torch.cat((before, xf[q0:q1, :channels]), dim=0)
            y = torch.zeros(q1 - q0, channels)
            for j in range(taps):
                y = y + stream[j:j + q1 - q0] * conv[:, j]
            y = y * torch.sigmoid(y)
            q, k = y[:, :G * D].view(-1, G, D), y[:, G * D:2 * G * D].view(-1, G, D)
            q = q * torch.rsqrt(q.square().sum(-1, keepdim=True) + unit_eps) * D ** -0.5
            k = k * torch.rsqrt(k.square().sum(-1, keepdim=True) + unit_eps)
            qkv[q0:q1] = torch.cat((q.reshape(q1 - q0, -1), k.reshape(q1 - q0, -1), y[:, 2 * G * D:]), dim=1)
            tail = xf[q0:q1, channels + H * V:]
            coef[q0:q1, :H] = torch.sigmoid(tail[:, :H])
            coef[q0:q1, H:] = torch.exp(-torch.exp(rate_log) * torch.nn.functional.softplus(tail[:, H:] + step_bias))

    def delta_scan(self, qkv, coef, x, norm_weight, state, cu_q, state_slots, scratch, out, num_heads, num_kv_heads,
                   head_dim, v_dim, taps, norm_eps):
        from ampere_kv_engine_b200.kernels import ops
        G, D, H, V = num_kv_heads, head_dim, num_heads, v_dim
        channels = 2 * G * D + H * V
        memory = ops.delta_state_floats(H, G, D, V, taps)[0]      # the stand-in keeps S in the first H * D * V floats of it
        cu, slots = cu_q.tolist(), state_slots.tolist()
        out.zero_()
        for s, slot in enumerate(slots):
            q0, q1 = cu[s], cu[s + 1]
            if slot < 0 or q1 <= q0:
                continue
            S = state[slot, :H * D * V].view(H, D, V).clone()
            for t in range(q0, q1):
                q, k = qkv[t, :G * D].view(G, D), qkv[t, G * D:2 * G * D].view(G, D)
                v = qkv[t, 2 * G * D:].view(H, V)
                gate = x[t, channels:channels + H * V].float().view(H, V)
                for h in range(H):
                    j = h // (H // G)
                    S[h] = S[h] * coef[t, H + h]
                    u = coef[t, h] * (v[h] - S[h].T @ k[j])
                    S[h] = S[h] + torch.outer(k[j], u)
                    o = S[h].T @ q[j]
                    o = o * torch.rsqrt(o.square().mean() + norm_eps) * norm_weight * (gate[h] * torch.sigmoid(gate[h]))
                    out[t, h * V:(h + 1) * V] = o.to(out.dtype)
            state[slot, :H * D * V] = S.reshape(-1)
            if taps > 1:
                before = state[slot, memory:memory + (taps - 1) * channels].view(taps - 1, channels)
                stream = torch.cat((before, x[q0:q1, :channels].float()), dim=0)
                state[slot, memory:memory + (taps - 1) * channels] = stream[-(taps - 1):].reshape(-1)

    # ------------------------------------------------------------------ rotary positions, linear memories, the stream

    def rotary_prep(self, x, positions, slots, freq, q_out, k_cache, v_cache, num_heads, num_kv_heads, head_dim, v_dim,
                    rotary_dims, layout, factor=1.0, value_from_key=False, value_norm=False, eps=0.0, status=None,
                    q_norm=None, k_norm=None, row_norm_eps=0.0, x_off=0):
        n = x.shape[0]
        xf = x.float()[:, x_off:]
        a, b = num_heads * head_dim, num_kv_heads * head_dim
        q_row, k_row = xf[:, :a], xf[:, a:a + b]
        k_plain = k_row.view(n, num_kv_heads, head_dim)
        if q_norm is not None:
            q_row = q_row * torch.rsqrt(q_row.square().mean(-1, keepdim=True) + row_norm_eps) * q_norm
            k_row = k_row * torch.rsqrt(k_row.square().mean(-1, keepdim=True) + row_norm_eps) * k_norm
        q, k = q_row.view(n, num_heads, head_dim), k_row.view(n, num_kv_heads, head_dim)
        angle = positions.float()[:, None] * freq.float()[None, :]
        cos, sin = (torch.cos(angle) * factor)[:, None, :], (torch.sin(angle) * factor)[:, None, :]

        def turn(t):
            out = t.clone()
            if layout == 0:
                u, v = t[..., :rotary_dims // 2], t[..., rotary_dims // 2:rotary_dims]
                out[..., :rotary_dims // 2] = u * cos - v * sin
                out[..., rotary_dims // 2:rotary_dims] = v * cos + u * sin
            else:
                u, v = t[..., 0:rotary_dims:2], t[..., 1:rotary_dims:2]
                out[..., 0:rotary_dims:2] = u * cos - v * sin
                out[..., 1:rotary_dims:2] = v * cos + u * sin
            return out

        q_out.copy_(turn(q).reshape(n, -1).to(q_out.dtype))
        if k_cache is None or slots is None:
            return
        if value_from_key:
            v = k_plain
        else:
            v = xf[:, a + b:a + b + num_kv_heads * v_dim].view(n, num_kv_heads, v_dim)
            if value_norm:
                v = v * torch.rsqrt(v.square().mean(-1, keepdim=True) + eps)
        page_size = k_cache.shape[2]
        keep = slots >= 0
        s = slots[keep].long()
        k_cache[s // page_size, :, s % page_size] = turn(k)[keep].to(k_cache.dtype)
        v_cache[s // page_size, :, s % page_size] = v[keep].to(v_cache.dtype)

    def linear_scan_state_floats(self, heads, dim, v_dim):
        from ampere_kv_engine_b200.kernels import ops
        return ops.linear_scan_state_floats(heads, dim, v_dim)

    def linear_scan(self, x, state, cu_q, state_slots, out, num_heads, head_dim, v_dim, mode, q_off, k_off, v_off,
                    gate_bias=None, lower=None, decay=None, qk_group=1, decay_off=0):
        H, D, V = num_heads, head_dim, v_dim
        cu, slots = cu_q.tolist(), state_slots.tolist()
        xf = x.float()
        silu = torch.nn.functional.silu
        if mode >= 2:           # prepared float32 rows: no activation; a decay per head, or per head and token
            for s, slot in enumerate(slots):
                q0, q1 = cu[s], cu[s + 1]
                if slot < 0 or q1 <= q0:
                    continue
                S = state[slot, :H * D * V].view(H, D, V).clone()
                for t in range(q0, q1):
                    q = xf[t, q_off:q_off + H // qk_group * D].view(-1, D).repeat_interleave(qk_group, 0)
                    k = xf[t, k_off:k_off + H // qk_group * D].view(-1, D).repeat_interleave(qk_group, 0)
                    v = xf[t, v_off:v_off + H * V].view(H, V)
                    a = decay if mode == 2 else xf[t, decay_off:decay_off + H]
                    S = a[:, None, None] * S + k[:, :, None] * v[:, None, :]
                    out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
                state[slot, :H * D * V] = S.reshape(-1)
            return
        for s, slot in enumerate(slots):
            q0, q1 = cu[s], cu[s + 1]
            if slot < 0 or q1 <= q0:
                continue
            S = state[slot, :H * D * V].view(H, D, V).clone()       # the stand-in keeps S in plain order
            for t in range(q0, q1):
                q = silu(xf[t, q_off:q_off + H * D]).view(H, D)
                raw = xf[t, k_off:k_off + H * D]
                v = xf[t, v_off:v_off + H * V].view(H, V)
                if mode == 0:
                    f = lower + (1 - lower) * torch.sigmoid(raw + (gate_bias if gate_bias is not None else 0))
                    a, k = f.view(H, D), (1 - f).view(H, D)
                else:
                    a, k, v = decay[:, None].expand(H, D), silu(raw).view(H, D), silu(v)
                S = a[:, :, None] * S + k[:, :, None] * v[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
            state[slot, :H * D * V] = S.reshape(-1)

    def group_norm_gate(self, o, out, weight, group, eps, factor=1.0, x=None, gate_off=0, gate_kind=0, gate_first=False,
                        skip=None, skip_off=0, skip_coef=None, skip_head=1):
        n, width = o.shape
        y = o
        gate = None
        if x is not None:
            z = x[:, gate_off:gate_off + width].float()
            gate = torch.sigmoid(z) if gate_kind == 0 else z * torch.sigmoid(z)
        if skip is not None:
            y = y + skip[:, skip_off:skip_off + width] * skip_coef.repeat_interleave(skip_head)
        if gate is not None and gate_first:
            y = y * gate
        y = y.view(n, width // group, group)
        y = (y * torch.rsqrt(y.square().mean(-1, keepdim=True) + eps)).reshape(n, width) * factor
        if weight is not None:
            y = y * weight.repeat(width // weight.numel())
        if gate is not None and not gate_first:
            y = y * gate
        out.copy_(y.to(out.dtype))

    def rotary_rows(self, x, positions, freq, out, num_heads, head_dim, v_dim, rotary_dims, q_off, k_off, v_off,
                    q_scale=1.0, k_scale=1.0):
        n, H, D = x.shape[0], num_heads, head_dim
        xf = x.float()
        angle = positions.float()[:, None] * freq.float()[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        half = rotary_dims // 2

        def turn(t):
            r = t.clone()
            u, v = t[..., :half], t[..., half:rotary_dims]
            r[..., :half] = u * cos - v * sin
            r[..., half:rotary_dims] = v * cos + u * sin
            return r

        out[:, :H * D] = (turn(xf[:, q_off:q_off + H * D].view(n, H, D)) * q_scale).reshape(n, -1)
        out[:, H * D:2 * H * D] = (turn(xf[:, k_off:k_off + H * D].view(n, H, D)) * k_scale).reshape(n, -1)
        out[:, 2 * H * D:2 * H * D + H * v_dim] = xf[:, v_off:v_off + H * v_dim]

    def ssm_prep(self, x, conv, conv_bias, step_bias, rate_log, state, tail_off, cu_q, state_slots, out, num_heads, v_dim,
                 state_dim, groups, taps, conv_off, step_off):
        H, P = num_heads, v_dim
        inner, gn = H * P, groups * state_dim
        channels = inner + 2 * gn
        cu, slots = cu_q.tolist(), state_slots.tolist()
        xf = x.float()
        out.zero_()
        for s, slot in enumerate(slots):
            q0, q1 = cu[s], cu[s + 1]
            if slot < 0 or q1 <= q0:
                continue
            before = state[slot, tail_off:tail_off + (taps - 1) * channels].view(taps - 1, channels)
            stream = torch.cat((before, xf[q0:q1, conv_off:conv_off + channels]), dim=0)
            y = torch.zeros(q1 - q0, channels) + (conv_bias if conv_bias is not None else 0.0)
            for j in range(taps):
                y = y + stream[j:j + q1 - q0] * conv[:, j]
            y = y * torch.sigmoid(y)
            dt = torch.nn.functional.softplus(xf[q0:q1, step_off:step_off + H] + step_bias)
            out[q0:q1, :gn] = y[:, inner + gn:]
            out[q0:q1, gn:2 * gn] = y[:, inner:inner + gn]
            out[q0:q1, 2 * gn:2 * gn + inner] = y[:, :inner] * dt.repeat_interleave(P, 1)
            out[q0:q1, 2 * gn + inner:2 * gn + inner + H] = torch.exp(-torch.exp(rate_log) * dt)
            out[q0:q1, 2 * gn + inner + H:2 * gn + 2 * inner + H] = y[:, :inner]

    def conv_tail(self, x, state, tail_off, cu_q, state_slots, conv_off, channels, taps):
        cu, slots = cu_q.tolist(), state_slots.tolist()
        for s, slot in enumerate(slots):
            q0, q1 = cu[s], cu[s + 1]
            if slot < 0 or q1 <= q0:
                continue
            before = state[slot, tail_off:tail_off + (taps - 1) * channels].view(taps - 1, channels)
            stream = torch.cat((before, x[q0:q1, conv_off:conv_off + channels].float()), dim=0)
            state[slot, tail_off:tail_off + (taps - 1) * channels] = stream[stream.shape[0] - (taps - 1):].reshape(-1)

    @staticmethod
    def _hyper_write(x, y, mix, write, scale):
        z = y.float() if scale is None else y.float() * scale
        return torch.einsum("st,nsw->ntw", mix, x) + write[None, :, None] * z[:, None, :]

    def hyper_step(self, x, y, mix, write, scale, read, weight, eps, out, rows=None, status=None):
        if y is not None:
            x.copy_(self._hyper_write(x, y, mix, write, scale))
        if out is not None:
            u = torch.einsum("s,nsw->nw", read, x)
            if rows is not None:
                u = u[rows.long()]
            out.copy_((u * torch.rsqrt(u.square().mean(-1, keepdim=True) + eps) * weight).to(out.dtype))

    def hyper_collapse(self, x, y, mix, write, scale, total):
        total.copy_((x if y is None else self._hyper_write(x, y, mix, write, scale)).sum(1))

    def hyper_expand(self, hidden, x):
        x.copy_(hidden[:, None, :].expand_as(x))

    def normed_pair_sum(self, a, b, wa, wb, out, eps, sa, sb):
        na = a * torch.rsqrt(a.square().mean(-1, keepdim=True) + eps) * wa
        nb = b * torch.rsqrt(b.square().mean(-1, keepdim=True) + eps) * wb
        out.copy_((sa * na + sb * nb).to(out.dtype))

    def pair_rows_add(self, hidden, ids, sampled, positions, cu_q, state_slots, last_token, table, vocab, buckets,
                      mul_prev, mul_cur):
        ids = ids.long()
        if sampled is not None:
            ids = torch.where(ids < 0, sampled.long()[(-ids - 1).clamp(min=0)], ids)
        cu, slots = cu_q.tolist(), state_slots.tolist()
        for s, slot in enumerate(slots):
            q0, q1 = cu[s], cu[s + 1]
            if q1 <= q0:
                continue
            prev = torch.empty(q1 - q0, dtype=torch.long)
            prev[0] = int(last_token[slot, 0]) if slot >= 0 else 0
            prev[1:] = ids[q0:q1 - 1]
            rows = (prev * mul_prev + ids[q0:q1] * mul_cur) % buckets
            rows = torch.where(positions[q0:q1].long() > 0, rows, torch.full_like(rows, buckets))
            hidden[q0:q1] += table[rows].float()
            if slot >= 0:
                last_token[slot, 0] = int(ids[q1 - 1])

    def stream_add(self, hidden, other):
        hidden += other

    def scaled_sum(self, a, b, out, sa, sb):
        out.copy_((a.float() * sa + b.float() * sb).to(out.dtype))

    # ------------------------------------------------------------------ routed experts

    def moe_route(self, logits, correction, chosen, weights, groups, keep_groups, group_top, scale, weight_eps,
                  score_kind=0):
        n, E = logits.shape
        top = chosen.shape[1]
        s = torch.sigmoid(logits.float()) if score_kind == 0 else torch.softmax(logits.float(), dim=-1)
        c = s if correction is None else s + correction
        per = E // groups
        grouped = c.view(n, groups, per)
        score = grouped.topk(min(group_top, per), dim=-1).values.sum(-1)
        # ties go to the lower index: a stable sort, descending
        kept = torch.sort(score, dim=-1, descending=True, stable=True).indices[:, :keep_groups]
        allowed = torch.zeros(n, groups, dtype=torch.bool).scatter_(1, kept, True)
        masked = torch.where(allowed[:, :, None].expand(n, groups, per), grouped,
                             torch.full_like(grouped, -math.inf)).reshape(n, E)
        ids = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :top]
        picked = s.gather(1, ids)
        chosen.copy_(ids.to(torch.int32))
        weights.copy_(picked / (picked.sum(-1, keepdim=True) + weight_eps) * scale)

    def moe_router(self, x, w, logits):
        logits.copy_(x.float() @ w.float().T)

    def moe_sort(self, chosen, order, offsets):
        flat = chosen.reshape(-1).long()
        order.copy_(torch.sort(flat, stable=True).indices.to(torch.int32))
        counts = torch.bincount(flat, minlength=offsets.numel() - 1)
        offsets[0] = 0
        offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)

    def moe_gate_up(self, x, w_gate_up, order, offsets, act, top, limit, slope, form=0, up_offset=1.0):
        inter = w_gate_up.shape[1] // 2
        off = offsets.tolist()
        for e in range(len(off) - 1):
            rows = order[off[e]:off[e + 1]].long()
            if rows.numel() == 0:
                continue
            both = x[rows // top].float() @ w_gate_up[e].float().T
            g, u = both[:, :inter].clamp(max=limit), both[:, inter:].clamp(min=-limit, max=limit)
            act[off[e]:off[e + 1]] = (g * torch.sigmoid(slope * g) * (u + up_offset)).to(act.dtype)

    def moe_down(self, act, w_down, order, offsets, weights, out, form=0):
        off = offsets.tolist()
        flat = weights.reshape(-1)
        for e in range(len(off) - 1):
            rows = order[off[e]:off[e + 1]].long()
            if rows.numel() == 0:
                continue
            out[rows] = (act[off[e]:off[e + 1]].float() @ w_down[e].float().T) * flat[rows][:, None]

    def moe_combine(self, parts, shared, out, top):
        total = parts.view(-1, top, parts.shape[1]).sum(1)
        out.copy_(total if shared is None else total + shared.float())
