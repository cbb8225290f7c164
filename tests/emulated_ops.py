"""A torch stand-in for the CUDA extension's call table, for tests without a GPU.

It gives every call of ``starter_b200.csrc.ops.Ops`` the same meaning in slow
torch code on whatever device the tensors are on, so that the host side of the
library (cache, paging, step cutting, generation loop) can be driven on a CPU.
It is test equipment: the library never falls back to it.  The GPU tests also
use these functions as the plain reference of each kernel.
"""

from __future__ import annotations

import math

import torch

from starter_b200.cache.cache import PAGE


def _rnd(t, dtype):
    return t.to(dtype).to(torch.float32)


class EmulatedOps:
    name = "emulated"

    def prepare_matrix(self, w, halves=1):
        return w

    # ---- rows ---------------------------------------------------------------------------

    def embed(self, tokens, table, status, out_float32=False):
        bad = (tokens < 0) | (tokens >= table.shape[0])
        if bool(bad.any()):
            status |= 1
        out = table[tokens.long().clamp(0, table.shape[0] - 1)].clone()
        return out.float() if out_float32 else out

    def grouped_rmsnorm(self, x, deltas, w, groups, eps, out_dtype):
        if deltas:
            total = deltas[0].float()
            for d in deltas[1:]:
                total = total + d.float()
            x.copy_((x.float() + total).to(x.dtype))
        parts = x.float().reshape(x.shape[0], groups, -1)
        n = parts * torch.rsqrt((parts * parts).mean(-1, keepdim=True) + eps)
        return (n.reshape(x.shape) * w.float()).to(out_dtype)

    def gated_clamp(self, gu, alpha, limit):
        inter = gu.shape[1] // 2
        g = gu[:, :inter].float().clamp(max=limit)
        u = gu[:, inter:].float().clamp(min=-limit, max=limit)
        return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(gu.dtype)

    def linear_gated_clamp(self, h, w_gate_up, alpha, limit):
        return self.gated_clamp(self.linear(h, w_gate_up), alpha, limit)

    def tanh(self, x):
        return torch.tanh(x.float()).to(x.dtype)

    def linear_heads(self, a, w, out):
        out.copy_(torch.einsum("rhk,hnk->rhn", a.float(), w.float()).to(out.dtype))
        return out

    @staticmethod
    def _turn(t, pos, freqs, rot):
        """t [rows, heads, R] with its first ``rot`` columns rotated in neighbouring pairs."""
        if freqs is None or not rot:
            return t.clone()
        angle = pos.float()[:, None] * freqs.float()[None, :]
        c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        a, b = t[..., 0:rot:2], t[..., 1:rot:2]
        out = t.clone()
        out[..., 0:rot:2] = a * c - b * s
        out[..., 1:rot:2] = b * c + a * s
        return out

    def rotate_pairs(self, ctx, src, dst, freqs, rot):
        _, pos = self._positions(ctx)
        dst.copy_(self._turn(src.float(), pos, freqs, rot).to(dst.dtype))

    def latent_prepare(self, ctx, down, layer_cache, q_rank, kv_rank, rot_dim, q_norm, kv_norm, eps, freqs, rot, rows_too=False):
        dt = down.dtype
        slots, pos = self._positions(ctx)
        d = down.float()

        def unit(t):
            return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps)

        cq = (unit(d[:, :q_rank]) * q_norm.float()).to(dt)
        latent = unit(d[:, q_rank:q_rank + kv_rank]) * kv_norm.float()
        shared = self._turn(d[:, None, q_rank + kv_rank:], pos, freqs, rot)[:, 0]
        page, off = self._physical(layer_cache.group, slots, pos)
        if bool((page < 0).any()):
            ctx.status |= 2
        ok = page >= 0
        kept = torch.cat([latent, shared], dim=-1).to(dt)
        layer_cache.k[page[ok], 0, off[ok]] = kept[ok]
        return (cq, kept) if rows_too else cq

    def kv_store(self, ctx, k, v, layer_cache, value_norm_eps=None):
        group = layer_cache.group
        G, D, V = group.request.num_kv_heads, group.request.head_dim, group.v_dim
        slots, pos = self._positions(ctx)
        vv = v.float().reshape(-1, G, V)
        if value_norm_eps is not None:
            vv = vv * torch.rsqrt((vv * vv).mean(-1, keepdim=True) + value_norm_eps)
        page, off = self._physical(group, slots, pos)
        if bool((page < 0).any()):
            ctx.status |= 2
        ok = page >= 0
        layer_cache.k[page[ok], :, off[ok]] = k.reshape(-1, G, D)[ok].to(layer_cache.k.dtype)
        layer_cache.v[page[ok], :, off[ok]] = vv[ok].to(layer_cache.v.dtype)

    def flex_attention(self, ctx, q, layer_cache, scale, v_dim, values_in_keys=False, sink=None, head_scale=None, slopes=None,
                       chunk=None, window=None):
        group = layer_cache.group
        M, H, dt = q.shape[0], q.shape[1], q.dtype
        G = group.request.num_kv_heads
        slots, pos = self._positions(ctx)
        out = torch.empty(M, H * v_dim, dtype=dt, device=q.device)
        qf = q.float()
        for r in range(M):
            p = int(pos[r])
            lo = 0
            if window is not None:
                lo = max(lo, p - window + 1)
            if chunk is not None:
                lo = max(lo, (p // chunk) * chunk)
            keys = torch.arange(lo, p + 1, device=q.device)
            page, off = self._physical(group, slots[r].expand(keys.numel()), keys)
            kk = layer_cache.k[page, :, off].float()                               # [n, G, Kd]
            vv = kk[..., :v_dim] if values_in_keys else layer_cache.v[page, :, off].float()
            kk, vv = kk.repeat_interleave(H // G, dim=1), vv.repeat_interleave(H // vv.shape[1], dim=1)
            s = torch.einsum("hd,nhd->hn", qf[r], kk) * scale
            if head_scale is not None:
                s = s * head_scale.float()[:, None]
            if slopes is not None:
                s = s - slopes.float()[:, None] * (p - keys).float()[None, :]
            top = s.max(dim=-1, keepdim=True).values
            if sink is not None:
                top = torch.maximum(top, sink.float()[:, None])
            e = torch.exp(s - top)
            total = e.sum(-1, keepdim=True)
            if sink is not None:
                total = total + torch.exp(sink.float()[:, None] - top)
            out[r] = (torch.einsum("hn,nhd->hd", e, vv) / total).reshape(-1).to(dt)
        return out

    def token_shift(self, ctx, h, state, prev_offset, mu):
        slots = ctx.seq_slot.long()[ctx.row_seq.long()]
        first = ctx.cu_q.long()[ctx.row_seq.long()]
        rows = torch.arange(ctx.n_rows, device=h.device)
        hf = h.float()
        before = torch.where((rows == first)[:, None], state[slots, prev_offset:prev_offset + h.shape[1]].float(),
                             hf[(rows - 1).clamp(min=0)])
        return (hf[None] + (before - hf)[None] * mu.float()[:, None, :]).to(h.dtype)

    def wkv_scan(self, ctx, r, k, v, g, decay_pre, w0, u, norm, eps, h, state, heads, dim, prev_offset):
        H, D = heads, dim
        out = torch.empty(r.shape[0], H * D, dtype=torch.float32, device=r.device)
        cu = ctx.cu_q.tolist()
        decay = torch.exp(-torch.exp(decay_pre.float() + w0.float())).reshape(-1, H, D)
        rr, kk, vv = (t.float().reshape(-1, H, D) for t in (r, k, v))
        uu = u.float().reshape(H, D)
        for b in range(ctx.n_seqs):
            slot = int(ctx.seq_slot[b])
            S = state[slot, :prev_offset].reshape(H, D, D).clone()
            for t in range(cu[b], cu[b + 1]):
                kv = kk[t][:, :, None] * vv[t][:, None, :]
                out[t] = torch.einsum("hk,hkv->hv", rr[t], S + uu[:, :, None] * kv).reshape(-1)
                S = decay[t][:, :, None] * S + kv
            state[slot, :prev_offset] = S.reshape(-1)
            if cu[b + 1] > cu[b]:
                state[slot, prev_offset:prev_offset + h.shape[1]] = h[cu[b + 1] - 1].float()
        o = out.reshape(-1, H, D)
        o = (o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps)).reshape(-1, H * D)
        gf = g.float()
        return (o * norm.float() * (gf * torch.sigmoid(gf))).to(r.dtype)

    # ---- streams, two-map attention, gated linear attention, experts ----------------------

    def embed_streams(self, tokens, table, status, scale, copies):
        rows = self.embed(tokens, table, status).float()
        if scale is not None:
            rows = rows * scale
        return rows.repeat(1, copies).contiguous()

    def stream_norm(self, x, streams, pending, read_w, weight, eps, out_dtype):
        rows = x.shape[0]
        X = x.view(rows, streams, -1)
        if pending is not None:
            y, mix, out = pending
            new = torch.einsum("st,rsw->rtw", mix.float(), X) + out.float()[None, :, None] * y.float()[:, None, :]
            X.copy_(new)
        if read_w is None:
            return None
        u = torch.einsum("s,rsw->rw", read_w.float(), X)
        return (u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * weight.float()).to(out_dtype)

    def rotate_half_store(self, ctx, q, k, v, layer_cache, freqs, rot, magnitude):
        group = layer_cache.group
        slots, pos = self._positions(ctx)

        def turn(t):
            t = t.float()
            if freqs is None or not rot:
                return t
            angle = pos.float()[:, None] * freqs.float()[None, :]
            c, s = (torch.cos(angle) * magnitude)[:, None, :], (torch.sin(angle) * magnitude)[:, None, :]
            a, b = t[..., :rot // 2], t[..., rot // 2:rot]
            return torch.cat([a * c - b * s, b * c + a * s, t[..., rot:]], dim=-1)

        page, off = self._physical(group, slots, pos)
        if bool((page < 0).any()):
            ctx.status |= 2
        ok = page >= 0
        layer_cache.k[page[ok], :, off[ok]] = turn(k)[ok].to(layer_cache.k.dtype)
        layer_cache.v[page[ok], :, off[ok]] = v.reshape(v.shape[0], group.v_heads, group.v_dim)[ok].to(layer_cache.v.dtype)
        return turn(q).to(q.dtype)

    def diff_combine(self, a, heads, kv_heads, v_dim, lam, eps, post, gate=None):
        rows, per = a.shape[0], heads // kv_heads
        maps = a.float().view(rows, kv_heads, 2, per, v_dim)
        o = maps[:, :, 0] - lam * maps[:, :, 1]
        o = (o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * post).reshape(rows, heads * v_dim)
        if gate is not None:
            o = o * torch.sigmoid(gate.float())
        return o.to(a.dtype)

    # ---- layers in passes, mixers side by side, keys as values, the matrix memory ----------

    def add_rows(self, x, rows_too=None, vector=None, out=None):
        total = x.float()
        if rows_too is not None:
            total = total + rows_too
        if vector is not None:
            total = total + vector[None, :]
        if out is None:
            return total.clone()
        out.copy_(total)
        return out

    def add_bias(self, y, bias):
        y.copy_((y.float() + bias.float()[None, :]).to(y.dtype))
        return y

    def linear_bias(self, a, w, bias):
        return self.add_bias(self.linear(a, w), bias)

    def scaled_sum(self, a, sa, b, sb):
        return (sa * a.float() + sb * b.float()).to(a.dtype)

    def relu2(self, z):
        return (torch.relu(z.float()) ** 2).to(z.dtype)

    def linear_relu2(self, h, w_up):
        return self.relu2(self.linear(h, w_up))

    def conv_qk_store(self, ctx, q, k, layer_cache, state, n_heads, q_bias, k_bias, q_conv, k_conv, q_norm, k_norm, eps,
                      temp_coef, temp_every):
        group = layer_cache.group
        G, D = group.request.num_kv_heads, group.request.head_dim
        rows = q.shape[0]
        u = torch.cat([q.float() + (q_bias.float() if q_bias is not None else 0.0),
                       k.float() + (k_bias.float() if k_bias is not None else 0.0)], dim=1)
        y = u
        if q_conv is not None:
            w = torch.cat([q_conv.float(), k_conv.float()], dim=0)
            taps = w.shape[1]
            y = torch.zeros_like(u)
            for b in range(ctx.n_seqs):
                slot, r0, r1 = int(ctx.seq_slot[b]), int(ctx.cu_q[b]), int(ctx.cu_q[b + 1])
                past = state[slot].float() if taps > 1 else u.new_zeros((0, u.shape[1]))
                hist = torch.cat([past, u[r0:r1]], dim=0)
                for j in range(taps):
                    y[r0:r1] += w[:, j][None, :] * hist[j:j + (r1 - r0)]
                if taps > 1:
                    state[slot] = hist[hist.shape[0] - (taps - 1):]
        yq, yk = y[:, :n_heads * D].reshape(rows, n_heads, D), y[:, n_heads * D:].reshape(rows, G, D)

        def unit(t, w):
            return t if w is None else t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.float()

        slots, pos = self._positions(ctx)
        qn = unit(yq, q_norm)
        if temp_every:
            qn = qn * (1.0 + temp_coef * torch.log((torch.div(pos + 1, temp_every, rounding_mode="floor") + 1).float()))[:, None, None]
        page, off = self._physical(group, slots, pos)
        if bool((page < 0).any()):
            ctx.status |= 2
        ok = page >= 0
        layer_cache.k[page[ok], :, off[ok]] = unit(yk, k_norm)[ok].to(layer_cache.k.dtype)
        layer_cache.v[page[ok], :, off[ok]] = yk[ok].to(layer_cache.v.dtype)
        return qn.to(q.dtype)

    def head_gate(self, a, z, z_col, heads, scale=1.0, out=None):
        rows, width = a.shape
        gate = torch.sigmoid(z[:, z_col:z_col + heads].float())
        res = (a.float().reshape(rows, heads, -1) * gate[:, :, None] * scale).reshape(rows, width).to(a.dtype)
        if out is None:
            return res
        out.copy_(res)
        return out

    def mlstm_scan(self, ctx, q, k, v, g, z, i_col, f_col, i_bias, f_bias, cap, norm, eps, q_scale, state, heads, dim, vdim,
                   out_scale=1.0, out=None):
        dest = out
        H, D, V = heads, dim, vdim
        rows = q.shape[0]
        out = torch.empty(rows, H, V, dtype=torch.float32, device=q.device)
        cu = ctx.cu_q.tolist()
        ig = cap * torch.tanh((z[:, i_col:i_col + H].float() + i_bias.float()) / cap)
        fg = torch.nn.functional.logsigmoid(cap * torch.tanh((z[:, f_col:f_col + H].float() + f_bias.float()) / cap))
        qq, kk, vv = q.float().reshape(rows, H, D) * q_scale, k.float().reshape(rows, H, D), v.float().reshape(rows, H, V)
        for b in range(ctx.n_seqs):
            slot = int(ctx.seq_slot[b])
            rec = state[slot]
            S = rec[:H * D * V].reshape(H, D, V).clone()
            n = rec[H * D * V:H * D * V + H * D].reshape(H, D).clone()
            m = rec[H * D * V + H * D:].clone()
            for t in range(cu[b], cu[b + 1]):
                m_new = torch.maximum(fg[t] + m, ig[t])
                a_, b_ = torch.exp(fg[t] + m - m_new), torch.exp(ig[t] - m_new)
                S = a_[:, None, None] * S + (b_[:, None] * kk[t])[:, :, None] * vv[t][:, None, :]
                n = a_[:, None] * n + b_[:, None] * kk[t]
                m = m_new
                den = torch.maximum((n * qq[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
                out[t] = torch.einsum("hk,hkv->hv", qq[t], S) / den[:, None]
            state[slot] = torch.cat([S.reshape(-1), n.reshape(-1), m])
        o = out * torch.rsqrt((out * out).mean(-1, keepdim=True) + eps)
        res = (o.reshape(rows, H * V) * norm.float() * torch.sigmoid(g.float()) * out_scale).to(q.dtype)
        if dest is None:
            return res
        dest.copy_(res)
        return dest

    def gla_scan(self, ctx, q, k, v, g, z, bias, norm, eps, tau, q_scale, state, heads, dim, vdim):
        H, D, V = heads, dim, vdim
        rows = q.shape[0]
        out = torch.empty(rows, H, V, dtype=torch.float32, device=q.device)
        cu = ctx.cu_q.tolist()
        decay = torch.exp(torch.nn.functional.logsigmoid(z.float() + bias.float()) / tau).reshape(rows, H, D)
        qq, kk, vv = q.float().reshape(rows, H, D) * q_scale, k.float().reshape(rows, H, D), v.float().reshape(rows, H, V)
        for b in range(ctx.n_seqs):
            slot = int(ctx.seq_slot[b])
            S = state[slot].reshape(H, D, V).clone()
            for t in range(cu[b], cu[b + 1]):
                S = decay[t][:, :, None] * S + kk[t][:, :, None] * vv[t][:, None, :]
                out[t] = torch.einsum("hk,hkv->hv", qq[t], S)
            state[slot] = S.reshape(-1)
        o = out * torch.rsqrt((out * out).mean(-1, keepdim=True) + eps) * norm.float()
        gf = g.float()
        return (o.reshape(rows, H * V) * (gf * torch.sigmoid(gf))).to(q.dtype)

    def moe_route(self, h, router, correction, top, scale, bias=None, over_chosen=False):
        z = h.float() @ router.float().T
        if bias is not None:
            z = z + bias.float()
        if over_chosen:
            chosen = torch.topk(z if correction is None else z + correction.float(), top, dim=-1).indices
            return chosen.to(torch.int32), torch.softmax(torch.gather(z, 1, chosen), dim=-1) * scale
        s = torch.softmax(z, dim=-1)
        chosen = torch.topk(s if correction is None else s + correction.float(), top, dim=-1).indices
        picked = torch.gather(s, 1, chosen)
        return chosen.to(torch.int32), picked / (picked.sum(-1, keepdim=True) + 1e-20) * scale

    def moe_experts(self, h, chosen, weight, w_gate_up, w_down, n_experts, alpha, limit, base):
        out = torch.zeros(h.shape, dtype=torch.float32, device=h.device) if base is None else base.float().clone()
        for r in range(h.shape[0]):
            for e, w in zip(chosen[r].tolist(), weight[r]):
                if e >= n_experts:
                    out[r] += w * h[r].float()
                else:
                    gu = self.linear(h[r:r + 1], w_gate_up[e])
                    act = self.swiglu(gu) if alpha is None else self.gated_clamp(gu, alpha, limit)
                    out[r] += w * self.linear(act, w_down[e])[0].float()
        return out.to(h.dtype)

    def gather_rows(self, x, rows):
        return x[rows.long()].clone()

    def rmsnorm(self, x, w, eps):
        xf = x.float()
        n = xf * torch.rsqrt((xf * xf).sum(-1, keepdim=True) / x.shape[-1] + eps)
        return (_rnd(n, x.dtype) * w.float()).to(x.dtype)

    def add_rmsnorm(self, x, delta, w, eps):
        x.copy_((x.float() + delta.float()).to(x.dtype))
        return self.rmsnorm(x, w, eps)

    def linear(self, a, w, out_float32=False):
        out = a.float() @ w.float().T
        return out if out_float32 else out.to(a.dtype)

    def swiglu(self, gu):
        inter = gu.shape[1] // 2
        g, u = gu[:, :inter].float(), gu[:, inter:].float()
        s = _rnd(g / (1.0 + torch.exp(-g)), gu.dtype)
        return (s * u).to(gu.dtype)

    def linear_swiglu(self, h, w_gate_up):
        return self.swiglu(self.linear(h, w_gate_up))

    # ---- cache --------------------------------------------------------------------------

    @staticmethod
    def _positions(ctx):
        slots = ctx.seq_slot.long()[ctx.row_seq.long()]
        first = ctx.cu_q.long()[ctx.row_seq.long()]
        rows = torch.arange(ctx.n_rows, device=slots.device)
        return slots, ctx.lengths.long()[slots] + rows - first

    @staticmethod
    def _physical(group, slots, pos):
        logical = pos // PAGE
        if group.ring_pages:
            pinned = getattr(group, "pinned_pages", 0)
            logical = torch.where(logical < pinned, logical, pinned + (logical - pinned) % group.ring_pages)
        return group.table.long()[slots, logical], pos % PAGE

    # ---- a position vector at the embedding, the short convolution, attention with scores mixed across heads ----

    def embed_sinusoid(self, ctx, tokens, table, freqs):
        bad = (tokens < 0) | (tokens >= table.shape[0])
        if bool(bad.any()):
            ctx.status |= 1
        x = table[tokens.long().clamp(0, table.shape[0] - 1)].float()
        _, pos = self._positions(ctx)
        angle = pos.float()[:, None] * freqs.float()[None, :]
        vec = torch.stack([torch.sin(angle), torch.cos(angle)], dim=-1).reshape(x.shape[0], -1)
        return x + vec[:, :x.shape[1]]

    def cast_rows(self, x, dtype):
        return x.to(dtype)

    def causal_conv(self, ctx, x, weight, state, out_dtype):
        taps = weight.shape[1]
        out = x.float().clone()
        w = weight.float()
        for b in range(ctx.n_seqs):
            slot, r0, r1 = int(ctx.seq_slot[b]), int(ctx.cu_q[b]), int(ctx.cu_q[b + 1])
            past = state[slot].float() if taps > 1 else x.new_zeros((0, x.shape[1]), dtype=torch.float32)
            hist = torch.cat([past, x[r0:r1].float()], dim=0)          # row t of the step is hist[t + taps - 1]
            for j in range(taps):
                out[r0:r1] += w[:, j][None, :] * hist[j:j + (r1 - r0)]
            if taps > 1:
                state[slot] = hist[hist.shape[0] - (taps - 1):]
        return out.to(out_dtype)

    def qk_norm_store(self, ctx, qkv, layer_cache, n_heads, q_norm, k_norm, eps):
        group = layer_cache.group
        G, D, V = group.request.num_kv_heads, group.request.head_dim, group.v_dim
        nq = n_heads * D
        dt = qkv.dtype

        def unit(t, w):
            t = t.float()
            return t if w is None else t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.float()

        q = unit(qkv[:, :nq], q_norm).to(dt)
        k = unit(qkv[:, nq:nq + G * D], k_norm).to(dt)
        slots, pos = self._positions(ctx)
        page, off = self._physical(group, slots, pos)
        if bool((page < 0).any()):
            ctx.status |= 2
        ok = page >= 0
        layer_cache.k[page[ok], :, off[ok]] = k.reshape(-1, G, D)[ok]
        layer_cache.v[page[ok], :, off[ok]] = qkv[:, nq + G * D:].reshape(-1, G, V)[ok]
        return q

    def talking_attention(self, ctx, q, layer_cache, n_heads, scale, softcap=None, talk=None, sink=None, window=None,
                          keep_first=0):
        group = layer_cache.group
        G, D, V = group.request.num_kv_heads, group.request.head_dim, group.v_dim
        H, M, dt = n_heads, q.shape[0], q.dtype
        slots, pos = self._positions(ctx)
        out = torch.empty(M, H * V, dtype=dt, device=q.device)
        qf = q.float().reshape(M, H, D)
        for r in range(M):
            p = int(pos[r])
            keys = torch.arange(0, p + 1, device=q.device)
            if window is not None:
                keys = keys[(p - keys < window) | (keys < keep_first)]
            page, off = self._physical(group, slots[r].expand(keys.numel()), keys)
            kk = layer_cache.k[page, :, off].float().repeat_interleave(H // G, dim=1)      # [n, H, D]
            vv = layer_cache.v[page, :, off].float().repeat_interleave(H // G, dim=1)
            s = torch.einsum("hd,nhd->hn", qf[r], kk) * scale
            if softcap is not None:
                s = softcap * torch.tanh(s / softcap)
            if talk is not None:
                s = talk.float() @ s
            top = s.max(dim=-1, keepdim=True).values
            if sink is not None:
                top = torch.maximum(top, sink.float()[:, None])
            e = torch.exp(s - top)
            total = e.sum(-1, keepdim=True)
            if sink is not None:
                total = total + torch.exp(sink.float()[:, None] - top)
            out[r] = (torch.einsum("hn,nhd->hd", e, vv) / total).reshape(-1).to(dt)
        return out

    def branch_norm_add(self, x, y, weight, scale, eps, out_dtype, next_norm=None):
        yf = y.float()
        n = yf * torch.rsqrt((yf * yf).mean(-1, keepdim=True) + eps) * weight.float()
        if scale is not None:
            n = n * scale.float()
        x.add_(n)
        if next_norm is not None:
            return (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + next_norm[1]) * next_norm[0].float()).to(y.dtype)
        if out_dtype is None:
            return None
        return x if x.dtype == out_dtype else x.to(out_dtype)

    def xielu(self, z, a_pos, a_neg):
        zf = z.float()
        neg = a_neg * (torch.exp(zf.clamp(max=0.0)) - 1.0 - zf) + 0.5 * zf
        return torch.where(zf > 0, a_pos * zf * zf + 0.5 * zf, neg).to(z.dtype)

    def linear_xielu(self, h, w_up, a_pos, a_neg):
        return self.xielu(self.linear(h, w_up), a_pos, a_neg)

    def qk_norm_rope_store(self, ctx, qkv, layer_cache, n_heads, n_kv_heads, head_dim, q_norm, k_norm, eps, rotary):
        M, D, dt = qkv.shape[0], head_dim, qkv.dtype
        slots, pos = self._positions(ctx)
        q = qkv[:, :n_heads * D].float().reshape(M, n_heads, D)
        k = qkv[:, n_heads * D:(n_heads + n_kv_heads) * D].float().reshape(M, n_kv_heads, D)
        v = qkv[:, (n_heads + n_kv_heads) * D:].reshape(M, n_kv_heads, D)

        def norm(t, w):
            if w is None:
                return t
            n = _rnd(t * torch.rsqrt((t * t).sum(-1, keepdim=True) / D + eps), dt)
            return _rnd(n * w.float(), dt)

        def rope(t):
            if rotary is None:
                return t
            cos, sin, rd = rotary
            half = rd // 2
            c = cos.float()[pos][:, None, :]
            s = sin.float()[pos][:, None, :]
            t1, t2 = t[..., :half], t[..., half:rd]
            o1 = _rnd(_rnd(t1 * c, dt) + _rnd(-t2 * s, dt), dt)
            o2 = _rnd(_rnd(t2 * c, dt) + _rnd(t1 * s, dt), dt)
            return torch.cat([o1, o2, t[..., rd:]], dim=-1)

        q = rope(norm(q, q_norm))
        if n_kv_heads:
            k = rope(norm(k, k_norm))
            group = layer_cache.group
            page, off = self._physical(group, slots, pos)
            if bool((page < 0).any()):
                ctx.status |= 2
            ok = page >= 0
            layer_cache.k[page[ok], :, off[ok]] = k[ok].to(dt)
            layer_cache.v[page[ok], :, off[ok]] = v[ok].to(dt)
        return q.reshape(M, n_heads * D).to(dt)

    def attention(self, ctx, q, layer_cache, n_heads, scale, window):
        group = layer_cache.group
        M, dt = q.shape[0], q.dtype
        D = group.request.head_dim
        hkv = group.request.num_kv_heads
        rep = n_heads // hkv
        slots, pos = self._positions(ctx)
        out = torch.empty(M, n_heads * D, dtype=dt, device=q.device)
        qf = q.float().reshape(M, n_heads, D)
        for r in range(M):
            p = int(pos[r])
            lo = 0 if window is None else max(0, p - window + 1)
            keys = torch.arange(lo, p + 1, device=q.device)
            page, off = self._physical(group, slots[r].expand(keys.numel()), keys)
            kk = layer_cache.k[page, :, off].float().repeat_interleave(rep, dim=1)  # [n, HQ, D]
            vv = layer_cache.v[page, :, off].float().repeat_interleave(rep, dim=1)
            s = torch.einsum("hd,nhd->hn", qf[r], kk) * scale
            pr = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            total = pr.sum(-1, keepdim=True)
            pv = torch.einsum("hn,nhd->hd", _rnd(pr, dt), vv) / total
            out[r] = pv.reshape(-1).to(dt)
        return out

    def advance_lengths(self, ctx):
        counts = (ctx.cu_q[1:] - ctx.cu_q[:-1]).to(ctx.lengths.dtype)
        slots = ctx.seq_slot.long()
        real = slots < ctx.cache.null_slot
        ctx.lengths[slots[real]] += counts[real]

    # ---- sampling -----------------------------------------------------------------------

    def argmax(self, logits):
        return logits.float().argmax(dim=-1).to(torch.int32)

    def sample(self, logits, temperature, top_k, seed, request_ids, steps, advance=False, device_params=None):
        from plain import qwen3_plain as plain
        if device_params is not None:
            import struct
            words = [int(v) & 0xffffffff for v in device_params.tolist()]
            (temperature,) = struct.unpack("<f", struct.pack("<I", words[0]))
            top_k, seed = words[1], words[2] | (words[3] << 32)
        out = []
        for r in range(logits.shape[0]):
            req = int(request_ids[r]) if request_ids is not None else r
            step = int(steps[r]) if steps is not None else 0
            tok, _ = plain.sample(logits[r].float().cpu(), temperature, top_k, plain.uniform_from_counter(seed, req, step))
            out.append(tok)
        if advance and steps is not None:
            steps += 1
        return torch.tensor(out, dtype=torch.int32, device=logits.device)
