"""A stand-in for the CUDA kernel table, for tests that run without a GPU.

It implements the same calls as ``leone_b200.ops.cuda.CudaOps`` with plain
torch on the CPU, reading and writing the same paged pools through the same
block tables.  It lets the ``-m "not gpu"`` tests exercise the step function,
the cache manager and the scheduler end to end.  It is a test fixture only:
the engine never falls back to it.
"""
from __future__ import annotations

import math

import numpy as np
import torch


class EmulatedOps:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype
        self.calls = []

    # -- weights ------------------------------------------------------------------------
    def prepare_matrix(self, w):
        return w

    def prepare_gate_up(self, gate, up):
        return torch.cat([gate, up], dim=0).contiguous()

    def describe_status(self, word):
        return f"emulated status {word}"

    # -- kernels ------------------------------------------------------------------------
    def embedding(self, table, ids, out, status, scale=1.0):
        out.copy_(table[ids.long()].float() * scale)

    def logit_post(self, logits, scale=1.0, soft_cap=None):
        logits.mul_(scale)
        if soft_cap:
            logits.copy_(soft_cap * torch.tanh(logits / soft_cap))

    def rms_norm(self, x, weight, out, eps, rows=None):
        src = x if rows is None else x[rows.long()]
        src = src.float()
        ms = (src * src).mean(dim=-1, keepdim=True)
        out.copy_((src * weight.float() * torch.rsqrt(ms + eps)).to(out.dtype))

    def linear(self, x, w, out, residual=None):
        y = x.float() @ w.float().t()
        if residual is not None:
            y = y + residual
        out.copy_(y.to(out.dtype))

    def linear_swiglu(self, x, w_gate_up, out, gate_shape=None):
        y = x.float() @ w_gate_up.float().t()
        inter = y.shape[1] // 2
        if self.dtype != torch.float32:
            y = y.to(self.dtype).float()
        g, u = y[:, :inter], y[:, inter:]
        slope, limit, shift = gate_shape or (1.0, float("inf"), 0.0)
        g, u = torch.clamp(g, max=limit), torch.clamp(u, min=-limit, max=limit)
        out.copy_((g / (1.0 + torch.exp(-slope * g)) * (u + shift)).to(out.dtype))

    def convert(self, src, out):
        out.copy_(src.to(out.dtype))

    def attention_prepare(self, ctx, qkv, n_q, n_kv, dk, dv, norm, q_w, k_w, eps, freqs, pairing, cache):
        n = qkv.shape[0]
        x = qkv.float()
        q, k = x[:, :n_q * dk], x[:, n_q * dk:(n_q + n_kv) * dk]
        v = qkv[:, (n_q + n_kv) * dk:]
        if norm == "whole":
            q = q * torch.rsqrt((q * q).mean(dim=-1, keepdim=True) + eps) * q_w.float()
            k = k * torch.rsqrt((k * k).mean(dim=-1, keepdim=True) + eps) * k_w.float()
        q, k = q.reshape(n, n_q, dk), k.reshape(n, n_kv, dk)
        if norm == "per_head":
            q = q * torch.rsqrt((q * q).mean(dim=-1, keepdim=True) + eps) * q_w.float()
            k = k * torch.rsqrt((k * k).mean(dim=-1, keepdim=True) + eps) * k_w.float()
        pos = ctx.positions.long()
        q = self._rotate(q, pos, freqs, 1.0, pairing).to(qkv.dtype)
        k = self._rotate(k, pos, freqs, 1.0, pairing).to(qkv.dtype)
        qkv[:, :n_q * dk] = q.reshape(n, -1)
        qkv[:, n_q * dk:(n_q + n_kv) * dk] = k.reshape(n, -1)
        if cache is None:
            return
        pt = cache.page_tokens
        page = cache.block_table[ctx.seq_of_token.long(), pos // pt].long()
        assert (page >= 0).all(), "write into a block without a page"
        cache.k_pool[page, :, pos % pt, :] = k
        cache.v_pool[page, :, pos % pt, :] = v.reshape(n, n_kv, dv)

    def attention_masked(self, ctx, qkv, out, n_q, n_kv, dk, dv, scale, mask, mask_size, weights, bias, cache):
        n = qkv.shape[0]
        q = qkv.float()[:, :n_q * dk].view(n, n_q, dk)
        g = n_q // n_kv
        pt = cache.page_tokens
        res = torch.zeros(n, n_q, dv)
        positions, seqs = ctx.positions.tolist(), ctx.seq_of_token.tolist()
        for t in range(n):
            p, s = positions[t], seqs[t]
            lo = {"causal": 0, "window": max(0, p - mask_size + 1) if mask_size else 0,
                  "chunk": (p // mask_size) * mask_size if mask_size else 0}[mask]
            idx = torch.arange(lo, p + 1)
            pages = cache.block_table[s, idx // pt].long()
            assert (pages >= 0).all(), "read from a block without a page"
            keys = cache.k_pool[pages, :, idx % pt, :].float()      # [ctx, n_kv, dk]
            vals = cache.v_pool[pages, :, idx % pt, :].float()
            for h in range(n_q):
                sc = (keys[:, h // g, :] @ q[t, h]) * scale
                if weights == "sigmoid":
                    w = torch.sigmoid(sc + bias[h])
                elif weights == "softmax_plus_one":
                    w = torch.softmax(torch.cat([sc, torch.zeros(1)]), dim=0)[:-1]
                else:
                    w = torch.softmax(sc, dim=0)
                res[t, h] = (w[:, None] * vals[:, h // g, :]).sum(0)
        out.copy_(res.reshape(n, n_q * dv).to(out.dtype))

    def qk_norm_rope_write(self, ctx, qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, table,
                           rotary_dim, cache, pairing="half_split"):
        n = qkv.shape[0]
        x = qkv.float().view(n, n_q + 2 * n_kv, d)
        q, k, v = x[:, :n_q], x[:, n_q:n_q + n_kv], x[:, n_q + n_kv:]

        def norm(t, w):
            if w is None:
                return t
            ms = (t * t).mean(dim=-1, keepdim=True)
            return t * w.float() * torch.rsqrt(ms + eps)

        def rope(t):
            if table is None:
                return t
            half = rotary_dim // 2
            cs = table[ctx.positions.long()]          # [n, half, 2]
            cos, sin = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
            out = t.clone()
            if pairing == "adjacent":
                a, b = t[..., 0:rotary_dim:2], t[..., 1:rotary_dim:2]
                out[..., 0:rotary_dim:2] = a * cos - b * sin
                out[..., 1:rotary_dim:2] = a * sin + b * cos
                return out
            a, b = t[..., :half], t[..., half:rotary_dim]
            out[..., :half] = a * cos - b * sin
            out[..., half:rotary_dim] = a * sin + b * cos
            return out

        q = rope(norm(q, q_norm_w))
        k = rope(norm(k, k_norm_w))
        new = torch.cat([q, k, v], dim=1).reshape(n, -1).to(qkv.dtype)
        qkv.copy_(new)
        if cache is None:
            return
        kk = new.view(n, n_q + 2 * n_kv, d)[:, n_q:n_q + n_kv]
        vv = new.view(n, n_q + 2 * n_kv, d)[:, n_q + n_kv:]
        pt = cache.page_tokens
        pos = ctx.positions.long()
        seq = ctx.seq_of_token.long()
        page = cache.block_table[seq, pos // pt].long()
        assert (page >= 0).all(), "write into a block without a page"
        cache.k_pool[page, :, pos % pt, :] = kk
        cache.v_pool[page, :, pos % pt, :] = vv

    def attention(self, ctx, qkv, out, n_q, n_kv, d, scale, window, cache):
        n = qkv.shape[0]
        q = qkv.float().view(n, n_q + 2 * n_kv, d)[:, :n_q]
        g = n_q // n_kv
        pt = cache.page_tokens
        res = torch.zeros(n, n_q, d)
        positions = ctx.positions.tolist()
        seqs = ctx.seq_of_token.tolist()
        for t in range(n):
            p, s = positions[t], seqs[t]
            lo = 0 if not window else max(0, p - window + 1)
            idx = torch.arange(lo, p + 1)
            pages = cache.block_table[s, idx // pt].long()
            assert (pages >= 0).all(), "read from a block without a page"
            keys = cache.k_pool[pages, :, idx % pt, :].float()      # [ctx, n_kv, d]
            vals = cache.v_pool[pages, :, idx % pt, :].float()
            for h in range(n_q):
                sc = (keys[:, h // g, :] @ q[t, h]) * scale
                w = torch.softmax(sc, dim=0)
                res[t, h] = (w[:, None] * vals[:, h // g, :]).sum(0)
        out.copy_(res.reshape(n, n_q * d).to(out.dtype))

    # -- stand-ins for the kernels of the 'mixers' module ----------------------------------------
    def rms_norm_pair(self, x, w_a, w_b, out_a, out_b, eps):
        self.rms_norm(x, w_a, out_a, eps)
        self.rms_norm(x, w_b, out_b, eps)

    def relu_squared(self, t):
        t.copy_((torch.relu(t.float()) ** 2).to(t.dtype))

    def linear_per_head(self, a, a_head_stride, w, c, c_head_stride, heads, k, n):
        for h in range(heads):
            c[:, h * c_head_stride:h * c_head_stride + n] = \
                (a[:, h * a_head_stride:h * a_head_stride + k].float() @ w[h].float().t()).to(c.dtype)

    def linear_attention(self, ctx, proj, out, state, decay, heads, dim, vdim, q_off, k_off, v_off, chunk=0):
        silu = torch.nn.functional.silu
        p = proj.float()
        bounds, slots = ctx.q_start.tolist(), ctx.slot_ids.tolist()
        for s, slot in enumerate(slots):
            st = state[slot]
            for t in range(bounds[s], bounds[s + 1]):
                q = silu(p[t, q_off:q_off + heads * dim]).view(heads, dim)
                k = silu(p[t, k_off:k_off + heads * dim]).view(heads, dim)
                v = silu(p[t, v_off:v_off + heads * vdim]).view(heads, vdim)
                st = decay[:, None, None] * st + k[:, :, None] * v[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", st, q).reshape(-1)
            state[slot] = st

    def gate_norm(self, o, weight, gate, out, eps):
        r = torch.rsqrt((o * o).mean(dim=-1, keepdim=True) + eps)
        out.copy_((o * r * weight.float() * torch.sigmoid(gate.float())).to(out.dtype))

    @staticmethod
    def _rotate(x, pos, freqs, magnitude, pairing):
        if freqs is None:
            return x
        ang = pos.float()[:, None] * freqs[None, :]
        cos, sin = torch.cos(ang) * magnitude, torch.sin(ang) * magnitude
        while cos.dim() < x.dim():
            cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
        rd = 2 * freqs.numel()
        out = x.clone()
        if pairing == "adjacent":
            u, v = x[..., 0:rd:2], x[..., 1:rd:2]
            out[..., 0:rd:2], out[..., 1:rd:2] = u * cos - v * sin, v * cos + u * sin
        else:
            u, v = x[..., :rd // 2], x[..., rd // 2:rd]
            out[..., :rd // 2], out[..., rd // 2:rd] = u * cos - v * sin, v * cos + u * sin
        return out

    def latent_prepare(self, ctx, proj, q_abs, heads, dim, rot_dim, rank, norm_w, eps, freqs, magnitude, pairing,
                       cache, q_off, dkv_off):
        n = proj.shape[0]
        p = proj.float()
        pos = ctx.positions.long()
        q = p[:, q_off:q_off + heads * (dim + rot_dim)].view(n, heads, dim + rot_dim)
        q_abs.view(n, heads, rank + rot_dim)[:, :, rank:] = \
            self._rotate(q[:, :, dim:], pos, freqs, magnitude, pairing).to(q_abs.dtype)
        if cache is None:
            return
        dkv = p[:, dkv_off:dkv_off + rank + rot_dim]
        c = dkv[:, :rank]
        c = c * torch.rsqrt((c * c).mean(dim=-1, keepdim=True) + eps) * norm_w.float()
        r = self._rotate(dkv[:, rank:], pos, freqs, magnitude, pairing)
        pt = cache.page_tokens
        page = cache.block_table[ctx.seq_of_token.long(), pos // pt].long()
        assert (page >= 0).all(), "write into a block without a page"
        cache.k_pool[page, 0, pos % pt, :] = torch.cat([c, r], dim=-1).to(cache.k_pool.dtype)

    def attention_latent(self, ctx, q_abs, out, cache, heads, dk, dv, scale, window, sink=None, gate=None):
        n = q_abs.shape[0]
        q = q_abs.float().view(n, heads, dk)
        pt = cache.page_tokens
        res = torch.zeros(n, heads, dv)
        positions, seqs = ctx.positions.tolist(), ctx.seq_of_token.tolist()
        for t in range(n):
            p, s = positions[t], seqs[t]
            lo = 0 if not window else max(0, p - window + 1)
            idx = torch.arange(lo, p + 1)
            pages = cache.block_table[s, idx // pt].long()
            assert (pages >= 0).all(), "read from a block without a page"
            rows = cache.k_pool[pages, 0, idx % pt, :].float()
            sc = (rows @ q[t].t()) * scale                       # [keys, heads]
            if sink is not None:
                sc = torch.cat([sc, sink.float()[None, :]], dim=0)
            w = torch.softmax(sc, dim=0)[:rows.shape[0]]
            res[t] = w.t() @ rows[:, :dv]
            if gate is not None:
                res[t] *= torch.sigmoid(gate[t, :heads].float())[:, None]
        out.copy_(res.reshape(n, heads * dv).to(out.dtype))

    def experts_route(self, x, w_router, chosen, weight, top, softmax=False, renormalize=False, groups=1,
                      groups_kept=None, weight_scale=1.0, bias=None, experts=None, correction=None):
        logits = x.float() @ w_router.float().t()
        z = logits if experts is None else logits[:, :experts]
        if bias is not None:
            z = z + bias
        if softmax == "chosen":
            val, idx = torch.topk(z, top, dim=-1)
            chosen.copy_(idx.reshape(-1).to(torch.int32))
            weight.copy_(torch.softmax(val, dim=-1).reshape(-1) * weight_scale)
            return logits
        s = torch.softmax(z, dim=-1) if softmax else torch.sigmoid(z)
        plain_scores = s
        if correction is not None:
            s = s + correction
        if groups > 1 and (groups_kept or groups) < groups:
            worth = s.view(s.shape[0], groups, -1).max(dim=-1).values
            kept = torch.zeros_like(worth, dtype=torch.bool).scatter_(1, torch.topk(worth, groups_kept, dim=-1).indices, True)
            s = s.masked_fill(~kept.repeat_interleave(s.shape[1] // groups, dim=1), float("-inf"))
        val, idx = torch.topk(s, top, dim=-1)
        if correction is not None:
            val = torch.gather(plain_scores, 1, idx)
        if renormalize:
            val = val / val.sum(dim=-1, keepdim=True)
        chosen.copy_(idx.reshape(-1).to(torch.int32))
        weight.copy_(val.reshape(-1) * weight_scale)
        return logits

    # -- short convolutions with state, the minGRU recurrence, pooled-window attention --------------
    @staticmethod
    def _conv_rows(ctx, x, weight, state, add_input):
        """fp32 rows after the convolution; inputs before the step come from the state."""
        x = x.float()
        taps = weight.shape[1]
        out = torch.zeros_like(x)
        bounds, slots = ctx.q_start.tolist(), ctx.slot_ids.tolist()
        for s, slot in enumerate(slots):
            a, b = bounds[s], bounds[s + 1]
            hist = x[a:b] if taps == 1 else torch.cat([state[slot].float(), x[a:b]], dim=0)
            for t in range(b - a):
                out[a + t] = (weight.t() * hist[t:t + taps]).sum(dim=0)
        return out + x if add_input else out

    def short_conv(self, ctx, x, weight, state, out, add_input=False, update_state=False, activation=None):
        rows = self._conv_rows(ctx, x, weight, state, add_input)
        if activation == "silu":
            rows = torch.nn.functional.silu(rows)
        out.copy_(rows.to(out.dtype))
        if update_state and state is not None:
            self.short_conv_state(ctx, x, state)

    def short_conv_state(self, ctx, x, state):
        keep, channels = state.shape[1], state.shape[2]
        bounds, slots = ctx.q_start.tolist(), ctx.slot_ids.tolist()
        for s, slot in enumerate(slots):
            hist = torch.cat([state[slot], x[bounds[s]:bounds[s + 1], :channels].float()], dim=0)
            state[slot] = hist[hist.shape[0] - keep:]

    def min_gru(self, ctx, proj, z_bias, x_bias, state, out, out_scale=1.0, chunk=0):
        width = out.shape[1]
        p = proj.float()
        z = torch.sigmoid(p[:, :width] + (0 if z_bias is None else z_bias))
        u = p[:, width:2 * width] + (0 if x_bias is None else x_bias)
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        g = p[:, 2 * width:]
        bounds, slots = ctx.q_start.tolist(), ctx.slot_ids.tolist()
        for s, slot in enumerate(slots):
            st = state[slot]
            for t in range(bounds[s], bounds[s + 1]):
                st = (1.0 - z[t]) * st + z[t] * cand[t]
                out[t] = (out_scale * st * g[t] * torch.sigmoid(g[t])).to(out.dtype)
            state[slot] = st

    def scale_rows(self, a, gate, scale=1.0):
        f = scale if gate is None else scale * torch.sigmoid(gate.float().reshape(-1, 1))
        a.copy_((a.float() * f).to(a.dtype))

    def add_scaled(self, x, y, scale=1.0):
        x.add_(y, alpha=scale)

    def attention_pooled_prepare(self, ctx, proj, q_out, n_q, n_kv, dk, dv, conv_w, conv_state, freqs, pairing,
                                 magnitude, unit_norm, eps, cache, update_state=False):
        n = proj.shape[0]
        x = proj.float() if conv_w is None else self._conv_rows(ctx, proj, conv_w, conv_state, False)
        if update_state and conv_state is not None:
            self.short_conv_state(ctx, proj, conv_state)
        q, k = x[:, :n_q * dk].reshape(n, n_q, dk), x[:, n_q * dk:(n_q + n_kv) * dk].reshape(n, n_kv, dk)
        v = x[:, (n_q + n_kv) * dk:].reshape(n, n_kv, dv)
        pos = ctx.positions.long()
        q, k = self._rotate(q, pos, freqs, magnitude, pairing), self._rotate(k, pos, freqs, magnitude, pairing)
        if unit_norm:
            q = q * torch.rsqrt((q * q).mean(dim=-1, keepdim=True) + eps)
            k = k * torch.rsqrt((k * k).mean(dim=-1, keepdim=True) + eps)
        q_out.copy_(q.reshape(n, -1).to(q_out.dtype))
        if not cache.writes:
            return
        pt = cache.page_tokens
        page = cache.block_table[ctx.seq_of_token.long(), pos // pt].long()
        assert (page >= 0).all(), "write into a block without a page"
        cache.k_pool[page, :, pos % pt, :] = k.to(cache.k_pool.dtype)
        cache.v_pool[page, :, pos % pt, :] = v.to(cache.v_pool.dtype)

    def attention_pool_blocks(self, ctx, tokens, blocks, n_kv, dk, dv, pool):
        pt = tokens.page_tokens
        for p, s in zip(ctx.positions.tolist(), ctx.seq_of_token.tolist()):
            if (p + 1) % pool:
                continue
            idx = torch.arange(p - pool + 1, p + 1)
            pages = tokens.block_table[s, idx // pt].long()
            assert (pages >= 0).all(), "a block's token was given back before the block was complete"
            dst = int(blocks.block_table[s, p // pt])
            assert dst >= 0
            row = (p % pt) // pool
            blocks.k_pool[dst, :, row, :] = tokens.k_pool[pages, :, idx % pt, :].float().mean(dim=0).to(blocks.k_pool.dtype)
            blocks.v_pool[dst, :, row, :] = tokens.v_pool[pages, :, idx % pt, :].float().mean(dim=0).to(blocks.v_pool.dtype)

    def attention_pooled(self, ctx, q, out, tokens, blocks, n_q, n_kv, dk, dv, scale, window, pool, out_scale=1.0):
        n = q.shape[0]
        qf = q.float().view(n, n_q, dk)
        g = n_q // n_kv
        pt = tokens.page_tokens
        res = torch.zeros(n, n_q, dv)
        for t, (p, s) in enumerate(zip(ctx.positions.tolist(), ctx.seq_of_token.tolist())):
            idx = torch.arange(max(0, p - window + 1), p + 1)
            pages = tokens.block_table[s, idx // pt].long()
            assert (pages >= 0).all(), "read from a block without a page"
            keys, vals = tokens.k_pool[pages, :, idx % pt, :].float(), tokens.v_pool[pages, :, idx % pt, :].float()
            seen = max(0, (p - window + 1) // pool)
            if seen:
                ends = torch.arange(seen) * pool + pool - 1
                bp = blocks.block_table[s, ends // pt].long()
                assert (bp >= 0).all()
                rows = (ends % pt) // pool
                keys = torch.cat([blocks.k_pool[bp, :, rows, :].float(), keys])
                vals = torch.cat([blocks.v_pool[bp, :, rows, :].float(), vals])
            for h in range(n_q):
                w = torch.softmax((keys[:, h // g, :] @ qf[t, h]) * scale, dim=0)
                res[t, h] = (w[:, None] * vals[:, h // g, :]).sum(0)
        out.copy_((res * out_scale).reshape(n, n_q * dv).to(out.dtype))

    # -- the norm of a sublayer's output, elementwise gates, mixed-head attention, the gated delta rule ----
    def zero(self, t):
        t.zero_()

    def rms_norm_add(self, dst, a, w_a, eps, b=None, w_b=None, coef=1.0, accumulate=True, rounded=None, then=None):
        def normed(x, w):
            return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w.float()
        v = normed(a, w_a)
        if b is not None:
            v = v + normed(b, w_b)
        v = coef * v
        if then is not None:
            v = normed(v, then)
        dst.copy_(dst + v if accumulate else v)
        if rounded is not None:
            rounded.copy_(dst.to(rounded.dtype))

    def gate_rows(self, a, gate, act="sigmoid"):
        g = gate.float()
        f = torch.sigmoid(g) if act == "sigmoid" else g * torch.sigmoid(g)
        a.copy_((a.float() * f).to(a.dtype))

    def gelu_gate(self, z, rows, offset, out):
        g = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
        out.copy_((g * rows[:, offset:offset + out.shape[1]]).to(out.dtype))

    def attention_mixed_heads(self, ctx, q, out, cache, n_q, n_kv, dk, dv, scale, temp, cap, mix, sink, mask, mask_size):
        n = q.shape[0]
        qf = q.float()[:, :n_q * dk].view(n, n_q, dk)
        g = n_q // n_kv
        pt = cache.page_tokens
        res = torch.zeros(n, n_q, dv)
        for t, (p, s) in enumerate(zip(ctx.positions.tolist(), ctx.seq_of_token.tolist())):
            lo = {"causal": 0, "window": max(0, p - mask_size + 1) if mask_size else 0,
                  "chunk": (p // mask_size) * mask_size if mask_size else 0}[mask]
            idx = torch.arange(lo, p + 1)
            pages = cache.block_table[s, idx // pt].long()
            assert (pages >= 0).all(), "read from a block without a page"
            keys = cache.k_pool[pages, :, idx % pt, :].float().repeat_interleave(g, dim=1)      # [ctx, n_q, dk]
            vals = cache.v_pool[pages, :, idx % pt, :].float().repeat_interleave(g, dim=1)
            sc = torch.einsum("jhd,hd->hj", keys, qf[t]) * scale
            if temp is not None:
                sc = sc * temp[:, None]
            if cap:
                sc = cap * torch.tanh(sc / cap)
            if mix is not None:
                sc = mix @ sc
            if sink is not None:
                sc = torch.cat([sc, sink[:, None]], dim=1)
            w = torch.softmax(sc, dim=1)[:, :idx.numel()]
            res[t] = torch.einsum("hj,jhv->hv", w, vals)
        out.copy_(res.reshape(n, n_q * dv).to(out.dtype))

    def gated_delta(self, ctx, act, raw, out, state, a_log, dt_bias, heads, kv_heads, dim, vdim, q_off, k_off, v_off,
                    a_off, b_off, q_scale):
        rep = heads // kv_heads
        bounds, slots = ctx.q_start.tolist(), ctx.slot_ids.tolist()

        def unit(x):
            return x * torch.rsqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)
        for s, slot in enumerate(slots):
            st = state[slot]
            for t in range(bounds[s], bounds[s + 1]):
                q = (unit(act[t, q_off:q_off + kv_heads * dim].view(kv_heads, dim)) * q_scale).repeat_interleave(rep, dim=0)
                k = unit(act[t, k_off:k_off + kv_heads * dim].view(kv_heads, dim)).repeat_interleave(rep, dim=0)
                v = act[t, v_off:v_off + heads * vdim].view(heads, vdim)
                beta = torch.sigmoid(raw[t, b_off:b_off + heads])
                g = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(raw[t, a_off:a_off + heads] + dt_bias))
                st = g[:, None, None] * st
                u = beta[:, None] * (v - torch.einsum("hdv,hd->hv", st, k))
                st = st + k[:, :, None] * u[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", st, q).reshape(-1)
            state[slot] = st

    def group_gate_norm(self, o, weight, gate, out, eps, heads, vdim, act="sigmoid"):
        n = o.shape[0]
        x = o.view(n, heads, vdim)
        y = x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight.float()
        if gate is not None:
            g = gate.float().reshape(n, heads, vdim)
            y = y * (torch.sigmoid(g) if act == "sigmoid" else g * torch.sigmoid(g))
        out.copy_(y.reshape(n, heads * vdim).to(out.dtype))

    def experts_forward(self, x, w_gate, w_up, w_down, chosen, weight, top, scale_input, hidden, rt, identity=0,
                        fresh=False):
        n = x.shape[0]
        silu = torch.nn.functional.silu
        xf = x.float()
        if fresh:
            hidden.zero_()
        for t in range(n):
            for j in range(top):
                e, w = int(chosen[t * top + j]), weight[t * top + j]
                if e >= w_up.shape[0]:
                    assert e < w_up.shape[0] + identity
                    hidden[t] += xf[t] * w
                    continue
                a = xf[t] * w if scale_input else xf[t]
                if w_gate is None:
                    y = w_down[e].float() @ (torch.relu(w_up[e].float() @ a) ** 2)
                else:
                    y = w_down[e].float() @ (silu(w_gate[e].float() @ a) * (w_up[e].float() @ a))
                hidden[t] += y if scale_input else y * w

    def sample(self, logits, temperature, seeds, positions, out):
        from tests.plain.model import sample
        for i in range(logits.shape[0]):
            out[i] = sample(logits[i].tolist(), float(temperature[i]), int(seeds[i]), int(positions[i]))

    def penalize(self, logits, entries, penalties):
        for row, token, count, dry in entries:
            p = penalties[row]
            value = logits[row, token].item()
            if count > 0 and (p.repetition != 1.0 or p.presence != 0.0 or p.frequency != 0.0):
                v = float(value)
                v = v / p.repetition if v > 0.0 else v * p.repetition
                v = v - p.presence - p.frequency * count
                value = float(np.float32(v))
            if dry > 0.0:
                value = float(np.float32(float(value) - dry))
            logits[row, token] = value

    def sample_truncated(self, logits, temperatures, seeds, positions, stages, want_probs=False,
                         maximum_surprise=None, rows=None, out=None):
        from leone_b200.sampling.sampler import TRUNCATION_STAGES
        from tests.plain.model import mirostat_select, select, truncated_probs, uniform
        import math
        names = {v: k for k, v in TRUNCATION_STAGES.items()}
        named = [(names[t], v) for t, v in stages]
        members = list(range(logits.shape[0])) if rows is None else list(rows)
        if out is None:
            out = torch.zeros(logits.shape[0], dtype=torch.int32)
        dists = [truncated_probs(logits[r].tolist(), temperatures[i], named) for i, r in enumerate(members)]
        if maximum_surprise is not None:
            drawn = [mirostat_select(p, maximum_surprise[i], uniform(seeds[i], positions[i])) for i, p in enumerate(dists)]
            for r, (t, _) in zip(members, drawn):
                out[r] = t
            return out, torch.tensor([math.exp(-s_) for _, s_ in drawn], dtype=torch.float64)
        for i, (r, p) in enumerate(zip(members, dists)):
            out[r] = select(p, uniform(seeds[i], positions[i]))
        return (out, torch.tensor(np.stack(dists))) if want_probs else out
