"""A plain, slow implementation of the Sakinex decoder for the tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 by default.  It shares
no code with ``leone_b200``: it takes the raw ``config.json`` mapping and a dict of tensors under the
checkpoint's names.  Notation: ``h`` is a sublayer's input ``[T, width]``; ``W["foo"]`` is the tensor
``<layer>.mix.foo`` or ``<layer>.mlp.foo``.

The design: layers are pre-norm with a residual multiplier ``m``, ``x <- x + m mixer(c1(norm1 x))``
then ``x <- x + m ff(c2(norm2 x))``, where ``c(h) = h + conv(h)`` is a short causal convolution over
time on every channel.  A span of layers may run several times in a row with the same weights; before
every pass but the first the embedding's rows are added to the stream.  The mixer is two mixers side
by side on the same input, summed with two scales: attention (grouped key/value heads, a short
convolution on the projected q, k and v, a partial half-split rotation with YaRN frequencies, a unit
RMS norm of q and k per head after the rotation, a sliding window and, before the window, one mean
key and value per block of ``pool`` positions) and a minGRU recurrence.  The feed-forward is a
mixture of gated experts chosen by the largest router logits (weights: softmax over the chosen
logits), plus a shared expert times a per-token sigmoid gate.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def linear(x, w):
    return x @ w.t()


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(u, w):
    """``u``: [T, C]; ``w``: [C, taps].  ``y_t = sum_j w[:, j] u_(t - taps + 1 + j)``, zeros before t = 0."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j                  # tap j reads the input `back` positions earlier
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def input_conv(h, w):
    """What a sublayer reads: its input plus the short convolution of its input."""
    return h + causal_conv(h, w)


def yarn_frequencies(dims, base, scaling):
    """Per pair i the angle per position, and the factor on cos and sin."""
    half = dims // 2
    f = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, angle_dtype=torch.float32):
    """``x``: [T, heads, dim]; element i < dims/2 of a head pairs with element i + dims/2."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = yarn_frequencies(dims, rot["base"], rot.get("scaling"))
    f = torch.tensor(f, dtype=torch.float64).to(angle_dtype)
    ang = torch.as_tensor(positions).to(angle_dtype)[:, None] * f[None, :]
    cos = (torch.cos(ang).to(torch.float64) * mag).to(x.dtype)[:, None, :]
    sin = (torch.sin(ang).to(torch.float64) * mag).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def pooled_window_attention(q, k, v, scale, size, pool, cache_round=None):
    """``q``: [T, H, d]; ``k``: [T, G, d]; ``v``: [T, G, dv] as the cache holds them.  Query i sees
    keys j with 0 <= i - j < size, and for every block b of ``pool`` positions with b pool + pool - 1
    <= i - size the mean key and mean value of the block; one softmax over all of them."""
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    n_blocks = T // pool
    if n_blocks:
        kp = k[:n_blocks * pool].reshape(n_blocks, pool, G, d).mean(dim=1)
        vp = v[:n_blocks * pool].reshape(n_blocks, pool, G, dv).mean(dim=1)
        if cache_round is not None:
            kp, vp = cache_round(kp), cache_round(vp)
    for i in range(T):
        lo = max(0, i - size + 1)
        seen = sum(1 for b in range(n_blocks) if b * pool + pool - 1 <= i - size)
        for h in range(H):
            g = h // (H // G)
            keys, vals = k[lo:i + 1, g], v[lo:i + 1, g]
            if seen:
                keys, vals = torch.cat([kp[:seen, g], keys]), torch.cat([vp[:seen, g], vals])
            w = torch.softmax((keys @ q[i, h]) * scale, dim=0)
            out[i, h] = w @ vals
    return out


def left_mixer(h, W, cfg, eps, cache_round=None):
    T = h.shape[0]
    H, G, d, dv = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"]), int(cfg["vdim"])
    q, k, v = linear(h, W["left.q"]), linear(h, W["left.k"]), linear(h, W["left.v"])
    if cfg.get("conv"):
        q, k, v = causal_conv(q, W["left.q.conv"]), causal_conv(k, W["left.k.conv"]), causal_conv(v, W["left.v.conv"])
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    pos = list(range(T))
    if cfg.get("rot"):
        q, k = rotate(q, pos, cfg["rot"]), rotate(k, pos, cfg["rot"])
    q, k = rms(q, eps), rms(k, eps)
    if cache_round is not None:
        k, v = cache_round(k), cache_round(v)
    o = pooled_window_attention(q, k, v, float(cfg["scale"]), int(cfg["mask"]["size"]), int(cfg["mask"]["pool"]),
                                cache_round)
    return linear(o.reshape(T, H * dv), W["left.o"])


def min_gru(h, W):
    """``S_t = (1 - z_t) S_(t-1) + z_t c_t`` element by element from a zero state; the candidate is
    u + 1/2 where u >= 0 and sigmoid(u) where u < 0; output ``W_o (S_t silu(W_g h_t))``."""
    z = torch.sigmoid(linear(h, W["right.z"]) + W["right.z.b"])
    u = linear(h, W["right.x"]) + W["right.x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(u.shape[1], dtype=h.dtype)
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S)
    return linear(torch.stack(rows) * silu(linear(h, W["right.g"])), W["right.o"])


def parallel_mixer(h, W, cfg, eps, cache_round=None):
    return float(cfg["left_scale"]) * left_mixer(h, W, cfg["left"], eps, cache_round) \
        + float(cfg["right_scale"]) * min_gru(h, W)


def gated_expert(h, gate, up, down):
    return linear(silu(linear(h, gate)) * linear(h, up), down)


def route(h, W, cfg):
    """Per token the chosen experts (largest logits, the lowest index among equal ones) and their
    weights (softmax over the chosen logits only)."""
    z = linear(h, W["router"]) + W["router.b"]
    top = int(cfg["router"]["top"])
    chosen, weights = [], []
    for t in range(h.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))[:top]
        chosen.append(order)
        weights.append(torch.softmax(z[t, order], dim=0))
    return chosen, weights


def moe(h, W, cfg):
    chosen, weights = route(h, W, cfg)
    out = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * gated_expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    if cfg.get("shared"):
        gate = torch.sigmoid(linear(h, W["shared.sg"]))            # [T, 1]
        out = out + gate * gated_expert(h, W["shared.gate"], W["shared.up"], W["shared.down"])
    return out


def run_order(config):
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n)), set()
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))
    later_passes = {start + k * (stop - start) for k in range(1, times)}
    return order, later_passes


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, dtype=DT, cache_round=None, streams=None):
    """Logits ``[T, vocab]`` of one whole sequence.  ``cache_round``: what storing a key or a value
    in the cache does to it (identity if None).  ``streams``: a list that receives the residual
    stream after every layer run."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    m = float(config["residual_mult"])
    canon = config.get("canon")
    x0 = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    order, later_passes = run_order(config)
    for pos, i in enumerate(order):
        if pos in later_passes:
            x = x + x0
        layer = config["layers"][i]
        h = rms(x, eps) * t[f"l{i}.norm1"]
        if canon:
            h = input_conv(h, t[f"l{i}.canon1"])
        if layer["type"] != "parallel":
            raise ValueError(f"mixer type {layer['type']}")
        x = x + m * parallel_mixer(h, sub(t, f"l{i}.mix."), layer["mixer"], eps, cache_round)
        if layer.get("mlp"):
            h = rms(x, eps) * t[f"l{i}.norm2"]
            if canon:
                h = input_conv(h, t[f"l{i}.canon2"])
            x = x + m * moe(h, sub(t, f"l{i}.mlp."), layer["mlp"])
        if streams is not None:
            streams.append(x.clone())
    return linear(rms(x, eps) * t["final.norm"], t["head"])


class PlainSakinex:
    def __init__(self, cfg, tensors, dtype=DT, cache_round=None):
        self.cfg, self.tensors, self.dtype, self.cache_round = cfg, tensors, dtype, cache_round
        self._memo = {}

    def logits(self, tokens):
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = forward(self.cfg, self.tensors, list(tokens), self.dtype, self.cache_round)
        return self._memo[key]

    def residuals(self, tokens):
        streams = []
        forward(self.cfg, self.tensors, list(tokens), self.dtype, self.cache_round, streams)
        return torch.stack(streams)
