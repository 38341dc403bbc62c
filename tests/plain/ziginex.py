"""A plain, slow implementation of the Ziginex decoder for the tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 by default.  It shares
no code with ``leone_b200``: it takes the raw ``config.json`` mapping and a dict of tensors under the
checkpoint's names.  Notation: ``h`` is a sublayer's input ``[T, width]``; ``W["foo"]`` is the tensor
``<layer>.mix.foo`` or ``<layer>.mlp.foo``.

The design: a sublayer reads the residual stream itself and its *output* is RMS-normed before it is
added, ``x <- x + norm1(mixer(x))``, ``x <- x + norm2(ff(x))``; after the feed-forward every layer adds
a small gated term made from a second embedding table of the token (``token_side``).  Mixers:
``parallel`` (softmax attention in chunks with per-head temperature, a soft cap, scores mixed across
heads and a sink, beside a gated delta-rule recurrence behind short convolutions; each output is
RMS-normed over the width, and the mixer is half their sum) and ``latent_attention`` (queries and
keys/values through normed latents, one rotated key part shared by the heads, YaRN frequencies, a
sink, an elementwise output gate).  Feed-forwards: a dense gated layer, or a mixture of gated experts
chosen among the best groups by ``softmax + correction`` and weighted by the softmax alone, the last
router outputs being experts that pass their input on unchanged.  The head is the embedding table.
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot):
    """Per pair i the angle per position and the factor on cos and sin (YaRN if ``scaling``)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, layout, angle_dtype=torch.float32):
    """``x``: [T, heads, dim]; the first ``dims`` elements of a head turn.  ``layout``: ``"interleaved"``
    (element 2i with 2i + 1) or ``"halves"`` (element i with i + dims/2)."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = frequencies(rot)
    f = torch.tensor(f, dtype=torch.float64).to(angle_dtype)
    ang = torch.as_tensor(positions).to(angle_dtype)[:, None] * f[None, :]
    cos = (torch.cos(ang).to(torch.float64) * mag).to(x.dtype)[:, None, :]
    sin = (torch.sin(ang).to(torch.float64) * mag).to(x.dtype)[:, None, :]
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


def sink_softmax(scores, seen, sink):
    """``scores``: [H, T, T]; ``seen``: bool [T, T]; ``sink``: [H] or None.  Softmax over the seen keys
    whose denominator also holds exp(sink_h), a member without key or value."""
    s = scores.masked_fill(~seen[None], float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def chunk_mask(T, size):
    i = torch.arange(T)
    return (i[None, :] <= i[:, None]) & ((i[None, :] // size) == (i[:, None] // size))


def causal_mask(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def talking_attention(h, W, cfg, eps, cache_round=None):
    """The left mixer: grouped heads, q/k norm per head before an interleaved partial rotation,
    ``score = q.k * scale * temp_h``, soft cap, scores mixed across heads, chunk mask, sink softmax."""
    T = h.shape[0]
    H, G, d, dv = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"]), int(cfg["vdim"])
    q = linear(h, W["q"]).reshape(T, H, d)
    k = linear(h, W["k"]).reshape(T, G, d)
    v = linear(h, W["v"]).reshape(T, G, dv)
    q, k = rms(q, eps) * W["q.norm"], rms(k, eps) * W["k.norm"]
    pos = list(range(T))
    if cfg.get("rot"):
        q, k = rotate(q, pos, cfg["rot"], "interleaved"), rotate(k, pos, cfg["rot"], "interleaved")
    if cache_round is not None:
        k, v = cache_round(k), cache_round(v)
    kh = k.repeat_interleave(H // G, dim=1)          # query head h uses key/value head h // (H/G)
    vh = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * float(cfg["scale"])
    if "temp" in W:
        s = s * W["temp"][:, None, None]
    cap = cfg.get("softcap")
    if cap:
        s = float(cap) * torch.tanh(s / float(cap))
    if "talk" in W:
        s = torch.einsum("hg,gij->hij", W["talk"], s)
    size = cfg.get("mask", {}).get("size")
    seen = chunk_mask(T, int(size)) if size else causal_mask(T)
    w = sink_softmax(s, seen, W.get("sink"))
    o = torch.einsum("hij,jhv->ihv", w, vh)
    return linear(o.reshape(T, H * dv), W["o"])


def causal_conv(u, w):
    """``u``: [T, C]; ``w``: [C, taps], the last column is the current token's; zeros before t = 0."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def unit(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta_rule(h, W, cfg, eps):
    """The right mixer.  Per head ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``."""
    T = h.shape[0]
    H, G, d, dv = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"]), int(cfg["vdim"])
    q, k, v = linear(h, W["q"]), linear(h, W["k"]), linear(h, W["v"])
    if cfg.get("conv"):
        q, k, v = causal_conv(q, W["q.conv"]), causal_conv(k, W["k.conv"]), causal_conv(v, W["v.conv"])
    q, k, v = silu(q).reshape(T, G, d), silu(k).reshape(T, G, d), silu(v).reshape(T, H, dv)
    q, k = unit(q) * d ** -0.5, unit(k)
    q, k = q.repeat_interleave(H // G, dim=1), k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(linear(h, W["b"]))                                        # [T, H]
    g = torch.exp(-torch.exp(W["A_log"]) * torch.nn.functional.softplus(linear(h, W["a"]) + W["dt_bias"]))
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    out = []
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = rms(torch.stack(out), eps) * W["norm"]                                     # per head over vdim
    o = o * silu(linear(h, W["g"])).reshape(T, H, dv)
    return linear(o.reshape(T, H * dv), W["o"])


def parallel_mixer(h, W, cfg, eps, cache_round=None):
    left = talking_attention(h, sub(W, "left."), cfg["left"], eps, cache_round)
    right = gated_delta_rule(h, sub(W, "right."), cfg["right"], eps)
    return 0.5 * (rms(left, eps) * W["left.out"] + rms(right, eps) * W["right.out"])


def latent_attention(h, W, cfg, eps, cache_round=None):
    T = h.shape[0]
    H, d, dr, dv, rank = int(cfg["heads"]), int(cfg["dim"]), int(cfg["rot_dim"]), int(cfg["vdim"]), int(cfg["kv_rank"])
    cq = rms(linear(h, W["dq"]), eps) * W["dq.norm"]
    q = linear(cq, W["uq"]).reshape(T, H, d + dr)
    dkv = linear(h, W["dkv"])
    c = rms(dkv[:, :rank], eps) * W["dkv.norm"]
    k_rot = dkv[:, rank:].reshape(T, 1, dr)
    pos = list(range(T))
    rot = dict(cfg["rot"], dims=dr)
    q_rot, k_rot = rotate(q[..., d:], pos, rot, "halves"), rotate(k_rot, pos, rot, "halves")
    if cache_round is not None:
        c, k_rot = cache_round(c), cache_round(k_rot)
    k_plain = linear(c, W["uk"]).reshape(T, H, d)
    v = linear(c, W["uv"]).reshape(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], k_plain)
         + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * float(cfg["scale"])
    w = sink_softmax(s, causal_mask(T), W.get("sink"))
    o = torch.einsum("hij,jhv->ihv", w, v).reshape(T, H * dv)
    if "g" in W:
        o = o * torch.sigmoid(linear(h, W["g"]))
    return linear(o, W["o"])


def gated_expert(h, gate, up, down):
    return linear(silu(linear(h, gate)) * linear(h, up), down)


def route(h, W, cfg):
    """Per token the chosen router outputs and their weights.  Scores are the softmax over all router
    outputs; the choice ranks ``score + correction`` among the outputs of the best groups (a group is
    worth its largest choice score; the others count as minus infinity); the weights are the chosen
    scores without the correction."""
    r = cfg["router"]
    n_all = int(r["experts"]) + int(r.get("identity", 0))
    top = int(r["top"])
    s = torch.softmax(linear(h, W["router"]), dim=-1)
    choice = s + W["correction"] if "correction" in W else s.clone()
    groups = r.get("groups")
    count, keep = (int(groups["count"]), int(groups["keep"])) if groups else (1, 1)
    per = n_all // count
    chosen, weights = [], []
    for t in range(h.shape[0]):
        worth = [max(float(choice[t, e]) for e in range(b * per, (b + 1) * per)) for b in range(count)]
        kept = sorted(range(count), key=lambda b: (-worth[b], b))[:keep]
        allowed = [e for b in sorted(kept) for e in range(b * per, (b + 1) * per)]
        order = sorted(allowed, key=lambda e: (-float(choice[t, e]), e))[:top]
        chosen.append(order)
        weights.append(s[t, order])
    return chosen, weights


def moe(h, W, cfg):
    chosen, weights = route(h, W, cfg)
    real = int(cfg["router"]["experts"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            if e >= real:                      # an identity expert: its output is its input
                out[t] += w * h[t]
            else:
                out[t] += w * gated_expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    return out


def feed_forward(h, W, cfg):
    if cfg["kind"] == "dense":
        return gated_expert(h, W["gate"], W["up"], W["down"])
    if cfg["kind"] == "moe":
        return moe(h, W, cfg)
    raise ValueError(f"mlp kind {cfg['kind']}")


def token_side(x, tokens, i, t, dim, eps):
    """The per-layer token input: layer i's slice of the token's row of the second table, gated by
    gelu_tanh of a projection of x, projected back, RMS-normed with a weight."""
    e = t["side.embed"][torch.as_tensor(tokens, dtype=torch.long)][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(linear(x, t[f"l{i}.side.gate"])) * e
    y = linear(g, t[f"l{i}.side.proj"])
    return rms(y, eps) * t[f"l{i}.side.norm"]


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, dtype=DT, cache_round=None, streams=None, read_round=None):
    """Logits ``[T, vocab]`` of one whole sequence.  ``cache_round``: what storing a row in the cache
    does to it; ``read_round``: what a sublayer's reading of the stream does to it (identity if None).
    ``streams``: a list that receives the residual stream after every layer."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    side = config.get("token_side")
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)].clone()
    read = read_round or (lambda a: a)
    for i, layer in enumerate(config["layers"]):
        W = sub(t, f"l{i}.mix.")
        if layer["type"] == "parallel":
            y = parallel_mixer(read(x), W, layer["mixer"], eps, cache_round)
        elif layer["type"] == "latent_attention":
            y = latent_attention(read(x), W, layer["mixer"], eps, cache_round)
        else:
            raise ValueError(f"mixer type {layer['type']}")
        x = x + rms(y, eps) * t[f"l{i}.norm1"]
        if layer.get("mlp"):
            y = feed_forward(read(x), sub(t, f"l{i}.mlp."), layer["mlp"])
            x = x + rms(y, eps) * t[f"l{i}.norm2"]
        if side:
            x = x + token_side(read(x), tokens, i, t, int(side["dim"]), eps)
        if streams is not None:
            streams.append(x.clone())
    return linear(rms(x, eps) * t["final.norm"], t["embed"])


class PlainZiginex:
    def __init__(self, cfg, tensors, dtype=DT, cache_round=None, read_round=None):
        self.cfg, self.tensors, self.dtype = cfg, tensors, dtype
        self.cache_round, self.read_round = cache_round, read_round
        self._memo = {}

    def logits(self, tokens):
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = forward(self.cfg, self.tensors, list(tokens), self.dtype, self.cache_round,
                                      read_round=self.read_round)
        return self._memo[key]

    def residuals(self, tokens):
        streams = []
        forward(self.cfg, self.tensors, list(tokens), self.dtype, self.cache_round, streams, self.read_round)
        return torch.stack(streams)
