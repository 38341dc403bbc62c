"""Tiny Sakinex configurations for the tests, and random weights for them.

They differ from one another in every size and option, and avoid coincidences: key and value widths
differ, rotated dimensions are not all rotated, windows and pooled blocks are no multiples of the page
sizes (a block larger than a page, a block that does not divide a page, a window shorter than a block,
a window and a block of 1), the convolutions have different numbers of taps or are absent, the looped
span starts at layer 0 or later, a model has no loop, a rotation has no YaRN scaling, a layer has no
feed-forward and one has no shared expert, heads share key/value heads in different ratios."""
import torch

from leone_b200.engine.model import weight_specs_for_config
from leone_b200.registry import config_from_dict
from leone_b200.weights.random_init import random_tensors


def left(heads, kv_heads, dim, vdim, scale, size, pool, conv=None, rot_dims=None, base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": size, "pool": pool}}
    if conv:
        m["conv"] = conv
    if rot_dims != 0:
        m["rot"] = {"base": base, "dims": dim if rot_dims is None else rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def mixer(left_part, right_width, left_scale=1.0, right_scale=1.0):
    return {"left": left_part, "right": {"width": right_width}, "left_scale": left_scale, "right_scale": right_scale}


def moe(ff, experts, top, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(m, mlp):
    return {"type": "parallel", "mixer": m, "mlp": mlp}


def model(vocab, width, eps, mult, layers, canon=None, loop=None):
    raw = {"architecture": "Sakinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
           "layers": layers}
    if canon:
        raw["canon"] = {"taps": canon}
    if loop:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    return raw


TINY = {
    # a loop over the first two layers (three passes), window 9 and blocks of 3 over pages of 4 (a block does not
    # divide a page), window 5 with blocks of 7 (a block longer than the window and than a page)
    "A": model(97, 64, 1e-5, 0.6, canon=3, loop=(0, 2, 3), layers=[
        layer(mixer(left(6, 2, 16, 24, 0.2, 9, 3, conv=4, rot_dims=8, base=500.0, scaling=(4.0, 32, 8.0, 1.0)), 40, 0.8, 1.1),
              moe(48, 6, 2, shared=32)),
        layer(mixer(left(4, 4, 24, 16, 0.15, 5, 7, conv=2, rot_dims=24), 72, 1.2, 0.7), moe(32, 4, 3)),
        layer(mixer(left(3, 1, 16, 40, 0.25, 20, 4, conv=3, rot_dims=4, scaling=(16.0, 64, 4.0, 0.5)), 64, 0.9, 0.9), None),
        layer(mixer(left(2, 2, 32, 8, 0.1, 12, 6, rot_dims=32, base=100000.0), 24, 1.0, 1.0), moe(24, 5, 1, shared=40))]),
    # a loop in the middle over one layer, sizes that are no multiple of 8, a window of 1 and blocks of 1, no
    # rotation in one layer, pages of 8
    "B": model(131, 72, 3e-6, 0.9, canon=2, loop=(1, 2, 2), layers=[
        layer(mixer(left(1, 1, 20, 28, 0.3, 1, 1, conv=5, rot_dims=12, scaling=(2.0, 16, 2.0, 1.0)), 36, 1.0, 0.5),
              moe(36, 3, 1, shared=20)),
        layer(mixer(left(5, 5, 12, 10, 0.35, 500, 3, conv=4, rot_dims=6, base=100.0), 100, 0.5, 1.5), moe(28, 7, 7, shared=12)),
        layer(mixer(left(2, 1, 36, 36, 0.2, 3, 5, conv=1, rot_dims=0), 60, 1.0, 1.0), moe(60, 2, 2)),
        layer(mixer(left(3, 3, 8, 8, 0.4, 7, 2, rot_dims=2), 8, 0.7, 1.3), None)]),
    # no loop and no convolution in front of the sublayers; head sizes the tensor-core forms take (64, 128, 32), a
    # window of 32 with blocks of 16 over pages of 16, eight query heads on one key/value head
    "C": model(256, 128, 1e-6, 1.0, layers=[
        layer(mixer(left(4, 2, 64, 64, 0.125, 40, 8, conv=4, base=30000.0, scaling=(6.0, 64, 24.0, 1.0)), 128, 0.8, 0.9),
              moe(64, 8, 2, shared=96)),
        layer(mixer(left(8, 1, 32, 64, 0.18, 32, 16, conv=4, rot_dims=16), 256, 1.0, 1.0), moe(32, 12, 4, shared=64)),
        layer(mixer(left(4, 2, 128, 32, 0.09, 48, 32, conv=3, rot_dims=64, scaling=(4.0, 128, 16.0, 2.0)), 64, 1.1, 0.6),
              moe(128, 4, 2)),
        layer(mixer(left(2, 2, 48, 80, 0.14, 17, 5, conv=4, rot_dims=48), 96, 0.9, 1.0), moe(16, 16, 3, shared=16))]),
    # the whole model looped twice; 18 query heads, wide heads, pages of 32
    "D": model(200, 96, 2e-6, 0.5, canon=4, loop=(0, 3, 2), layers=[
        layer(mixer(left(18, 6, 16, 16, 0.2, 70, 10, conv=4, rot_dims=8, base=1000.0), 96, 1.0, 1.0), None),
        layer(mixer(left(2, 1, 144, 48, 0.08, 33, 33, conv=2, rot_dims=100, scaling=(32.0, 40, 8.0, 1.0)), 48, 0.8, 1.2),
              moe(24, 6, 6, shared=8)),
        layer(mixer(left(5, 5, 32, 32, 0.17, 64, 32, conv=6, rot_dims=16), 200, 1.3, 0.4), moe(64, 9, 2, shared=24))]),
}
PAGE_TOKENS = {"A": 4, "B": 8, "C": 16, "D": 32}


def tiny_config(which):
    return config_from_dict(TINY[which])


def tiny_tensors(which, seed=5, gain=4.0, raw=None):
    """fp32 random tensors; matrices are scaled up so that scores, gates and routers are far from
    uniform and every mechanism matters to the logits."""
    specs = weight_specs_for_config(config_from_dict(raw) if raw is not None else tiny_config(which))
    tensors = random_tensors(specs, seed)
    for name, t in tensors.items():
        if name == "embed":
            tensors[name] = t * 40.0
        elif name.endswith(".conv") or ".canon" in name:
            tensors[name] = t * 2.0
        elif t.dim() == 2:
            tensors[name] = t * gain
    return tensors


def as_bf16(tensors):
    return {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
