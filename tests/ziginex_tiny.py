"""Tiny Ziginex configurations for the tests, and random weights for them.

They differ from one another in every size and option, and avoid coincidences: key and value widths
differ, query heads share key/value heads in different ratios (also one to one, also all on one), the
two mixers of a parallel layer have different head counts and sizes, rotated dimensions are not all
rotated (or none), chunks are no multiples of the page sizes (a chunk of 1, a chunk longer than any
prompt, no chunk at all), the convolutions have 1 to 6 taps or are absent, latents are narrower and
wider than the heads they feed, the rotated part is wider and narrower than the unrotated one, routers
have identity experts or none, groups or none, every output chosen or one, a layer has no
feed-forward, a model has no token table of its own, layers come in every order."""
import torch

from leone_b200.engine.model import weight_specs_for_config
from leone_b200.registry import config_from_dict
from leone_b200.weights.random_init import random_tensors


def left(heads, kv_heads, dim, vdim, scale, chunk=None, softcap=None, rot_dims=None, base=10000.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if softcap:
        m["softcap"] = softcap
    if rot_dims != 0:
        m["rot"] = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    return m


def right(heads, kv_heads, dim, vdim, conv=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim}
    if conv:
        m["conv"] = conv
    return m


def parallel(left_part, right_part, mlp=None):
    return {"type": "parallel", "mixer": {"left": left_part, "right": right_part}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, scaling=None, mlp=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": rot}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, identity=0, groups=None):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def model(vocab, width, eps, layers, side=None):
    raw = {"architecture": "Ziginex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        raw["token_side"] = {"dim": side}
    return raw


TINY = {
    # chunks of 9 and 5 over pages of 4; a latent layer in the middle and at the end; identity experts in groups
    "A": model(97, 64, 1e-5, side=6, layers=[
        parallel(left(6, 2, 16, 24, 0.2, chunk=9, softcap=12.0, rot_dims=8, base=500.0), right(4, 2, 12, 20, conv=3), dense(48)),
        latent(3, 8, 12, 10, 24, 20, 0.3, base=1000.0, scaling=(4.0, 32, 8.0, 1.0), mlp=moe(24, 5, 2, identity=3, groups=(4, 2))),
        parallel(left(4, 4, 24, 16, 0.15, chunk=5, rot_dims=24), right(2, 1, 20, 8, conv=2), None),
        latent(2, 16, 4, 24, 12, 40, 0.25, base=50000.0, mlp=dense(40))]),
    # sizes that are no multiple of 8, a chunk of 1, one head, every router output chosen, pages of 8
    "B": model(131, 72, 3e-6, side=5, layers=[
        latent(5, 12, 6, 10, 20, 36, 0.35, base=100.0, scaling=(2.0, 16, 2.0, 1.0), mlp=moe(28, 4, 7, identity=3)),
        parallel(left(1, 1, 20, 28, 0.3, chunk=1, softcap=5.0, rot_dims=12), right(1, 1, 36, 12, conv=5), moe(36, 3, 1)),
        parallel(left(5, 5, 12, 10, 0.35, chunk=500, rot_dims=0), right(6, 3, 10, 14, conv=1), dense(60)),
        parallel(left(3, 1, 8, 8, 0.4, chunk=7, softcap=50.0, rot_dims=2), right(3, 3, 8, 8), None)]),
    # head sizes of real models (64, 128, 32), a chunk of 40 over pages of 16, eight query heads on one key/value head
    "C": model(256, 128, 1e-6, side=8, layers=[
        parallel(left(4, 2, 64, 64, 0.125, chunk=40, softcap=30.0, rot_dims=32, base=30000.0), right(4, 2, 64, 64, conv=4),
                 moe(64, 12, 3, identity=4, groups=(4, 3))),
        parallel(left(8, 1, 32, 64, 0.18, chunk=32, softcap=20.0, rot_dims=16), right(2, 1, 128, 128, conv=4), dense(256)),
        latent(4, 32, 32, 64, 64, 48, 0.12, base=200000.0, scaling=(8.0, 128, 16.0, 2.0), mlp=moe(32, 6, 2, groups=(3, 1))),
        parallel(left(2, 2, 128, 32, 0.09, chunk=48, rot_dims=64), right(8, 2, 32, 32, conv=3), moe(16, 14, 4, identity=2))]),
    # no token table of its own, a latent layer first, 18 query heads, wide recurrent heads (the forms of the
    # recurrence's kernel for up to 256 and up to 512 rows), no chunk and no cap in one layer, pages of 32
    "D": model(200, 96, 2e-6, layers=[
        latent(6, 24, 16, 16, 40, 32, 0.2, base=1000.0, scaling=(32.0, 40, 8.0, 1.0), mlp=None),
        parallel(left(18, 6, 16, 16, 0.2, chunk=70, softcap=8.0, rot_dims=8, base=1000.0), right(2, 1, 144, 24, conv=6), dense(64)),
        parallel(left(2, 1, 48, 80, 0.08, rot_dims=20), right(1, 1, 300, 40, conv=2), moe(24, 6, 6, identity=2, groups=(2, 2)))]),
}
PAGE_TOKENS = {"A": 4, "B": 8, "C": 16, "D": 32}


def tiny_config(which):
    return config_from_dict(TINY[which])


def tiny_tensors(which, seed=5, gain=4.0, raw=None):
    """fp32 random tensors; matrices are scaled up so that scores, gates and routers are far from
    uniform and every mechanism matters to the logits; the matrix that mixes the heads' scores is
    the identity plus noise."""
    specs = weight_specs_for_config(config_from_dict(raw) if raw is not None else tiny_config(which))
    tensors = random_tensors(specs, seed)
    for name, t in tensors.items():
        if name in ("embed", "side.embed"):
            tensors[name] = t * 30.0
        elif name.endswith(".talk"):
            tensors[name] = t + torch.eye(t.shape[0])
        elif name.endswith(".conv"):
            tensors[name] = t * 2.0
        elif name.endswith(".router"):
            tensors[name] = t * 2.0 * gain
        elif t.dim() == 2:
            tensors[name] = t * gain
    return tensors


def as_bf16(tensors):
    return {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
