"""The Ziginex decoder as a :class:`ModelSpec`.

Every layer is the ``post_norm`` arrangement: a sublayer reads the residual stream itself and its
output is RMS-normed (``norm1`` / ``norm2``) before it is added; after the feed-forward comes the
layer's ``token_gate``, which gates its slice of the token's row of a second table (``side.embed``,
gathered by the embedding part) with a projection of the stream and adds the normed result.

Mixer type ``parallel`` is ``side_by_side`` with the normed mean: ``attention`` (per-head q/k norm, a
partial rotation of adjacent pairs, a temperature per head, a soft cap, scores mixed across the heads, a
chunk mask, a sink) and ``gated_delta_rule``.  Mixer type ``latent_attention`` is the part of that name
with a query latent, YaRN frequencies on a half-split rotation, a sink and an elementwise output gate.
The feed-forward is ``swiglu`` or ``routed_experts`` (softmax scores, a correction for the choice,
groups, identity experts, weights as they are, at the experts' outputs).  The head is tied.

Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.left.q|k|v|o|q.norm|k.norm|
talk|temp|sink|out``, ``l<i>.mix.right.q|k|v|q.conv|k.conv|v.conv|b|a|A_log|dt_bias|norm|g|o|out``,
``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|sink|g|o``, ``l<i>.mlp.gate|up|down``,
``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.router|correction``, ``l<i>.side.gate|proj|norm``,
``final.norm``.
"""
from __future__ import annotations

from ..config.ziginex import DenseMlp, ZiginexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec
from ..registry import ARCHITECTURES

SIDE_TABLE = "side.embed"


def build_spec(cfg: ZiginexConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms_norm", {"size": width, "eps": eps})
    encodings = {}

    def encoding_for(dims, base, pairing, scaling):
        if not dims:
            return None
        params = {"rotary_dim": dims, "base": base, "pairing": pairing,
                  "scaling": None if scaling is None else scaling.to_json()}
        for name, ps in encodings.items():
            if ps.params == params:
                return name
        name = f"rot{len(encodings)}"
        encodings[name] = PartSpec("rotary_computed", params)
        return name

    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "parallel":
            lf, rg = m.left, m.right
            left = {"hidden_size": width, "num_heads": lf.heads, "num_kv_heads": lf.kv_heads, "head_dim": lf.dim,
                    "value_head_dim": lf.vdim, "scale": lf.scale, "qk_norm": True, "qk_norm_eps": eps,
                    "mask": "chunk" if lf.chunk else "causal", "chunk": lf.chunk or None,
                    "position_encoding": encoding_for(lf.rot_dims, lf.rot_base, "adjacent", None),
                    "score_cap": lf.softcap or None, "head_temp_name": "mix.left.temp", "head_mix_name": "mix.left.talk",
                    "sink_name": "mix.left.sink", "q_name": "mix.left.q", "k_name": "mix.left.k", "v_name": "mix.left.v",
                    "o_name": "mix.left.o", "q_norm_name": "mix.left.q.norm", "k_norm_name": "mix.left.k.norm"}
            right = {"hidden_size": width, "heads": rg.heads, "kv_heads": rg.kv_heads, "dim": rg.dim, "vdim": rg.vdim,
                     "conv_taps": rg.conv, "norm_eps": eps,
                     **{f"{k}_name": f"mix.right.{k}" for k in ("q", "k", "v", "g", "a", "b", "o", "norm", "A_log", "dt_bias")}}
            mixer = PartSpec("side_by_side", {"combine": "normed_mean", "hidden_size": width, "norm_eps": eps, "branches": [
                {"name": "left", "kind": "attention", "params": left, "norm_name": "mix.left.out"},
                {"name": "right", "kind": "gated_delta_rule", "params": right, "norm_name": "mix.right.out"}]})
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "window": None, "eps": eps, "sink": True,
                "gate": "elementwise",
                "position_encoding": encoding_for(m.rot_dims, m.rot_base, "half_split", m.rot_scaling),
                "dq_name": "mix.dq", "dq_norm_name": "mix.dq.norm", "uq_name": "mix.uq", "dkv_name": "mix.dkv",
                "dkv_norm_name": "mix.dkv.norm", "uk_name": "mix.uk", "uv_name": "mix.uv", "sink_name": "mix.sink",
                "g_name": "mix.g", "o_name": "mix.o"})
        f = layer.mlp
        if f is None:
            ffn = None
        elif isinstance(f, DenseMlp):
            ffn = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": f.ff, "gate_name": "mlp.gate",
                                      "up_name": "mlp.up", "down_name": "mlp.down"})
        else:
            ffn = PartSpec("routed_experts", {
                "hidden_size": width, "expert_size": f.expert_ff, "num_experts": f.experts, "top": f.top,
                "identity": f.identity, "score": "softmax", "renormalize": False, "scale": "output",
                "groups": f.groups, "groups_kept": f.groups_kept, "router_name": "mlp.router",
                "correction_name": "mlp.correction", "expert_pattern": "mlp.e{}.{}"})
        extra = {}
        if cfg.side_dim:
            extra["after"] = ("feed_forward", PartSpec("token_gate", {
                "hidden_size": width, "dim": cfg.side_dim, "offset": i * cfg.side_dim, "table": SIDE_TABLE,
                "norm_eps": eps, "gate_name": "side.gate", "proj_name": "side.proj", "norm_name": "side.norm"}))
        layers.append(LayerSpec(
            prefix=f"l{i}", block="post_norm", mixer=mixer, feed_forward=ffn,
            mixer_norm=PartSpec(norm.kind, {**norm.params, "name": "norm1"}),
            ffn_norm=None if ffn is None else PartSpec(norm.kind, {**norm.params, "name": "norm2"}), extra=extra))
    embedding = {"name": "embed"}
    if cfg.side_dim:
        embedding["side_tables"] = [{"name": SIDE_TABLE, "width": cfg.side_dim * len(cfg.layers)}]
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding_name="embed", layers=tuple(layers), run_order=tuple(range(len(layers))), final_norm=norm,
        final_norm_name="final.norm", lm_head_name=None, position_encodings=encodings,
        embedding=PartSpec("token_embedding", embedding), head=PartSpec("linear_head", {"name": None}))
    spec.validate()
    return spec


ARCHITECTURES.add(ZiginexConfig.ARCHITECTURE, ZiginexConfig, build_spec)
