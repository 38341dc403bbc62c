"""The Sakinex decoder as a :class:`ModelSpec`.

Every layer is the ``pre_norm_conv`` arrangement: what the mixer and the feed-forward read passes
through a short causal convolution over time that is added to its input (``short_conv`` with
``add_input``).  A sublayer's output enters the residual stream times ``residual_mult``; the
multiplier is handed to the parts as their output scale.  A span of layers may run several times in
a row with the same weights (each run owns its caches and states); before every pass but the first
the ``add_origin`` injection adds the embedding's rows to the stream.

The mixer is ``side_by_side``: ``pooled_window_attention`` (a convolution on the projected q, k and
v, a partial half-split rotation with YaRN frequencies whose angles the kernel forms in fp32, a
unit RMS norm of q and k per head after the rotation, a sliding window with one mean key and value
per block of positions before it) and ``min_gru``, each with its own scale.  The feed-forward is
``routed_experts``: the largest router logits (with a bias) choose, the weights are the softmax over
the chosen logits, and a shared expert is multiplied by a per-token sigmoid gate.

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.canon1|canon2``, ``l<i>.mix.left.q|k|v|o``,
``l<i>.mix.left.q|k|v.conv``, ``l<i>.mix.right.z|x|g|o``, ``l<i>.mix.right.z.b|x.b``,
``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.router``, ``l<i>.mlp.router.b``,
``l<i>.mlp.shared.gate|up|down|sg``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.sakinex import SakinexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec
from ..registry import ARCHITECTURES


def build_spec(cfg: SakinexConfig) -> ModelSpec:
    width, eps, mult = cfg.width, cfg.norm_eps, cfg.residual_mult
    norm = PartSpec("rms_norm", {"size": width, "eps": eps})
    encodings = {}

    def encoding_for(left):
        if not left.rot_dims:
            return None
        scaling = None if left.rot_scaling is None else left.rot_scaling.to_json()
        params = {"rotary_dim": left.rot_dims, "base": left.rot_base, "pairing": "half_split", "scaling": scaling}
        for name, ps in encodings.items():
            if ps.params == params:
                return name
        name = f"rot{len(encodings)}"
        encodings[name] = PartSpec("rotary_computed", params)
        return name

    def canon(name):
        return ("conv", PartSpec("short_conv", {"channels": width, "taps": cfg.canon_taps, "add_input": True, "name": name}))

    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        left = {"hidden_size": width, "num_heads": m.left.heads, "num_kv_heads": m.left.kv_heads, "head_dim": m.left.dim,
                "value_head_dim": m.left.vdim, "scale": m.left.scale, "window": m.left.mask_size, "pool": m.left.mask_pool,
                "conv_taps": m.left.conv, "position_encoding": encoding_for(m.left), "unit_norm": True, "norm_eps": eps,
                "out_scale": mult * m.left_scale, "q_name": "mix.left.q", "k_name": "mix.left.k", "v_name": "mix.left.v",
                "o_name": "mix.left.o"}
        right = {"hidden_size": width, "width": m.right_width, "out_scale": mult * m.right_scale,
                 "z_name": "mix.right.z", "x_name": "mix.right.x", "g_name": "mix.right.g", "o_name": "mix.right.o",
                 "z_bias_name": "mix.right.z.b", "x_bias_name": "mix.right.x.b"}
        mixer = PartSpec("side_by_side", {"branches": [
            {"name": "left", "kind": "pooled_window_attention", "params": left},
            {"name": "right", "kind": "min_gru", "params": right}]})
        f = layer.mlp
        ffn = None
        if f is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": width, "expert_size": f.expert_ff, "num_experts": f.experts, "top": f.top,
                "score": "softmax_chosen", "scale": "output", "out_scale": mult, "shared_size": f.shared_ff or None,
                "router_name": "mlp.router", "router_bias_name": "mlp.router.b", "expert_pattern": "mlp.e{}.{}",
                "shared_pattern": "mlp.shared.{}", "shared_gate_name": "mlp.shared.sg" if f.shared_ff else None})
        extra = {}
        if cfg.canon_taps:
            extra["mixer_conv"] = canon("canon1")
            if ffn is not None:
                extra["ffn_conv"] = canon("canon2")
        layers.append(LayerSpec(
            prefix=f"l{i}", block="pre_norm_conv", mixer=mixer, feed_forward=ffn,
            mixer_norm=PartSpec(norm.kind, {**norm.params, "name": "norm1"}),
            ffn_norm=None if ffn is None else PartSpec(norm.kind, {**norm.params, "name": "norm2"}), extra=extra))
    again = PartSpec("add_origin", {"scale": 1.0})
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding_name="embed", layers=tuple(layers), run_order=cfg.run_order(), final_norm=norm,
        final_norm_name="final.norm", lm_head_name="head", position_encodings=encodings,
        embedding=PartSpec("token_embedding", {"name": "embed"}), head=PartSpec("linear_head", {"name": "head"}),
        injections=tuple((pos, again) for pos in cfg.later_pass_starts()))
    spec.validate()
    return spec


ARCHITECTURES.add(SakinexConfig.ARCHITECTURE, SakinexConfig, build_spec)
