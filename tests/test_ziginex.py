"""The Ziginex decoder through the engine against the plain implementation (tests/plain/ziginex.py).

Without a GPU the engine runs on the stand-in kernels (tests/emulated_ops.py), which checks the
configuration, the model description, the post-norm arrangement, the bundles of caches and states, and
the step function's cutting and batching; on a B200 the same traces run on the CUDA kernels in 32-bit
and in bfloat16, together with tests that aim at single mechanisms."""
import copy
import math
import os

import numpy as np
import pytest
import torch

from leone_b200.engine.engine import Engine
from leone_b200.registry import config_from_dict, spec_from_config
from tests import replay
from tests.plain import ziginex as plain
from tests.ziginex_tiny import (PAGE_TOKENS, TINY, as_bf16, dense, latent, left, model, moe, parallel, right, tiny_config,
                                tiny_tensors)

FP32 = dict(rtol=3e-5, atol_scale=3e-5)
# bfloat16: the gained weights make scores, gates and routers sharp, which also amplifies rounding; the
# 32-bit runs are the sharp tests, these catch a wrong path or operand
BF16 = dict(rtol=1e-1, atol_scale=1e-1)
LENGTHS = [40, 7, 75, 33, 1, 64, 50]


def _bf16_round(t):
    return t.to(torch.bfloat16).to(t.dtype)


def _plain(which, tensors, bf16=False, raw=None):
    """In bfloat16 the plain model has the same stored weights and rounds what the cache holds and what
    the sublayers read of the stream."""
    return plain.PlainZiginex(raw or TINY[which], as_bf16(tensors) if bf16 else tensors,
                              cache_round=_bf16_round if bf16 else None, read_round=_bf16_round if bf16 else None)


def _engine(which, tensors, dtype, device, ops=None, max_tokens=512, page=None, raw=None, **kw):
    spec = spec_from_config(config_from_dict(raw) if raw is not None else tiny_config(which))
    return Engine(spec, dict(tensors), dtype=dtype, device=device, ops=ops, page_tokens=page or PAGE_TOKENS[which],
                  max_tokens=max_tokens, max_requests=kw.pop("max_requests", 4),
                  max_batch_tokens=kw.pop("max_batch_tokens", 128), **kw)


def _requests(vocab, lengths=LENGTHS, seed=100):
    return {f"r{i}": replay.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


def _without_routers(raw):
    """The same model with every mixture of experts replaced by a dense layer: in bfloat16 a router's close
    call chooses another expert than the plain model's, and every later position reads the difference;
    without routers the bfloat16 runs can be held to a bound row by row."""
    raw = copy.deepcopy(raw)
    for entry in raw["layers"]:
        if entry["mlp"] and entry["mlp"]["kind"] == "moe":
            entry["mlp"] = dense(2 * entry["mlp"]["expert"]["ff"])
    return raw


def _compare_bf16_with_routers(steps, out, oracle, reqs, what):
    """With routers in bfloat16: most rows agree closely, and nothing is far off everywhere."""
    pos = {rid: 0 for rid in reqs}
    errs = []
    for st in steps:
        rows = []
        for e in st["entries"]:
            full = oracle.logits(reqs[e["id"]])
            rows += [full[pos[e["id"]] + w] for w in e["want"]]
            pos[e["id"]] += len(e["tokens"])
        if rows:
            want = torch.stack(rows).double().numpy()
            got = np.asarray(out[st["step"]], dtype=np.float64).reshape(want.shape)
            errs += list(np.abs(got - want).max(axis=1) / np.abs(want).max())
    errs = np.sort(np.asarray(errs))
    assert errs[len(errs) // 2] < 0.03 and errs[int(len(errs) * 0.7)] < 0.1, (what, errs[len(errs) // 2], errs[int(len(errs) * 0.7)])


def _traces(reqs):
    return {"whole": replay.trace_whole(reqs), "tail": replay.trace_decode_tail(reqs, tail=20),
            "portions": replay.trace_portions(reqs), "mixed": replay.trace_mixed(reqs, seed=3)}


def _random(raw, seed, gain=4.0):
    return tiny_tensors(None, seed=seed, gain=gain, raw=raw)


def _one_layer(entry, vocab=64, width=32, eps=1e-6, side=None):
    return model(vocab, width, eps, [entry], side=side)


# -- configuration and description (CPU) ---------------------------------------------------------
def test_config_round_trip_and_spec():
    for which, raw in TINY.items():
        cfg = config_from_dict(raw)
        assert cfg.to_json_dict() == raw
        spec = spec_from_config(cfg)
        assert all(ls.block == "post_norm" for ls in spec.layers) and spec.lm_head_name is None
        assert [ls.mixer.kind for ls in spec.layers] == \
            ["side_by_side" if e["type"] == "parallel" else "latent_attention" for e in raw["layers"]]
        assert [ls.feed_forward is None for ls in spec.layers] == [e["mlp"] is None for e in raw["layers"]]
        assert all(("after" in ls.extra) == ("token_side" in raw) for ls in spec.layers)


def test_config_rejections():
    from leone_b200.config.base import ConfigError
    for patch in (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4),
                  lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=3),
                  lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18),
                  lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0),
                  lambda c: c["layers"][0]["mixer"].pop("right"),
                  lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=3),
                  lambda c: c["layers"][0].update(type="conv"),
                  lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8),
                  lambda c: c["layers"][1]["mixer"].pop("kv_rank"),
                  lambda c: c["layers"][1]["mlp"]["router"].update(top=5),
                  lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3),
                  lambda c: c["layers"][1]["mlp"].update(kind="sparse"),
                  lambda c: c["token_side"].update(dim=0),
                  lambda c: c.pop("width"), lambda c: c.update(layers=[])):
        raw = copy.deepcopy(TINY["A"])
        patch(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)


# -- the plain implementation's own mechanisms, against their definitions (CPU) -----------------------
def test_plain_chunks_and_sink():
    """Values that name their position: with all scores equal and a sink of the same score, the output
    is the sum of what is seen over (count + 1)."""
    T, size = 14, 4
    W = {"q": torch.zeros(2, 2, dtype=torch.float64), "k": torch.zeros(2, 2, dtype=torch.float64),
         "v": torch.tensor([[1.0, 0.0]], dtype=torch.float64), "o": torch.eye(1, dtype=torch.float64),
         "q.norm": torch.ones(2, dtype=torch.float64), "k.norm": torch.ones(2, dtype=torch.float64),
         "sink": torch.zeros(1, dtype=torch.float64)}
    h = torch.stack([torch.arange(T, dtype=torch.float64), torch.ones(T, dtype=torch.float64)], dim=1)
    cfg = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0, "mask": {"size": size}}
    out = plain.talking_attention(h, W, cfg, 1e-6)[:, 0]
    for i in range(T):
        seen = list(range((i // size) * size, i + 1))
        assert abs(float(out[i]) - sum(seen) / (len(seen) + 1)) < 1e-12, i
    assert plain.chunk_mask(6, 3).int().tolist() == [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0],
                                                       [0, 0, 0, 1, 0, 0], [0, 0, 0, 1, 1, 0], [0, 0, 0, 1, 1, 1]]


def test_plain_delta_rule_by_hand():
    """One head of one key dimension: the state is a row of values, k = 1 after the unit norm."""
    W = {"q": torch.tensor([[1.0]]), "k": torch.tensor([[1.0]]), "v": torch.eye(2), "b": torch.zeros(1, 1),
         "a": torch.zeros(1, 1), "A_log": torch.zeros(1), "dt_bias": torch.zeros(1), "norm": torch.ones(2),
         "g": torch.zeros(2, 1), "o": torch.eye(2)}
    W = {k: v.double() for k, v in W.items()}
    # g = exp(-softplus(0)) = 1/2, beta = 1/2; q, k = silu(h) normed to 1 (q times dim^-1/2 = 1)
    h = torch.tensor([[3.0], [3.0]], dtype=torch.float64)
    cfg = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 2}
    v = plain.silu(h @ W["v"].t().new_ones(1, 2))            # both value channels read h
    W["v"] = torch.ones(2, 1, dtype=torch.float64)
    S1 = 0.5 * v[0]
    S2 = 0.5 * S1 + 0.5 * (v[1] - 0.5 * S1)
    want = torch.stack([S1, S2])
    W["g"] = torch.zeros(2, 1, dtype=torch.float64)
    out = plain.gated_delta_rule(h, W, cfg, 1e-6)
    # the gate silu(0) = 0 would hide everything: look at the read-out before the gate instead
    assert float(out.abs().max()) == 0.0
    W["g"] = torch.full((2, 1), 10.0, dtype=torch.float64)    # silu(30) = 30 for all purposes
    out = plain.gated_delta_rule(h, W, cfg, 0.0)
    assert torch.allclose(out, plain.rms(want, 0.0) * plain.silu(torch.tensor(30.0, dtype=torch.float64)), atol=1e-9)


def test_plain_router_groups_correction_and_identity():
    z = torch.log(torch.tensor([[0.05, 0.30, 0.10, 0.15, 0.25, 0.15]], dtype=torch.float64))
    W = {"router": torch.eye(6, dtype=torch.float64),
         "correction": torch.tensor([0.0, -0.2, 0.0, 0.0, 0.0, 0.12], dtype=torch.float64)}
    # choice scores 0.05 0.10 | 0.10 0.15 | 0.25 0.27: groups worth 0.10, 0.15, 0.27; the best two are kept
    cfg = {"router": {"experts": 4, "identity": 2, "top": 3, "groups": {"count": 3, "keep": 2}}}
    chosen, weights = plain.route(z, W, cfg)
    assert chosen == [[5, 4, 3]]
    assert torch.allclose(weights[0], torch.tensor([0.15, 0.25, 0.15], dtype=torch.float64))
    # an identity expert gives its input back: with every weight on output 5 the layer is w * h
    h = torch.tensor([[1.0, -2.0, 0.5, 0.0, 3.0, 7.0]], dtype=torch.float64)
    Wm = {"router": torch.eye(6, dtype=torch.float64) * 0, "correction": torch.tensor([0, 0, 0, 0, 0, 1.0]).double()}
    Wm["router"][5] = 0.0
    out = plain.moe(h, Wm, {"router": {"experts": 5, "identity": 1, "top": 1}})
    assert torch.allclose(out, h / 6)


def test_plain_rotation_layouts_and_gelu():
    x = torch.arange(1.0, 7.0, dtype=torch.float64).view(1, 1, 6)
    rot = {"base": 100.0, "dims": 4}
    a = [2.0 * 100.0 ** (-2.0 * i / 4) for i in range(2)]
    inter = plain.rotate(x, [2], rot, "interleaved", torch.float64)[0, 0]
    halves = plain.rotate(x, [2], rot, "halves", torch.float64)[0, 0]
    assert abs(float(inter[0]) - (1 * math.cos(a[0]) - 2 * math.sin(a[0]))) < 1e-12
    assert abs(float(inter[3]) - (4 * math.cos(a[1]) + 3 * math.sin(a[1]))) < 1e-12
    assert abs(float(halves[0]) - (1 * math.cos(a[0]) - 3 * math.sin(a[0]))) < 1e-12
    assert abs(float(halves[3]) - (4 * math.cos(a[1]) + 2 * math.sin(a[1]))) < 1e-12
    assert inter[4:].tolist() == [5.0, 6.0] and halves[4:].tolist() == [5.0, 6.0]
    z = torch.tensor([0.7], dtype=torch.float64)
    assert abs(float(plain.gelu_tanh(z)) - 0.35 * (1 + math.tanh(math.sqrt(2 / math.pi) * (0.7 + 0.044715 * 0.343)))) < 1e-15


# -- the step function on stand-in kernels (CPU) ------------------------------------------------
@pytest.mark.parametrize("which", ["A", "B", "D"])
@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_replay_on_stand_in_kernels(which, mode):
    from tests.emulated_ops import EmulatedOps
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"], [23, 7, 30, 1, 12], seed=300)
    steps = _traces(reqs)[mode]
    eng = _engine(which, tensors, "float32", "cpu", EmulatedOps(), max_tokens=replay.max_live_tokens(steps))
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain(which, tensors), reqs, what=f"{which} {mode} stand-in", rtol=2e-5, atol_scale=2e-5)
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


def test_residual_stream_after_every_layer_on_stand_in_kernels():
    """The stream after each layer, read from the engine's buffer by a hook on the blocks."""
    from tests.emulated_ops import EmulatedOps
    tensors = tiny_tensors("A")
    toks = replay.random_tokens(97, 19, 4)
    eng = _engine("A", tensors, "float32", "cpu", EmulatedOps())
    seen = []
    for block in eng.model.blocks:
        inner = block.forward

        def hooked(ctx, cache, hidden, inner=inner):
            inner(ctx, cache, hidden)
            seen.append(hidden.clone())
        block.forward = hooked
    eng.step([("r", toks, [])])
    want = _plain("A", tensors).residuals(toks)
    assert len(seen) == 4
    for i, got in enumerate(seen):
        assert float((got.double() - want[i]).abs().max()) <= 3e-5 * float(want[i].abs().max()), i


def test_caches_and_states_of_a_layer_run():
    from tests.emulated_ops import EmulatedOps
    eng = _engine("A", tiny_tensors("A"), "float32", "cpu", EmulatedOps())
    # a chunked attention layer keeps its pages for the request's life; a latent layer caches one row per token
    kinds = sorted((g.spec.kind, g.spec.head_dim, g.spec.value_head_dim, g.spec.num_kv_heads) for g in eng.cache.groups)
    assert kinds == [("full", 12 + 4, 0, 1), ("full", 16, 24, 2), ("full", 24, 16, 4), ("full", 24 + 12, 0, 1)]
    # per parallel layer: the recurrence's state and the convolution's last inputs
    shapes = sorted(tuple(t.shape[1:]) for t in eng._run_state.values())
    assert shapes == sorted([(4, 12, 20), (3 - 1, 2 * 2 * 12 + 4 * 20), (2, 20, 8), (2 - 1, 2 * 1 * 20 + 2 * 8)])


# -- on the GPU ----------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_on_the_gpu(which, dtype, mode):
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"])
    steps = _traces(reqs)[mode]
    pool = replay.max_live_tokens(steps)
    eng = _engine(which, tensors, dtype, "cuda:0", max_tokens=pool)
    out = replay.run_trace_engine(eng, steps)
    if dtype == "float32":
        replay.compare(steps, out, _plain(which, tensors), reqs, what=f"{which}/{dtype}/{mode}", **FP32)
    else:
        _compare_bf16_with_routers(steps, out, _plain(which, tensors, True), reqs, f"{which}/{dtype}/{mode}")
    if mode == "mixed":
        blocks = sum(-(-len(t) // eng.page_tokens) for t in reqs.values())
        assert blocks > eng.num_pages and len(reqs) > eng.max_requests, "pages and slots must be used again"
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_bfloat16_replay_without_routers_row_by_row(which, mode):
    """Every mixer, the dense layers and the token gate in bfloat16, held to a bound at every row."""
    raw = _without_routers(TINY[which])
    tensors = _random(raw, 5)
    reqs = _requests(raw["vocab"])
    steps = _traces(reqs)[mode]
    eng = _engine(which, tensors, "bfloat16", "cuda:0", raw=raw, max_tokens=replay.max_live_tokens(steps))
    out = replay.run_trace_engine(eng, steps)
    # (a single position whose sums nearly cancel magnifies the rounding: a few rows may pass the bound, by no more than three times)
    replay.compare(steps, out, _plain(which, tensors, True, raw=raw), reqs, what=f"{which}/bfloat16/{mode}", rows_over=0.02,
                   **BF16)


@pytest.mark.gpu
@pytest.mark.parametrize("switch", ["LEONE_NO_LATENT_MMA", "LEONE_NO_TENSOR_CORES", "LEONE_NO_MIXED_MMA"])
@pytest.mark.parametrize("which", ["C", "D"])
def test_bfloat16_kernel_switches(which, switch, monkeypatch):
    """With a bfloat16 kernel's switch thrown its any-size form runs, and the same traces still agree
    with the plain implementation (prompt portions of 100 tokens and decode)."""
    monkeypatch.setenv(switch, "1")
    raw = _without_routers(TINY[which])
    tensors = _random(raw, 5)
    reqs = _requests(raw["vocab"], [130, 40, 75])
    steps = replay.trace_portions(reqs, sizes=(100, 2, 1, 1, 30))
    eng = _engine(which, tensors, "bfloat16", "cuda:0", raw=raw, max_tokens=replay.max_live_tokens(steps),
                  max_batch_tokens=128)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain(which, tensors, True, raw=raw), reqs, what=f"{which} with {switch}", rows_over=0.02,
                   **BF16)


@pytest.mark.gpu
@pytest.mark.parametrize("which,index", [(w, i) for w in ("A", "B", "C") for i in range(4)] + [("D", i) for i in range(3)])
def test_each_layer_alone(which, index):
    """A model of one layer: its mixer, feed-forward and token gate with nothing else to hide behind, in
    portions down to one token; the residual stream after the layer too."""
    raw = copy.deepcopy(TINY[which])
    raw["layers"] = [raw["layers"][index]]
    tensors = {k.replace(f"l{index}.", "l0."): v for k, v in tiny_tensors(which).items()
               if not k.startswith("l") or k.startswith(f"l{index}.")}
    if "token_side" in raw:
        d = raw["token_side"]["dim"]
        tensors["side.embed"] = tensors["side.embed"][:, index * d:(index + 1) * d].contiguous()
    reqs = _requests(raw["vocab"], [45, 2, 19])
    steps = replay.trace_portions(reqs, sizes=(2, 7, 1, 2, 13))
    eng = _engine(which, tensors, "float32", "cuda:0", raw=raw, max_tokens=192, max_requests=2, max_batch_tokens=64)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, plain.PlainZiginex(raw, tensors), reqs, what=f"{which} layer {index}", **FP32)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_no_vector_load_fits(dtype):
    """Odd widths everywhere (model width 50, heads of 6 and 7, latents of 9 and 5, a token table of 3, experts of
    11, a vocabulary of 101): every kernel takes its element-by-element form, in both dtypes."""
    raw = model(101, 50, 1e-5, side=3, layers=[
        parallel(left(3, 1, 6, 7, 0.4, chunk=11, softcap=9.0, rot_dims=4), right(3, 1, 5, 7, conv=3), moe(11, 3, 2, identity=2)),
        latent(3, 5, 2, 7, 9, 5, 0.3, base=300.0, scaling=(3.0, 20, 4.0, 1.0), mlp=dense(13))])
    tensors = _random(raw, 12)
    reqs = _requests(101, [37, 5, 18, 26], seed=3)
    steps = replay.trace_mixed(reqs, seed=4, max_live=3)
    eng = _engine(None, tensors, dtype, "cuda:0", max_tokens=replay.max_live_tokens(steps), page=8, raw=raw)
    out = replay.run_trace_engine(eng, steps)
    if dtype == "float32":
        replay.compare(steps, out, plain.PlainZiginex(raw, tensors), reqs, what="odd sizes", **FP32)
    else:
        _compare_bf16_with_routers(steps, out, _plain(None, tensors, True, raw=raw), reqs, "odd sizes")


@pytest.mark.gpu
def test_long_prompt_and_long_decode():
    """A prompt of many pages, then 150 single-token steps across pages and chunks; position 0 alone first."""
    for dtype, tol in (("float32", FP32), ("bfloat16", BF16)):
        tensors = tiny_tensors("C")
        reqs = {"one": replay.random_tokens(256, 1, 5), "long": replay.random_tokens(256, 460, 77)}
        steps = replay.trace_decode_tail(reqs, tail=150)
        eng = _engine("C", tensors, dtype, "cuda:0", max_tokens=512, max_batch_tokens=512)
        out = replay.run_trace_engine(eng, steps)
        if dtype == "float32":
            replay.compare(steps, out, _plain("C", tensors), reqs, what=f"long {dtype}", **tol)
        else:
            _compare_bf16_with_routers(steps, out, _plain("C", tensors, True), reqs, f"long {dtype}")


@pytest.mark.gpu
def test_page_size_does_not_change_fp32_logits():
    """Pages of another size hold the same rows; only the split of a token's keys over blocks (decided from
    the step, not the pages) could change sums, so the logits are equal to the bit."""
    tensors = tiny_tensors("A")
    reqs = _requests(97, [50, 21, 64])
    steps = replay.trace_mixed(reqs, seed=5)
    outs = []
    for pt in (4, 16, 64):
        eng = _engine("A", tensors, "float32", "cuda:0", max_tokens=replay.max_live_tokens(steps), page=pt)
        outs.append(replay.run_trace_engine(eng, steps))
    for k in outs[0]:
        assert np.array_equal(outs[0][k], outs[1][k]) and np.array_equal(outs[0][k], outs[2][k])


@pytest.mark.gpu
def test_a_slot_used_again_starts_from_nothing():
    """One state slot: the second request gets the slot (recurrent state, the convolution's inputs) and the
    pages the first one left, and must read none of it; its first tokens see zeros before the sequence's
    start."""
    tensors = tiny_tensors("A")
    reqs = _requests(97, [37, 29], seed=31)
    steps = replay.trace_portions(reqs, sizes=(1, 1, 2, 9, 40))
    eng = _engine("A", tensors, "float32", "cuda:0", max_tokens=64, max_requests=1)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain("A", tensors), reqs, what="slot used again", **FP32)


def _stand_out_model(chunk, branch):
    """A one-layer model in which token 7, and no other, writes something that token 9, and no other,
    reads.  ``branch = "left"``: a key dimension that only token 7 fills and a query dimension that only
    token 9 fills (scores far above all others); the recurrent branch is silenced by a zero output
    projection.  ``branch = "right"``: the same through the recurrence's keys and queries, with the
    attention silenced.  ``branch = "latent"``: through the latent layer's unrotated key part."""
    if branch == "latent":
        raw = _one_layer(latent(2, 8, 4, 6, 12, 10, 3.0, base=100.0, mlp=None))
    else:
        raw = _one_layer(parallel(left(2, 1, 8, 12, 3.0, chunk=chunk, rot_dims=4), right(2, 1, 8, 6, conv=1)))
    t = _random(raw, 3)
    t["embed"][:, :2] = 0.0
    for tok, coord in ((7, 0), (9, 1)):
        t["embed"][tok] = 0.0
        t["embed"][tok, coord] = 1.0
    if branch == "left":
        # key dimension 4 (not rotated) reads coordinate 0 only; query dimension 4 reads coordinate 1
        t["l0.mix.left.k"][4] = 0.0
        t["l0.mix.left.k"][4, 0] = 60.0
        t["l0.mix.left.q"][4, 1] += 60.0
        t["l0.mix.left.talk"] = torch.eye(2)
        t["l0.mix.right.o"] *= 0.0
    elif branch == "right":
        for name in ("q", "k"):
            t[f"l0.mix.right.{name}"][:, :2] = 0.0
            t[f"l0.mix.right.{name}.conv"][:] = 1.0
        t["l0.mix.right.k"][3, 0] = 80.0               # token 7's key is the unit vector of dimension 3
        t["l0.mix.right.q"][3, 1] = 80.0               # and token 9's query too
        t["l0.mix.right.a"] *= 0.0
        t["l0.mix.right.A_log"][:] = -9.0              # a decay that forgets next to nothing
        t["l0.mix.right.dt_bias"][:] = 0.0
        t["l0.mix.left.o"] *= 0.0
    else:
        t["l0.mix.dkv"][:, :2] = 0.0
        t["l0.mix.dkv"][5, 0] = 50.0                   # latent dimension 5 is token 7's
        t["l0.mix.dq"][:, 1] = 0.0
        t["l0.mix.dq"][2, 1] = 50.0                    # query latent dimension 2 is token 9's
        t["l0.mix.uq"][3] = 0.0
        t["l0.mix.uq"][3, 2] = 20.0                    # ... and feeds unrotated query dimension 3 of head 0
        t["l0.mix.uk"][3] = 0.0
        t["l0.mix.uk"][3, 5] = 20.0
    return raw, t


def _check_stand_out(raw, tensors, q_pos, k_pos, seen, page=16):
    length = q_pos + 4
    base = [t if t not in (7, 9) else 8 for t in replay.random_tokens(64, length, 9)]
    base[q_pos] = 9
    marked = list(base)
    if k_pos != q_pos:
        marked[k_pos] = 7
    oracle = plain.PlainZiginex(raw, tensors)
    delta = float((oracle.logits(marked)[q_pos] - oracle.logits(base)[q_pos]).abs().max())
    if k_pos != q_pos:
        assert (delta > 1e-3) == seen, ("the test's own premise", delta)
    eng = _engine(None, tensors, "float32", "cuda:0", raw=raw, page=page, max_tokens=704, max_requests=2,
                  max_batch_tokens=352)
    for name, toks in (("marked", marked), ("base", base)):
        want = oracle.logits(toks)[q_pos]
        bound = 3e-5 * float(want.abs().max())
        whole = eng.step([(name, toks, [q_pos])])[0].cpu()
        eng.close(name)
        assert float((whole.double() - want).abs().max()) <= bound, (name, "prompt")
        for cut in {max(1, q_pos - 2), min(k_pos + 1, q_pos)}:
            eng.step([(name, toks[:cut], [])])
            last = None
            for p in range(cut, q_pos + 1):
                last = eng.step([(name, [toks[p]], [0])])[0].cpu()
            eng.close(name)
            if last is not None:
                assert float((last.double() - want).abs().max()) <= bound, (name, "decoded from", cut)


@pytest.mark.gpu
@pytest.mark.parametrize("chunk,q_pos,k_pos", [
    (40, 79, 40), (40, 80, 79), (40, 80, 80), (40, 119, 80), (40, 120, 119), (40, 60, 39), (40, 60, 40),
    (17, 50, 34), (17, 50, 33), (17, 51, 50), (17, 51, 51), (16, 47, 32), (16, 47, 31), (16, 48, 47), (16, 31, 16), (16, 31, 15),
    (32, 63, 32), (32, 64, 63), (300, 299, 0), (300, 300, 299), (300, 310, 300),
    (1, 10, 9), (1, 10, 10), (3, 10, 9), (3, 10, 8), (3, 11, 9), (3, 11, 8), (None, 330, 0), (None, 200, 17)])
def test_one_key_at_a_chunk_edge(chunk, q_pos, k_pos):
    """The logits at ``q_pos`` change when the stand-out key sits at ``k_pos`` of the same chunk (its first
    position, a page border, hundreds of tokens back) and not at all when it sits in the chunk before
    (its last position included); in a prompt, decoded after a prompt that ends near the query, and
    decoded from right after the key."""
    raw, tensors = _stand_out_model(chunk, "left")
    seen = k_pos <= q_pos and (chunk is None or k_pos // chunk == q_pos // chunk)
    _check_stand_out(raw, tensors, q_pos, k_pos, seen)


@pytest.mark.gpu
@pytest.mark.parametrize("branch,q_pos,k_pos", [("right", 300, 2), ("right", 40, 39), ("right", 65, 0), ("right", 17, 16),
                                                ("latent", 330, 0), ("latent", 48, 47), ("latent", 64, 15), ("latent", 33, 16)])
def test_a_far_write_is_read(branch, q_pos, k_pos):
    """What one token wrote hundreds of tokens back (into the recurrent state; into the latent cache, across
    pages) is what another reads, in a prompt and through decoding."""
    raw, tensors = _stand_out_model(None, branch)
    _check_stand_out(raw, tensors, q_pos, k_pos, True)


@pytest.mark.gpu
def test_the_sink_counts_once_at_the_first_position_of_every_chunk():
    """At a chunk's first position the only members of the softmax are the token itself and the sink: with
    the sinks moved, the logits there move as the plain model's do; everywhere the engine follows."""
    raw = _one_layer(parallel(left(3, 1, 8, 8, 0.5, chunk=6, softcap=4.0, rot_dims=4), right(1, 1, 8, 8, conv=2), dense(24)))
    toks = replay.random_tokens(64, 26, 2)
    for shift in (0.0, 3.0, -30.0):
        tensors = _random(raw, 8)
        tensors["l0.mix.left.sink"] += shift
        eng = _engine(None, tensors, "float32", "cuda:0", raw=raw, page=4, max_tokens=64)
        got = eng.step([("r", toks[:13], list(range(13)))]).cpu()
        got = torch.cat([got, eng.step([("r", toks[13:], list(range(13)))]).cpu()])
        want = plain.PlainZiginex(raw, tensors).logits(toks)
        assert float((got.double() - want).abs().max()) <= 3e-5 * float(want.abs().max()), shift


def _step_ctx(q_lens, ctx_lens, slots, dev="cuda:0"):
    """What the kernels read of a step: ``q_lens[s]`` new tokens of sequence ``s`` that end at ``ctx_lens[s]``."""
    from types import SimpleNamespace
    starts = [0]
    for x in q_lens:
        starts.append(starts[-1] + x)
    pos = torch.cat([torch.arange(c - x, c) for c, x in zip(ctx_lens, q_lens)])
    seq = torch.cat([torch.full((x,), i) for i, x in enumerate(q_lens)])
    return SimpleNamespace(positions=pos.to(torch.int32).to(dev), seq_of_token=seq.to(torch.int32).to(dev),
                           n_seqs=len(q_lens), n_tokens=int(sum(q_lens)), q_lens=np.asarray(q_lens),
                           q_start=torch.tensor(starts, dtype=torch.int32, device=dev),
                           slot_ids=torch.tensor(slots, dtype=torch.int32, device=dev),
                           ctx_len=torch.tensor(ctx_lens, dtype=torch.int32, device=dev), max_q_len=max(q_lens),
                           max_ctx_len=max(ctx_lens), decode_only=max(q_lens) == 1,
                           status=torch.zeros(4, dtype=torch.int32, device=dev)), starts


def _paged_sequences(ctx_lens, n_kv, dk, dv, page, dtype, g, dev="cuda:0"):
    """Random keys and values of sequences in shuffled pages."""
    from leone_b200.parts.base import PagedCacheView
    pages = sum(-(-c // page) for c in ctx_lens)
    order = torch.randperm(pages, generator=g)
    table = torch.full((len(ctx_lens), -(-max(ctx_lens) // page)), -1, dtype=torch.int32)
    k_pool, v_pool = torch.zeros(pages, n_kv, page, dk, dtype=dtype), torch.zeros(pages, n_kv, page, dv, dtype=dtype)
    keys, vals, at = [], [], 0
    for s, c in enumerate(ctx_lens):
        kk, vv = torch.randn(c, n_kv, dk, generator=g).to(dtype), torch.randn(c, n_kv, dv, generator=g).to(dtype)
        keys.append(kk.double()), vals.append(vv.double())
        for b in range(-(-c // page)):
            table[s, b] = order[at]
            span = slice(b * page, min((b + 1) * page, c))
            k_pool[order[at], :, :span.stop - span.start] = kk[span].transpose(0, 1)
            v_pool[order[at], :, :span.stop - span.start] = vv[span].transpose(0, 1)
            at += 1
    return PagedCacheView(k_pool.to(dev), v_pool.to(dev), table.to(dev), page), keys, vals


def _mixed_scores_attention(q, k, v, scale, temp, cap, mix, sink, mask, size):
    """The rule once more, for one sequence: q [T, H, dk] (zero rows before the step), k [T, G, dk], v [T, G, dv]."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    kh, vh = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * scale
    if temp is not None:
        s = s * temp[:, None, None]
    if cap:
        s = cap * torch.tanh(s / cap)
    if mix is not None:
        s = torch.einsum("hg,gij->hij", mix, s)
    i = torch.arange(T)
    seen = i[None, :] <= i[:, None]
    if mask == "chunk":
        seen &= (i[None, :] // size) == (i[:, None] // size)
    elif mask == "window":
        seen &= i[:, None] - i[None, :] < size
    w = plain.sink_softmax(s, seen, sink)
    return torch.einsum("hij,jhv->ihv", w, vh)


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,dk,dv,mask,size,page,parts", [
    (6, 2, 12, 20, "chunk", 9, 8, "tcms"), (4, 4, 24, 16, "chunk", 70, 16, "tms"), (3, 1, 40, 8, "chunk", 1, 4, "cs"),
    (2, 1, 16, 136, "causal", 0, 16, "tcm"), (8, 2, 128, 128, "chunk", 64, 16, "tcms"), (16, 4, 96, 96, "window", 17, 16, "ms"),
    (5, 5, 16, 16, "chunk", 400, 16, "t"), (32, 8, 64, 64, "chunk", 128, 32, "tcms"), (1, 1, 7, 5, "chunk", 33, 16, "cms"),
    (7, 7, 9, 3, "causal", 0, 8, ""),
    # the tensor-core form's other shapes: two blocks a query tile with the query tile left in global memory, two
    # heads a warp, value width 96 on a key width of 48
    (32, 8, 128, 128, "chunk", 100, 16, "tcms"), (32, 4, 32, 32, "causal", 0, 16, "ms"), (8, 2, 48, 96, "window", 50, 16, "tcms")])
def test_mixed_heads_attention_kernel_against_the_plain_rule(n_q, n_kv, dk, dv, mask, size, page, parts):
    """The attention kernel alone over shuffled pages: three sequences of unequal lengths as prompt
    portions that start in the middle of a sequence, and as a decode step (where a token's keys are split
    over blocks), in 32-bit and in bfloat16, with each of temperature, cap, mixing and sink present or
    not, against the rule on the same stored values."""
    from leone_b200.ops.cuda import CudaOps
    ctx_lens = [300, 77, 130]
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)):
        ops = CudaOps("cuda:0", dtype)
        g = torch.Generator().manual_seed(dk + dv)
        cache, keys, vals = _paged_sequences(ctx_lens, n_kv, dk, dv, page, dtype, g)
        temp = (1.0 + 0.3 * torch.randn(n_q, generator=g)) if "t" in parts else None
        mix = (torch.eye(n_q) + 0.3 * torch.randn(n_q, n_q, generator=g)) if "m" in parts else None
        sink = torch.randn(n_q, generator=g) * 2 if "s" in parts else None
        cap = 3.0 if "c" in parts else None
        dev = [None if x is None else x.cuda() for x in (temp, mix, sink)]
        for q_lens in ([130, 77, 1], [1, 1, 1], [300, 2, 64], [1, 0 + 1, 5]):
            ctx, starts = _step_ctx(q_lens, ctx_lens, [0, 1, 2])
            n = sum(q_lens)
            q = (torch.randn(n, n_q, dk, generator=g) * 1.5).to(dtype)
            # the queries come first in a wider row, as the part's fused product leaves them
            rows = torch.zeros(n, n_q * dk + 24, dtype=dtype)
            rows[:, :n_q * dk] = q.reshape(n, -1)
            out = torch.zeros(n, n_q * dv, dtype=dtype, device="cuda:0")
            ops.attention_mixed_heads(ctx, rows.cuda(), out, cache, n_q, n_kv, dk, dv, 0.2, dev[0], cap, dev[1], dev[2],
                                      mask, size)
            assert int(ctx.status[0]) == 0
            for i, x in enumerate(q_lens):
                c = ctx_lens[i]
                full_q = torch.zeros(c, n_q, dk, dtype=torch.float64)
                full_q[c - x:] = q[starts[i]:starts[i + 1]].double()
                want = _mixed_scores_attention(full_q, keys[i], vals[i], 0.2, None if temp is None else temp.double(), cap,
                                               None if mix is None else mix.double(),
                                               None if sink is None else sink.double(), mask, size)[c - x:]
                got = out[starts[i]:starts[i + 1]].cpu().double().view(x, n_q, dv)
                err = float((got - want).abs().max()) / float(want.abs().max())
                assert err < tol, (dtype, q_lens, i, err)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 12, 20), (1, 1, 36, 12), (6, 3, 10, 14), (2, 1, 64, 64),
                                                     (2, 2, 128, 128), (3, 1, 144, 24), (1, 1, 300, 40), (8, 2, 32, 33),
                                                     (2, 1, 256, 8), (1, 1, 512, 64)])
def test_gated_delta_kernel_against_the_plain_recurrence(heads, kv_heads, dim, vdim):
    """The recurrence's kernel alone, every register form of it: three sequences in steps of unequal sizes
    (one of 40 tokens, single tokens, two tokens) with the state carried in slots that are not in order."""
    from leone_b200.ops.cuda import CudaOps
    ops = CudaOps("cuda:0", torch.float32)
    g = torch.Generator().manual_seed(dim + vdim)
    lengths, slots = [57, 3, 21], [2, 0, 3]
    qk, hv = kv_heads * dim, heads * vdim
    acts = [torch.randn(n, 2 * qk + hv, generator=g) for n in lengths]
    raws = [torch.randn(n, 2 * heads + 3, generator=g) * 2 for n in lengths]
    a_log, dt_bias = torch.randn(heads, generator=g) * 0.5, torch.randn(heads, generator=g) * 0.5
    state = torch.randn(4, heads, dim, vdim, generator=g).cuda()        # what a slot held before must not matter
    state[slots] = 0.0
    cuts = [[40, 1, 1, 2, 13], [1, 2], [2, 1, 18]]
    done = [0, 0, 0]
    got = [torch.zeros(n, hv) for n in lengths]
    for step in range(5):
        live = [s for s in range(3) if step < len(cuts[s])]
        q_lens = [cuts[s][step] for s in live]
        ctx, starts = _step_ctx(q_lens, [done[s] + cuts[s][step] for s in live], [slots[s] for s in live])
        act = torch.cat([acts[s][done[s]:done[s] + cuts[s][step]] for s in live]).cuda()
        raw = torch.cat([raws[s][done[s]:done[s] + cuts[s][step]] for s in live]).cuda()
        out = torch.zeros(sum(q_lens), hv, device="cuda:0")
        ops.gated_delta(ctx, act, raw, out, state, a_log.cuda(), dt_bias.cuda(), heads, kv_heads, dim, vdim, 0, qk, 2 * qk,
                        3, 3 + heads, dim ** -0.5)
        assert int(ctx.status[0]) == 0
        for j, s in enumerate(live):
            got[s][done[s]:done[s] + cuts[s][step]] = out[starts[j]:starts[j + 1]].cpu()
            done[s] += cuts[s][step]
    rep = heads // kv_heads
    for s, n in enumerate(lengths):
        a, r = acts[s].double(), raws[s].double()
        q = (plain.unit(a[:, :qk].view(n, kv_heads, dim)) * dim ** -0.5).repeat_interleave(rep, dim=1)
        k = plain.unit(a[:, qk:2 * qk].view(n, kv_heads, dim)).repeat_interleave(rep, dim=1)
        v = a[:, 2 * qk:].view(n, heads, vdim)
        beta = torch.sigmoid(r[:, 3 + heads:3 + 2 * heads])
        dec = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(r[:, 3:3 + heads] + dt_bias.double()))
        S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
        for t in range(n):
            S = dec[t][:, None, None] * S
            u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
            S = S + k[t][:, :, None] * u[:, None, :]
            want = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
            assert float((got[s][t].double() - want).abs().max()) <= 2e-5 * max(float(want.abs().max()), 1e-3), (s, t)
        assert float((state[slots[s]].cpu().double() - S).abs().max()) <= 2e-5 * float(S.abs().max())


@pytest.mark.gpu
def test_small_kernels_against_their_definitions():
    """The convolution's activation, the norm of a sublayer's output added to the stream (one and two
    sources, written and added, with its rounded copy), the gates, the per-head norm with its gate."""
    from leone_b200.ops.cuda import CudaOps
    g = torch.Generator().manual_seed(1)
    for dtype in (torch.float32, torch.bfloat16):
        ops = CudaOps("cuda:0", dtype)
        n, width = 37, 70
        a, b, dst = (torch.randn(n, width, generator=g) for _ in range(3))
        wa, wb = (1 + 0.1 * torch.randn(width, generator=g)).to(dtype), (1 + 0.1 * torch.randn(width, generator=g)).to(dtype)

        def normed(x, w):
            return plain.rms(x.double(), 1e-5) * w.double()
        for two, acc in ((False, True), (True, True), (True, False), (False, False)):
            d = dst.clone().cuda()
            rounded = torch.zeros(n, width, dtype=dtype, device="cuda:0")
            ops.rms_norm_add(d, a.cuda(), wa.cuda(), 1e-5, b=b.cuda() if two else None, w_b=wb.cuda() if two else None,
                             coef=0.5 if two else 1.0, accumulate=acc, rounded=rounded)
            want = (0.5 * (normed(a, wa) + normed(b, wb)) if two else normed(a, wa)) + (dst.double() if acc else 0)
            assert float((d.cpu().double() - want).abs().max()) < 1e-5
            assert torch.equal(rounded.cpu(), d.cpu().to(dtype))
        # the mean of two normed rows, normed once more before it is added
        d = dst.clone().cuda()
        ops.rms_norm_add(d, a.cuda(), wa.cuda(), 1e-5, b=b.cuda(), w_b=wb.cuda(), coef=0.5, then=wb.cuda())
        want = normed(0.5 * (normed(a, wa) + normed(b, wb)), wb) + dst.double()
        assert float((d.cpu().double() - want).abs().max()) < 1e-5
        x, gate = torch.randn(n, width, generator=g).to(dtype), torch.randn(n, width + 3, generator=g).to(dtype)
        for act in ("sigmoid", "silu"):
            y = x.clone().cuda()
            ops.gate_rows(y, gate.cuda()[:, 3:], act)
            f = torch.sigmoid(gate[:, 3:].double())
            want = x.double() * (f if act == "sigmoid" else f * gate[:, 3:].double())
            assert float((y.cpu().double() - want).abs().max()) <= (1e-6 if dtype == torch.float32 else 2e-2) * float(want.abs().max())
        z, rows = torch.randn(n, 6, generator=g) * 2, torch.randn(n, 30, generator=g)
        out = torch.zeros(n, 6, dtype=dtype, device="cuda:0")
        ops.gelu_gate(z.cuda(), rows.cuda(), 12, out)
        want = plain.gelu_tanh(z.double()) * rows[:, 12:18].double()
        assert float((out.cpu().double() - want).abs().max()) <= (1e-6 if dtype == torch.float32 else 1e-2) * float(want.abs().max())
        heads, vdim = 5, 14
        o, gt = torch.randn(n, heads * vdim, generator=g), torch.randn(n, heads * vdim + 8, generator=g)
        w = (1 + 0.1 * torch.randn(vdim, generator=g)).to(dtype)
        out = torch.zeros(n, heads * vdim, dtype=dtype, device="cuda:0")
        ops.group_gate_norm(o.cuda(), w.cuda(), gt.cuda()[:, 8:], out, 1e-5, heads, vdim, act="silu")
        want = (plain.rms(o.double().view(n, heads, vdim), 1e-5) * w.double()).reshape(n, -1) * plain.silu(gt[:, 8:].double())
        assert float((out.cpu().double() - want).abs().max()) <= (1e-5 if dtype == torch.float32 else 2e-2) * float(want.abs().max())
    # the convolution followed by silu, over two steps with state
    ops = CudaOps("cuda:0", torch.float32)
    x, w = torch.randn(29, 10, generator=g), torch.randn(10, 3, generator=g)
    state = torch.zeros(2, 2, 10, device="cuda:0")
    got = []
    for lo, hi in ((0, 17), (17, 18), (18, 29)):
        ctx, _ = _step_ctx([hi - lo], [hi], [1])
        out = torch.zeros(hi - lo, 10, device="cuda:0")
        part = x[lo:hi].cuda()
        ops.short_conv(ctx, part, w.cuda(), state, out, activation="silu", update_state=hi - lo == 1)
        if hi - lo != 1:
            ops.short_conv_state(ctx, part, state)
        got.append(out.cpu())
    want = plain.silu(plain.causal_conv(x.double(), w.double()))
    assert float((torch.cat(got).double() - want).abs().max()) < 1e-5


@pytest.mark.gpu
def test_router_with_correction_groups_and_identity_experts():
    """The selection kernel against the plain choice: softmax scores, a correction that moves the choice
    and the groups' worth but not the weights, the best groups only, identity outputs among the chosen;
    then the layer's output with identity experts, written and added."""
    from leone_b200.ops.cuda import CudaOps
    g = torch.Generator().manual_seed(4)
    for experts, identity, top, groups in ((5, 3, 2, (4, 2)), (12, 4, 3, (4, 3)), (4, 3, 7, None), (6, 0, 2, (3, 1)), (7, 2, 4, (3, 2))):
        n, width, ff = 41, 24, 16
        outputs = experts + identity
        cfg = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}}
        if groups:
            cfg["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
        W = {"router": torch.randn(outputs, width, generator=g) * 0.5, "correction": torch.randn(outputs, generator=g) * 0.1}
        for e in range(experts):
            W[f"e{e}.gate"], W[f"e{e}.up"] = torch.randn(ff, width, generator=g) * 0.3, torch.randn(ff, width, generator=g) * 0.3
            W[f"e{e}.down"] = torch.randn(width, ff, generator=g) * 0.3
        x = torch.randn(n, width, generator=g)
        ops = CudaOps("cuda:0", torch.float32)
        chosen = torch.zeros(n * top, dtype=torch.int32, device="cuda:0")
        weight = torch.zeros(n * top, dtype=torch.float32, device="cuda:0")
        cnt, keep = groups or (1, 1)
        ops.experts_route(x.cuda(), W["router"].cuda(), chosen, weight, top, True, False, groups=cnt, groups_kept=keep,
                          correction=W["correction"].cuda())
        Wd = {k: v.double() for k, v in W.items()}
        want_c, want_w = plain.route(x.double(), Wd, cfg)
        assert chosen.view(n, top).tolist() == want_c
        assert torch.allclose(weight.view(n, top).cpu().double(), torch.stack(want_w), atol=1e-6)
        want = plain.moe(x.double(), Wd, cfg)
        stack = lambda which: torch.stack([W[f"e{e}.{which}"] for e in range(experts)]).cuda()      # noqa: E731
        from leone_b200.parts.base import Runtime
        rt = Runtime("cuda:0", torch.float32, ops, 64)
        for fresh in (False, True):
            hidden = torch.full((n, width), 0.5, device="cuda:0")
            ops.experts_forward(x.cuda(), stack("gate"), stack("up"), stack("down"), chosen, weight, top, False, hidden, rt,
                                identity=identity, fresh=fresh)
            assert float((hidden.cpu().double() - (want + (0.0 if fresh else 0.5))).abs().max()) < 2e-5 * float(want.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype, which, tmp_path):
    """generate(): admission, prompt portions mixed with decode, captured decode steps (with the
    recurrent states and the convolutions' inputs in their slots), finish."""
    from leone_b200 import generate
    from leone_b200.weights.safetensors import write_safetensors
    folder = str(tmp_path / "model")
    cfg = tiny_config(which)
    cfg.write(folder)
    tensors = tiny_tensors(which)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    oracle = _plain(which, tensors, dtype == "bfloat16")
    prompts = [replay.random_tokens(TINY[which]["vocab"], n, 60 + n) for n in (1, 9, 40, 23, 5)]
    for kw in (dict(), dict(prefill_chunk=7, max_batch_tokens=16, use_graphs=False, prefill_first=False)):
        got = generate(folder, prompts, 10, dtype=dtype, eos_token_id=-1, max_running=3, **kw)
        for p, toks in zip(prompts, got):
            assert len(toks) == 10
            seq = list(p)
            for t in toks:
                logits = oracle.logits(seq)[-1]
                gap = float(logits.max() - logits[t])
                assert gap <= (1e-4 if dtype == "float32" else 0.04) * float(logits.abs().max()), (kw, seq, t, gap)
                seq.append(t)


@pytest.mark.gpu
def test_trace_program_on_a_written_model(tmp_path):
    """bin/trace_run as a user runs it: a folder with config.json and model.safetensors, steps over stdin."""
    from leone_b200.weights.safetensors import write_safetensors
    folder, out = str(tmp_path / "model"), str(tmp_path / "out")
    tiny_config("A").write(folder)
    tensors = {k: (v.to(torch.bfloat16) if v.dtype == torch.float32 else v) for k, v in tiny_tensors("A").items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    reqs = _requests(97, [30, 5, 41, 17, 8])
    steps = replay.trace_mixed(reqs, seed=11)
    got = replay.run_trace_program(folder, "float32", steps, out, replay.max_live_tokens(steps), extra=("--page-tokens", "4"))
    oracle = plain.PlainZiginex(TINY["A"], {k: v.float() for k, v in tensors.items()})
    replay.compare(steps, got, oracle, reqs, what="trace program", **FP32)
