"""The Sakinex decoder through the engine against the plain implementation (tests/plain/sakinex.py).

Without a GPU the engine runs on the stand-in kernels (tests/emulated_ops.py), which checks the
configuration, the model description, the loop's run order and injections, the bundles of caches and
states, and the step function's cutting and batching; on a B200 the same traces run on the CUDA
kernels in 32-bit and in bfloat16, together with tests that aim at single mechanisms."""
import copy
import math
import os

import numpy as np
import pytest
import torch

from leone_b200.engine.engine import Engine
from leone_b200.registry import config_from_dict, spec_from_config
from tests import replay
from tests.plain import sakinex as plain
from tests.sakinex_tiny import PAGE_TOKENS, TINY, as_bf16, layer, left, mixer, model, moe, tiny_config, tiny_tensors

FP32 = dict(rtol=3e-5, atol_scale=3e-5)
# bfloat16: the gained weights make scores, gates and routers sharp, which also amplifies rounding; the
# 32-bit runs are the sharp tests, these catch a wrong path or operand
BF16 = dict(rtol=1e-1, atol_scale=1e-1)
LENGTHS = [40, 7, 75, 33, 1, 64, 50]


def _bf16_round(t):
    return t.to(torch.bfloat16).to(t.dtype)


def _plain(which, tensors, bf16=False, raw=None):
    """In bfloat16 the plain model has the same stored weights and rounds what the cache holds."""
    return plain.PlainSakinex(raw or TINY[which], as_bf16(tensors) if bf16 else tensors,
                              cache_round=_bf16_round if bf16 else None)


def _engine(which, tensors, dtype, device, ops=None, max_tokens=512, page=None, raw=None, **kw):
    spec = spec_from_config(config_from_dict(raw) if raw is not None else tiny_config(which))
    return Engine(spec, dict(tensors), dtype=dtype, device=device, ops=ops, page_tokens=page or PAGE_TOKENS[which],
                  max_tokens=max_tokens, max_requests=kw.pop("max_requests", 4),
                  max_batch_tokens=kw.pop("max_batch_tokens", 128), **kw)


def _requests(vocab, lengths=LENGTHS, seed=100):
    return {f"r{i}": replay.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


def _traces(reqs):
    return {"whole": replay.trace_whole(reqs), "tail": replay.trace_decode_tail(reqs, tail=20),
            "portions": replay.trace_portions(reqs), "mixed": replay.trace_mixed(reqs, seed=3)}


def _random(raw, seed, gain=4.0):
    return tiny_tensors(None, seed=seed, gain=gain, raw=raw)


def _one_layer(m, mlp=None, vocab=64, width=32, canon=None, loop=None, mult=0.8, eps=1e-6):
    return model(vocab, width, eps, mult, [layer(m, mlp)], canon=canon, loop=loop)


# -- configuration and description (CPU) ---------------------------------------------------------
def test_config_round_trip_and_spec():
    for which, raw in TINY.items():
        cfg = config_from_dict(raw)
        assert cfg.to_json_dict() == raw
        spec = spec_from_config(cfg)
        assert all(ls.mixer.kind == "side_by_side" and ls.block == "pre_norm_conv" for ls in spec.layers)
        assert [ls.feed_forward is None for ls in spec.layers] == [e["mlp"] is None for e in raw["layers"]]
        order, later = plain.run_order(raw)
        assert list(spec.run_order) == order and {pos for pos, _ in spec.injections} == later


def test_run_order_of_loops():
    assert tiny_config("A").run_order() == (0, 1, 0, 1, 0, 1, 2, 3) and tiny_config("A").later_pass_starts() == (2, 4)
    assert tiny_config("B").run_order() == (0, 1, 1, 2, 3) and tiny_config("B").later_pass_starts() == (2,)
    assert tiny_config("C").run_order() == (0, 1, 2, 3) and tiny_config("C").later_pass_starts() == ()
    assert tiny_config("D").run_order() == (0, 1, 2, 0, 1, 2) and tiny_config("D").later_pass_starts() == (3,)


def test_config_rejections():
    from leone_b200.config.base import ConfigError
    for patch in (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4),
                  lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=3),
                  lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18),
                  lambda c: c["layers"][0]["mixer"]["left"].pop("mask"),
                  lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(pool=0),
                  lambda c: c["layers"][0]["mixer"].pop("right"),
                  lambda c: c["layers"][0].update(type="conv"),
                  lambda c: c["layers"][1]["mlp"]["router"].update(top=5),
                  lambda c: c["layers"][1]["mlp"].update(kind="dense"),
                  lambda c: c["loop"].update(stop=9), lambda c: c["loop"].update(start=2),
                  lambda c: c["canon"].update(taps=0),
                  lambda c: c.pop("width"), lambda c: c.update(layers=[])):
        raw = copy.deepcopy(TINY["A"])
        patch(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)


# -- the plain implementation's own mechanisms, against their definitions (CPU) -----------------------
def test_plain_convolution_and_candidate():
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]            # one channel: 1 2 3 4 5
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)        # the last tap reads the current input
    assert plain.causal_conv(u, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    assert plain.input_conv(u, w)[:, 0].tolist() == [2.0, 14.0, 126.0, 238.0, 350.0]
    # minGRU with identity projections: z = 1/2 everywhere (zero gate logits), candidates 2.5 and sigmoid(-1)
    eye = torch.eye(2, dtype=torch.float64)
    W = {"right.z": eye * 0, "right.z.b": torch.zeros(2, dtype=torch.float64), "right.x": eye,
         "right.x.b": torch.zeros(2, dtype=torch.float64), "right.g": eye, "right.o": eye}
    h = torch.tensor([[2.0, -1.0], [2.0, -1.0]], dtype=torch.float64)
    out = plain.min_gru(h, W)
    c = torch.tensor([2.5, 1 / (1 + math.e)], dtype=torch.float64)
    gate = h[0] * torch.sigmoid(h[0])
    assert torch.allclose(out[0], 0.5 * c * gate) and torch.allclose(out[1], 0.75 * c * gate)


def test_plain_window_and_pooled_blocks():
    """Values that name their position: with all scores equal the output is the mean of what is seen."""
    T, size, pool = 14, 4, 3
    q = torch.zeros(T, 1, 2, dtype=torch.float64)
    k = torch.zeros(T, 1, 2, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1)
    out = plain.pooled_window_attention(q, k, v, 1.0, size, pool)[:, 0, 0]
    for i in range(T):
        members = [float(j) for j in range(max(0, i - size + 1), i + 1)]
        members += [b * pool + (pool - 1) / 2 for b in range(T) if b * pool + pool - 1 <= i - size]
        assert abs(float(out[i]) - sum(members) / len(members)) < 1e-12, i
    # position 6 sees tokens 3..6 and block 0 (positions 0..2, whose last is 6 - 4); position 5 sees no block
    assert abs(float(out[6]) - (3 + 4 + 5 + 6 + 1) / 5) < 1e-12 and abs(float(out[5]) - (2 + 3 + 4 + 5) / 4) < 1e-12


def test_plain_yarn_and_router():
    f, mag = plain.yarn_frequencies(8, 100.0, None)
    assert mag == 1.0 and f == [100.0 ** (-2.0 * i / 8) for i in range(4)]
    f2, mag2 = plain.yarn_frequencies(8, 100.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})
    assert abs(mag2 - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert f2[0] == f[0] and abs(f2[3] - f[3] / 4.0) < 1e-15 and f[1] / 4.0 < f2[1] < f[1]
    z = torch.tensor([[0.1, 2.0, 2.0, -1.0, 1.5]], dtype=torch.float64)
    W = {"router": torch.eye(5, dtype=torch.float64), "router.b": torch.tensor([0.0, 0.0, 0.0, 3.2, 0.0], dtype=torch.float64)}
    chosen, weights = plain.route(z, W, {"router": {"experts": 5, "top": 3}})
    assert chosen == [[3, 1, 2]]                      # the bias lifts expert 3 to 2.2; equal logits: lowest index first
    e = torch.exp(torch.tensor([2.2, 2.0, 2.0], dtype=torch.float64))
    assert torch.allclose(weights[0], e / e.sum())


# -- the step function on stand-in kernels (CPU) ------------------------------------------------
@pytest.mark.parametrize("which", ["A", "B", "D"])
@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_replay_on_stand_in_kernels(which, mode):
    from tests.emulated_ops import EmulatedOps
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"], [23, 7, 30, 1, 12])
    steps = _traces(reqs)[mode]
    eng = _engine(which, tensors, "float32", "cpu", EmulatedOps(), max_tokens=replay.max_live_tokens(steps))
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain(which, tensors), reqs, what=f"{which} {mode} stand-in", rtol=2e-5, atol_scale=2e-5)
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


def test_caches_and_states_of_a_layer_run():
    from tests.emulated_ops import EmulatedOps
    eng = _engine("A", tiny_tensors("A"), "float32", "cpu", EmulatedOps())
    # every run of a looped layer owns its caches: token rows (given back once window + pool positions lie
    # behind them) and block means (one row per `pool` positions, kept for the request's life)
    kinds = sorted((g.spec.kind, g.spec.head_dim, g.spec.window, g.spec.tokens_per_row, len(g.spec.layers))
                   for g in eng.cache.groups)
    assert kinds == [("full", 16, None, 3, 3), ("full", 16, None, 4, 1), ("full", 24, None, 7, 3), ("full", 32, None, 6, 1),
                     ("window", 16, 12, 1, 3), ("window", 16, 24, 1, 1), ("window", 24, 12, 1, 3), ("window", 32, 18, 1, 1)]
    # states per run: the minGRU's, the convolution on q, k and v, and the two in front of the sublayers
    shapes = sorted(tuple(t.shape[1:]) for t in eng._run_state.values())
    assert shapes.count((40,)) == 3 and shapes.count((2, 64)) == 3 * 2 + 3 * 2 + 1 + 2
    assert shapes.count((3, 6 * 16 + 2 * 16 + 2 * 24)) == 3 and shapes.count((1, 4 * 24 + 4 * 24 + 4 * 16)) == 3


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
    tol = FP32 if dtype == "float32" else BF16
    replay.compare(steps, out, _plain(which, tensors, dtype == "bfloat16"), reqs, what=f"{which}/{dtype}/{mode}", **tol)
    if mode == "mixed":
        blocks = sum(-(-len(t) // eng.page_tokens) for t in reqs.values())
        assert blocks > eng.num_pages and len(reqs) > eng.max_requests, "pages and slots must be used again"
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


@pytest.mark.gpu
@pytest.mark.parametrize("switch", ["LEONE_NO_POOLED_TC", "LEONE_NO_POOLED_MMA", "LEONE_NO_EXPERT_MMA", "LEONE_NO_TENSOR_CORES", "LEONE_NO_FUSED_NORM"])
@pytest.mark.parametrize("which", ["C", "D"])
def test_bfloat16_kernel_switches(which, switch, monkeypatch):
    """Every bfloat16 kernel has an any-size form behind a switch; with the switch thrown the same
    traces still agree with the plain implementation (prompt portions of 100 tokens and decode)."""
    monkeypatch.setenv(switch, "1")
    tensors = tiny_tensors(which)
    reqs = _requests(TINY[which]["vocab"], [130, 40, 75])
    steps = replay.trace_portions(reqs, sizes=(100, 2, 1, 1, 30)) + []
    eng = _engine(which, tensors, "bfloat16", "cuda:0", max_tokens=replay.max_live_tokens(steps), max_batch_tokens=128)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain(which, tensors, True), reqs, what=f"{which} with {switch}", **BF16)


@pytest.mark.gpu
@pytest.mark.parametrize("which,index", [(w, i) for w in ("A", "B", "C") for i in range(4)])
def test_each_layer_alone(which, index):
    """A model of one layer (looped twice where the configuration has a loop): its mixer and
    feed-forward with nothing else to hide behind; the residual stream after every run too."""
    raw = copy.deepcopy(TINY[which])
    raw["layers"] = [raw["layers"][index]]
    if "loop" in raw:
        raw["loop"] = {"start": 0, "stop": 1, "times": 2}
    tensors = {k.replace(f"l{index}.", "l0."): v for k, v in tiny_tensors(which).items()
               if not k.startswith("l") or k.startswith(f"l{index}.")}
    reqs = _requests(raw["vocab"], [45, 2, 19])
    steps = replay.trace_portions(reqs, sizes=(2, 7, 1, 2, 13))
    eng = _engine(which, tensors, "float32", "cuda:0", raw=raw, max_tokens=192, max_requests=2, max_batch_tokens=64)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, plain.PlainSakinex(raw, tensors), reqs, what=f"{which} layer {index}", **FP32)


@pytest.mark.gpu
def test_convolutions_of_one_tap():
    """One tap in every convolution (in front of the sublayers and on q, k, v): nothing is carried from
    token to token, and no state is asked for; two taps beside it."""
    for canon, conv in ((1, 1), (1, 2), (2, 1)):
        raw = model(80, 48, 1e-6, 0.7, canon=canon, layers=[
            layer(mixer(left(4, 2, 8, 12, 0.3, 6, 3, conv=conv, rot_dims=4), 24, 1.0, 0.8), moe(16, 4, 2, shared=8)),
            layer(mixer(left(2, 2, 16, 8, 0.2, 11, 2, conv=conv), 40, 0.9, 1.0), None)])
        tensors = _random(raw, 21 + canon + conv)
        reqs = _requests(80, [37, 5, 18], seed=3)
        steps = replay.trace_mixed(reqs, seed=4)
        eng = _engine(None, tensors, "float32", "cuda:0", max_tokens=replay.max_live_tokens(steps), page=8, raw=raw)
        out = replay.run_trace_engine(eng, steps)
        replay.compare(steps, out, plain.PlainSakinex(raw, tensors), reqs, what=f"taps {canon}, {conv}", **FP32)


@pytest.mark.gpu
def test_long_prompt_and_long_decode():
    """A prompt of many pages, then 150 single-token steps across pages, windows and blocks;
    position 0 alone first.  The prompt is long enough for the recurrence to run in chunks."""
    for dtype, tol in (("float32", FP32), ("bfloat16", BF16)):
        tensors = tiny_tensors("C")
        reqs = {"one": replay.random_tokens(256, 1, 5), "long": replay.random_tokens(256, 460, 77)}
        steps = replay.trace_decode_tail(reqs, tail=150)
        eng = _engine("C", tensors, dtype, "cuda:0", max_tokens=512, max_batch_tokens=512)
        out = replay.run_trace_engine(eng, steps)
        replay.compare(steps, out, _plain("C", tensors, dtype == "bfloat16"), reqs, what=f"long {dtype}",
                       rows_over=0.01 if dtype == "bfloat16" else 0.0, **tol)


@pytest.mark.gpu
def test_page_size_does_not_change_fp32_logits():
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
    """One state slot: the second request gets the slot (recurrent state, three convolutions' inputs)
    and the pages the first one left, and must read none of it; its first tokens see zeros before
    the sequence's start."""
    tensors = tiny_tensors("A")
    reqs = _requests(97, [37, 29], seed=31)
    steps = replay.trace_portions(reqs, sizes=(1, 1, 2, 9, 40))
    eng = _engine("A", tensors, "float32", "cuda:0", max_tokens=64, max_requests=1)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, _plain("A", tensors), reqs, what="slot used again", **FP32)


def _seen(size, pool, q_pos, k_pos):
    """The design's rule, stated once more for the test's own premise."""
    if k_pos > q_pos:
        return False
    if q_pos - k_pos < size:
        return True
    block = k_pos // pool
    return block * pool + pool - 1 <= q_pos - size


@pytest.mark.gpu
@pytest.mark.parametrize("size,pool,q_pos,k_pos", [
    (40, 8, 60, 21), (40, 8, 60, 20), (40, 8, 63, 20), (40, 8, 62, 20), (40, 8, 62, 15),
    (17, 5, 48, 32), (17, 5, 48, 31), (17, 5, 51, 31), (17, 5, 50, 31),
    (16, 16, 47, 32), (16, 16, 47, 31), (16, 16, 46, 31), (16, 16, 46, 15), (16, 16, 62, 32), (16, 16, 63, 32),
    (30, 4, 299, 0), (30, 4, 299, 151), (300, 7, 200, 0),
    (5, 32, 40, 10), (5, 32, 36, 10), (5, 32, 35, 10), (5, 32, 35, 31),
    (1, 1, 10, 9), (1, 1, 10, 10), (1, 1, 10, 0), (3, 2, 10, 7), (3, 2, 10, 8), (3, 2, 9, 6), (3, 2, 8, 6)])
def test_one_key_that_stands_out(size, pool, q_pos, k_pos):
    """A one-layer model (attention branch only, no convolutions) whose token 7, and no other, makes a
    key that token 9's query scores far above all others: the logits at ``q_pos`` change when that key
    sits at ``k_pos`` and the query may see it (just inside the window, through a block whose last
    position has just left the window, at a page border, hundreds of tokens back), and not at all
    when it may not (out of the window with its block not yet complete or not yet wholly before the
    window).  Checked for the position in a prompt, decoded after a prompt that ends near it, and
    decoded from right after ``k_pos``, so that the block's means are formed by a decode step."""
    raw = _one_layer(mixer(left(2, 1, 8, 12, 3.0, size, pool, rot_dims=4), 16, 1.0, 0.0))
    tensors = _random(raw, 3)
    # coordinate 0 belongs to token 7 and coordinate 1 to token 9; key dimension 4 (not rotated) reads coordinate 0
    # only, so every other token's key is zero there; query dimension 4 reads coordinate 1
    tensors["embed"][:, :2] = 0.0
    for tok, coord in ((7, 0), (9, 1)):
        tensors["embed"][tok] = 0.0
        tensors["embed"][tok, coord] = 1.0
    tensors["l0.mix.left.k"][4] = 0.0
    tensors["l0.mix.left.k"][4, 0] = 60.0
    tensors["l0.mix.left.q"][4, 1] += 60.0
    length = q_pos + 4
    base = [t if t not in (7, 9) else 8 for t in replay.random_tokens(64, length, 9)]
    base[q_pos] = 9
    marked = list(base)
    if k_pos != q_pos:
        marked[k_pos] = 7
    oracle = plain.PlainSakinex(raw, tensors)
    delta = float((oracle.logits(marked)[q_pos] - oracle.logits(base)[q_pos]).abs().max())
    if k_pos != q_pos:
        assert (delta > 1e-3) == _seen(size, pool, q_pos, k_pos), "the test's own premise"
    eng = _engine(None, tensors, "float32", "cuda:0", raw=raw, page=16, max_tokens=704, max_requests=2,
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


@pytest.mark.gpu
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_with_state_against_the_plain_sum(taps):
    """Two sequences cut into steps of unequal sizes (steps of one token, steps shorter than the taps):
    the convolution reads what earlier steps left in the state, and zeros before a sequence's start.
    Then steps of more than a hundred tokens, which a kernel takes that forms eight tokens a thread:
    a sequence that ends inside such a group, one that starts from the state inside it."""
    from leone_b200.ops.cuda import CudaOps
    g = torch.Generator().manual_seed(taps)
    channels = 70
    w = torch.randn(channels, taps, generator=g)
    for lens, cuts in (([23, 9], ([1, 3], [2, 1], [1, 0], [8, 5], [11, 0])),
                       ([310, 214], ([3, 2], [133, 67], [1, 1], [0, 144], [173, 0]))):
      xs = [torch.randn(n, channels, generator=g) for n in lens]
      for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        ops = CudaOps("cuda:0", dtype)
        for add_input in (False, True):
            state = torch.full((3, max(taps - 1, 0), channels), 7.0, device="cuda:0")
            state[[2, 0]] = 0.0                                   # the slots of the two sequences start from zeros
            done, got = [0, 0], [[], []]
            for cut in cuts:
                seqs = [s for s in (0, 1) if cut[s]]
                ctx, starts = _step_ctx([cut[s] for s in seqs], [done[s] + cut[s] for s in seqs], [(2, 0)[s] for s in seqs])
                x = torch.cat([xs[s][done[s]:done[s] + cut[s]] for s in seqs]).to(dtype).cuda()
                out = torch.zeros_like(x)
                # a step of single tokens: the convolution's kernel moves the state on itself
                fused = taps > 1 and bool(ctx.decode_only)
                ops.short_conv(ctx, x, w.cuda(), state if taps > 1 else None, out, add_input=add_input, update_state=fused)
                if taps > 1 and not fused:
                    ops.short_conv_state(ctx, x, state)
                assert int(ctx.status[0]) == 0
                for i, s in enumerate(seqs):
                    got[s].append(out[starts[i]:starts[i + 1]].float().cpu())
                    done[s] += cut[s]
            for s in (0, 1):
                xin = xs[s].to(dtype).double()
                want = plain.causal_conv(xin, w.double()) + (xin if add_input else 0)
                err = float((torch.cat(got[s]).double() - want).abs().max()) / float(want.abs().max())
                assert err <= tol, (dtype, add_input, s, err)
            assert float(state[1].min()) == 7.0 if taps > 1 else True        # a slot of no sequence is left alone


@pytest.mark.gpu
@pytest.mark.parametrize("width", [150, 152])      # 152: the chunk kernels take four channels a thread
def test_min_gru_in_one_walk_and_in_chunks_against_the_plain_recurrence(width):
    """Gate logits and candidates on both sides of zero; a state carried over from an earlier step; the
    walk token by token and the chunked form agree with the plain recurrence."""
    from leone_b200.ops.cuda import CudaOps
    ops = CudaOps("cuda:0", torch.float32)
    g = torch.Generator().manual_seed(4)
    lens = [61, 1, 18]
    proj = torch.randn(sum(lens), 3 * width, generator=g) * 3.0
    zb, xb = torch.randn(width, generator=g), torch.randn(width, generator=g)
    start = torch.randn(4, width, generator=g)
    want, at = [], 0
    for s, n in enumerate(lens):
        p = proj[at:at + n].double()
        z = torch.sigmoid(p[:, :width] + zb.double())
        u = p[:, width:2 * width] + xb.double()
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        S = start[(3, 1, 0)[s]].double()
        for t in range(n):
            S = (1 - z[t]) * S + z[t] * cand[t]
            want.append(0.7 * S * plain.silu(p[t, 2 * width:]))
        at += n
    want = torch.stack(want)
    assert float((proj[:, width:2 * width] + xb < 0).float().mean()) > 0.2
    for chunk in (0, 4, 7, 64):
        ctx, _ = _step_ctx(lens, [100, 1, 50], [3, 1, 0])
        state = start.clone().cuda()
        out = torch.zeros(sum(lens), width, device="cuda:0")
        ops.min_gru(ctx, proj.cuda(), zb.cuda(), xb.cuda(), state, out, out_scale=0.7, chunk=chunk)
        assert float((out.cpu().double() - want).abs().max()) <= 2e-5 * float(want.abs().max()), chunk
        assert torch.equal(state[2].cpu(), start[2])
        half = torch.zeros(sum(lens), width, device="cuda:0", dtype=torch.bfloat16)
        ops.min_gru(ctx, proj.cuda(), zb.cuda(), xb.cuda(), start.clone().cuda(), half, out_scale=0.7, chunk=chunk)
        assert float((half.cpu().double() - want).abs().max()) <= 1e-2 * float(want.abs().max()), chunk


@pytest.mark.gpu
def test_router_with_a_bias_and_weights_over_the_chosen_logits():
    from leone_b200.ops.cuda import CudaOps
    ops = CudaOps("cuda:0", torch.float32)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(50, 72, generator=g)
    for experts, top in ((12, 4), (5, 5), (7, 1), (33, 6)):
        w = torch.randn(experts + 1, 72, generator=g) * 0.3            # one more row: another per-token logit
        b = torch.randn(experts, generator=g)
        chosen = torch.zeros(50 * top, dtype=torch.int32, device="cuda:0")
        weight = torch.zeros(50 * top, dtype=torch.float32, device="cuda:0")
        logits = ops.experts_route(x.cuda(), w.cuda(), chosen, weight, top, "chosen", False, weight_scale=0.5,
                                   bias=b.cuda(), experts=experts)
        want_e, want_w = plain.route(x.double(), {"router": w[:experts].double(), "router.b": b.double()},
                                     {"router": {"experts": experts, "top": top}})
        assert chosen.cpu().view(50, top).tolist() == want_e
        assert torch.allclose(weight.cpu().view(50, top).double(), 0.5 * torch.stack(want_w), rtol=1e-5, atol=1e-7)
        assert torch.allclose(logits[:, experts].cpu().double(), x.double() @ w[experts].double(), rtol=1e-5, atol=1e-5)


def _paged_sequences(ctx_lens, n_kv, dk, dv, page, pool, dtype, g, dev="cuda:0"):
    """Random keys and values of three sequences in shuffled pages, and every complete block's means in the
    cache of blocks (formed in fp32 from the stored rows, stored in the cache's dtype)."""
    from leone_b200.parts.base import PagedCacheView
    pages = sum(-(-c // page) for c in ctx_lens)
    order = torch.randperm(pages, generator=g)
    rows = -(-page // pool)
    table = torch.full((len(ctx_lens), -(-max(ctx_lens) // page)), -1, dtype=torch.int32)
    k_pool, v_pool = torch.zeros(pages, n_kv, page, dk, dtype=dtype), torch.zeros(pages, n_kv, page, dv, dtype=dtype)
    kb_pool, vb_pool = torch.zeros(pages, n_kv, rows, dk, dtype=dtype), torch.zeros(pages, n_kv, rows, dv, dtype=dtype)
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
        for b in range(c // pool):
            e = b * pool + pool - 1
            pg, row = table[s, e // page], (e % page) // pool
            kb_pool[pg, :, row] = kk[b * pool:e + 1].float().mean(dim=0).to(dtype)
            vb_pool[pg, :, row] = vv[b * pool:e + 1].float().mean(dim=0).to(dtype)
    tokens = PagedCacheView(k_pool.to(dev), v_pool.to(dev), table.to(dev), page)
    blocks = PagedCacheView(kb_pool.to(dev), vb_pool.to(dev), table.to(dev), page, True, pool)
    return tokens, blocks, keys, vals


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,dk,dv,window,pool,page", [
    (6, 2, 12, 20, 9, 3, 8), (4, 4, 24, 16, 70, 7, 16), (3, 1, 40, 8, 1, 1, 4), (2, 1, 16, 136, 33, 40, 16),
    (8, 2, 128, 128, 64, 16, 16), (4, 1, 64, 64, 100, 16, 16), (6, 2, 32, 48, 130, 24, 32), (16, 4, 96, 96, 17, 64, 16),
    (5, 5, 16, 16, 400, 4, 16), (8, 1, 128, 16, 48, 8, 16),
    # more than 128 blocks (several tiles of block means on the tcgen05 form), pool 1, a window past the prompt
    (4, 2, 64, 64, 5, 2, 16), (16, 2, 128, 128, 40, 1, 16), (2, 1, 64, 64, 1, 1, 32), (8, 8, 128, 128, 290, 3, 16)])
def test_pooled_window_attention_kernels_against_the_plain_rule(n_q, n_kv, dk, dv, window, pool, page):
    """The attention kernels alone over shuffled pages: three sequences of unequal lengths as prompt
    portions that start in the middle of a sequence, and as a decode step, in 32-bit (the any-size
    kernel) and in bfloat16 (the tensor-core forms where the sizes allow), against the plain rule on
    the same stored values."""
    from leone_b200.ops.cuda import CudaOps
    ctx_lens = [300, 77, 130]
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)):
        ops = CudaOps("cuda:0", dtype)
        g = torch.Generator().manual_seed(dk + dv)
        tokens, blocks, keys, vals = _paged_sequences(ctx_lens, n_kv, dk, dv, page, pool, dtype, g)
        for q_lens in ([130, 77, 1], [1, 1, 1], [300, 2, 64]):
            ctx, starts = _step_ctx(q_lens, ctx_lens, [0, 1, 2])
            n = sum(q_lens)
            q = (torch.randn(n, n_q, dk, generator=g) * 1.5).to(dtype)
            out = torch.zeros(n, n_q * dv, dtype=dtype, device="cuda:0")
            ops.attention_pooled(ctx, q.reshape(n, -1).cuda(), out, tokens, blocks, n_q, n_kv, dk, dv, 0.2, window, pool,
                                 out_scale=0.9)
            assert int(ctx.status[0]) == 0
            for i, x in enumerate(q_lens):
                c = ctx_lens[i]
                full_q = torch.zeros(c, n_q, dk, dtype=torch.float64)
                full_q[c - x:] = q[starts[i]:starts[i + 1]].double()
                round_ = (lambda t: t.to(dtype).double()) if dtype != torch.float32 else None
                want = 0.9 * plain.pooled_window_attention(full_q, keys[i], vals[i], 0.2, window, pool, round_)[c - x:]
                got = out[starts[i]:starts[i + 1]].cpu().double().view(x, n_q, dv)
                err = float((got - want).abs().max()) / float(want.abs().max())
                assert err < tol, (dtype, q_lens, i, err)


@pytest.mark.gpu
@pytest.mark.parametrize("q_lens,ctx_lens,pool,page", [
    ([600, 5, 230], [700, 77, 230], 7, 16), ([4200, 300], [4300, 900], 24, 16), ([1, 1, 1], [64, 63, 130], 32, 32)])
def test_block_means_of_long_steps(q_lens, ctx_lens, pool, page):
    """The kernel that forms the block means looks through 1, 8 or 32 tokens a thread block, by the
    step's length: every block that one of the step's tokens ends gets its means, the others stay as
    they were, whatever the grouping."""
    from leone_b200.ops.cuda import CudaOps
    n_kv, dk, dv = 2, 24, 40
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        ops = CudaOps("cuda:0", dtype)
        g = torch.Generator().manual_seed(pool)
        tokens, blocks, keys, vals = _paged_sequences(ctx_lens, n_kv, dk, dv, page, pool, dtype, g)
        want_k, want_v = blocks.k_pool.clone(), blocks.v_pool.clone()
        # the blocks that this step's tokens end are wiped, the others keep a mark
        table = tokens.block_table.cpu()
        for s, (x, c) in enumerate(zip(q_lens, ctx_lens)):
            for b in range(c // pool):
                e = b * pool + pool - 1
                pg, row = int(table[s, e // page]), (e % page) // pool
                if e >= c - x:
                    blocks.k_pool[pg, :, row] = 0
                    blocks.v_pool[pg, :, row] = 0
                else:
                    blocks.k_pool[pg, :, row] = 5.0
                    want_k[pg, :, row] = 5.0
        ctx, _ = _step_ctx(q_lens, ctx_lens, [0, 1, 2][:len(q_lens)])
        ops.attention_pool_blocks(ctx, tokens, blocks, n_kv, dk, dv, pool)
        assert int(ctx.status[0]) == 0
        assert float((blocks.k_pool.float() - want_k.float()).abs().max()) <= tol * 4
        assert float((blocks.v_pool.float() - want_v.float()).abs().max()) <= tol * 4


@pytest.mark.gpu
def test_preparation_and_block_means_against_the_plain_steps():
    """The preparation kernel (convolution with state, partial rotation with YaRN frequencies and their
    magnitude, unit norm per head, cache write) and the kernel that forms the block means, over two
    steps of one sequence, in 32-bit."""
    from leone_b200.ops.cuda import CudaOps
    from leone_b200.parts.base import PagedCacheView
    from leone_b200.parts.rotary import RotaryComputed
    ops = CudaOps("cuda:0", torch.float32)
    g = torch.Generator().manual_seed(8)
    n, n_q, n_kv, dk, dv, page, pool, taps, eps = 45, 6, 2, 12, 20, 8, 5, 3, 1e-5
    rot = {"base": 300.0, "dims": 8, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 0.5}}
    pe = RotaryComputed({"rotary_dim": 8, "base": 300.0, "pairing": "half_split", "scaling": rot["scaling"]}, None)
    cols = (n_q + n_kv) * dk + n_kv * dv
    proj = torch.randn(n, cols, generator=g)
    conv_w = torch.randn(cols, taps, generator=g)
    pages = -(-n // page)
    table = torch.randperm(pages, generator=g).to(torch.int32).view(1, pages).cuda()
    tokens = PagedCacheView(torch.zeros(pages, n_kv, page, dk, device="cuda:0"), torch.zeros(pages, n_kv, page, dv, device="cuda:0"),
                            table, page)
    rows = -(-page // pool)
    blocks = PagedCacheView(torch.zeros(pages, n_kv, rows, dk, device="cuda:0"), torch.zeros(pages, n_kv, rows, dv, device="cuda:0"),
                            table, page, True, pool)
    state = torch.zeros(2, taps - 1, cols, device="cuda:0")
    q_got = []
    for a, b in ((0, 28), (28, 29), (29, 30), (30, 45)):     # the steps of one token move the state on in the kernel
        ctx, _ = _step_ctx([b - a], [b], [1])
        q_out = torch.zeros(b - a, n_q * dk, device="cuda:0")
        fused = bool(ctx.decode_only)
        ops.attention_pooled_prepare(ctx, proj[a:b].cuda(), q_out, n_q, n_kv, dk, dv, conv_w.cuda(), state,
                                     pe._freqs_host.cuda(), "half_split", float(pe.magnitude), True, eps, tokens,
                                     update_state=fused)
        if not fused:
            ops.short_conv_state(ctx, proj[a:b].cuda(), state)
        ops.attention_pool_blocks(ctx, tokens, blocks, n_kv, dk, dv, pool)
        assert int(ctx.status[0]) == 0
        q_got.append(q_out.cpu())
    x = plain.causal_conv(proj.double(), conv_w.double())
    q, k = x[:, :n_q * dk].reshape(n, n_q, dk), x[:, n_q * dk:(n_q + n_kv) * dk].reshape(n, n_kv, dk)
    v = x[:, (n_q + n_kv) * dk:].reshape(n, n_kv, dv)
    q, k = plain.rms(plain.rotate(q, list(range(n)), rot), eps), plain.rms(plain.rotate(k, list(range(n)), rot), eps)
    assert torch.allclose(torch.cat(q_got).double(), q.reshape(n, -1), rtol=2e-5, atol=2e-5)
    pos = torch.arange(n)
    slot = table[0].cpu().long()[pos // page]
    assert torch.allclose(tokens.k_pool.cpu().double()[slot, :, pos % page, :], k, rtol=2e-5, atol=2e-5)
    assert torch.allclose(tokens.v_pool.cpu().double()[slot, :, pos % page, :], v, rtol=2e-5, atol=2e-5)
    for b in range(n // pool):
        e = b * pool + pool - 1
        pg, row = int(table[0, e // page]), (e % page) // pool
        assert torch.allclose(blocks.k_pool[pg, :, row].cpu().double(), k[b * pool:e + 1].mean(dim=0), rtol=2e-5, atol=2e-5)
        assert torch.allclose(blocks.v_pool[pg, :, row].cpu().double(), v[b * pool:e + 1].mean(dim=0), rtol=2e-5, atol=2e-5)


@pytest.mark.gpu
def test_gated_shared_expert_and_residual_multiplier():
    """One layer whose routed experts are silent (zero down projections), so that the feed-forward is the
    shared expert times its per-token gate times the multiplier; gate logits on both sides of zero."""
    raw = _one_layer(mixer(left(2, 2, 8, 8, 0.3, 6, 2, rot_dims=8), 16, 1.0, 1.0), moe(24, 4, 2, shared=40), canon=2, mult=0.35)
    tensors = _random(raw, 21, gain=6.0)
    for e in range(4):
        tensors[f"l0.mlp.e{e}.down"] *= 0.0
    toks = replay.random_tokens(64, 40, 3)
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 5e-2)):
        oracle = _plain(None, tensors, dtype == "bfloat16", raw=raw)
        eng = _engine(None, tensors, dtype, "cuda:0", raw=raw, page=16, max_tokens=64, max_requests=2, max_batch_tokens=64)
        got = eng.step([("g", toks, list(range(40)))]).cpu().double()
        want = oracle.logits(toks)
        assert float((got - want).abs().max()) <= tol * float(want.abs().max())
    quiet = copy.deepcopy(tensors)
    quiet["l0.mlp.shared.sg"] = quiet["l0.mlp.shared.sg"] * 0 - 0.0
    other = plain.PlainSakinex(raw, quiet).logits(toks)
    assert float((other - plain.PlainSakinex(raw, tensors).logits(toks)).abs().max()) > 1e-2, "the gate matters"


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype, which, tmp_path):
    """generate(): admission, prompt portions mixed with decode, captured decode steps (with the
    looped layers, their states and windows whose pages go back while decoding), finish."""
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
    oracle = plain.PlainSakinex(TINY["A"], {k: v.float() for k, v in tensors.items()})
    replay.compare(steps, got, oracle, reqs, what="trace program", **FP32)
