"""The Vunasun decoder against the plain float64 implementation (tests/plain/vunasun_plain.py):
every mechanism alone and together, in whole prompts, portions, single decoded tokens, mixed
batches, reused slots and pages, and through the engine's own entry point."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

from plain import vunasun_plain as VP
from vunasun_util import (CONFIGS, assert_close, model_dir, needle_model, plain_logits, random_config,
                          runner_for, sensitivity, tokens_for, weights)

DTYPES = ("float32", "bfloat16")


# --------------------------------------------------------------------------------------------
# no GPU: configuration, and the plain implementation against itself
# --------------------------------------------------------------------------------------------
def test_configuration_round_trip_and_tensor_names():
    from llmario_b200.config import ConfigError, VunasunConfig, resolve_architecture
    from llmario_b200.weights.loader import check_tensors, expected_tensors

    for name, raw in CONFIGS.items():
        assert resolve_architecture(raw) == "Vunasun"
        cfg = VunasunConfig.from_dict(raw)
        assert VunasunConfig.from_dict(cfg.to_dict()) == cfg
        spec = cfg.to_spec()
        want = expected_tensors(spec)
        have = {n: a.shape for n, a in weights(name).items()}
        assert set(want) == set(have), name
        check_tensors(spec, have)
        assert len(spec.layers) == len(raw["layers"])
        for layer, entry in zip(spec.layers, raw["layers"]):
            assert layer.mixer.kind == entry["type"]
            assert (layer.feed_forward.kind == "none") == (entry["mlp"] is None)
    bad = json.loads(json.dumps(CONFIGS["mix"]))
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ConfigError, match="unsupported type"):
        VunasunConfig.from_dict(bad)
    bad = json.loads(json.dumps(CONFIGS["mix"]))
    bad["layers"][0]["mlp"]["kind"] = "routed"
    with pytest.raises(ConfigError, match="mlp kind"):
        VunasunConfig.from_dict(bad)
    bad = json.loads(json.dumps(CONFIGS["attn"]))
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    with pytest.raises(ConfigError, match="query heads"):
        VunasunConfig.from_dict(bad)
    bad = json.loads(json.dumps(CONFIGS["attn"]))
    del bad["norm"]
    with pytest.raises(ConfigError, match="eps"):
        VunasunConfig.from_dict(bad)


def test_a_rank_that_only_the_files_know():
    """The low rank of the decay of a ``gla`` layer is no configuration key: the spec leaves
    that size open and the stored tensors decide it."""
    from llmario_b200.config import VunasunConfig
    from llmario_b200.weights.loader import WeightError, check_tensors

    raw = json.loads(json.dumps(CONFIGS["gla"]))
    del raw["layers"][0]["mixer"]["rank"]
    spec = VunasunConfig.from_dict(raw).to_spec()
    have = {n: a.shape for n, a in weights("gla").items()}
    check_tensors(spec, have)
    have["l0.mix.q"] = (7, 64)
    with pytest.raises(WeightError, match="wrong shape"):
        check_tensors(spec, have)


def test_mask_code():
    from llmario_b200.kernels import KernelError, mask_code

    assert mask_code() == 0 and mask_code(window=5) == 5 and mask_code(chunk=12) == -12
    with pytest.raises(KernelError):
        mask_code(window=4, chunk=4)


def test_plain_recurrence_does_not_depend_on_the_cut():
    t = weights("gla")
    m = CONFIGS["gla"]["layers"][0]["mixer"]
    h = np.random.default_rng(3).standard_normal((23, CONFIGS["gla"]["width"]))
    whole, _ = VP.gla_mixer(h, t, "l0.mix.", m, 1e-5)
    a, S = VP.gla_mixer(h[:9], t, "l0.mix.", m, 1e-5)
    b, _ = VP.gla_mixer(h[9:], t, "l0.mix.", m, 1e-5, state=S)
    np.testing.assert_allclose(np.concatenate([a, b]), whole, rtol=1e-12, atol=1e-12)


# --------------------------------------------------------------------------------------------
# kernels alone
# --------------------------------------------------------------------------------------------
def _segments(rows_per_slot, n_slots, device):
    """row_slot of a step whose requests hold the given slots, and its segment table."""
    from llmario_b200 import kernels

    row_slot = torch.tensor([s for s, n in rows_per_slot for _ in range(n)], dtype=torch.int32,
                            device=device)
    seg = torch.full((n_slots, 3), -7, dtype=torch.int32, device=device)
    kernels.segment_table(row_slot, seg)
    return row_slot, seg


@pytest.mark.gpu
def test_segment_table():
    row_slot, seg = _segments([(3, 5), (0, 1), (2, 7)], 5, "cuda:0")
    table = seg.cpu().numpy()
    assert table[:, :2].tolist() == [[5, 6], [0, 0], [6, 13], [0, 5], [0, 0]]
    assert sorted(table[:3, 2].tolist()) == [0, 2, 3] and table[3:, 2].tolist() == [-1, -1]


@pytest.mark.gpu
@pytest.mark.parametrize("kind", (0, 1, 2))
@pytest.mark.parametrize("H,G,K,V", [(2, 2, 8, 4), (3, 3, 24, 16), (4, 2, 40, 24), (2, 1, 72, 20),
                                     (1, 1, 136, 33), (2, 2, 256, 16), (2, 2, 30, 7), (2, 1, 320, 12)])
def test_linear_recurrence_kernel(kind, H, G, K, V):
    """One kernel, three ways to make the decay, state rows of every register count, value
    channels that do not fill a block, several requests in a step and steps that carry on."""
    from llmario_b200 import kernels

    if kind != 2 and G != H:
        G = H
    dev = "cuda:0"
    rng = np.random.default_rng(K * 7 + V + kind)
    n_slots = 4
    state = torch.zeros(n_slots, H * V * K + 5, dtype=torch.float32, device=dev)
    S = np.zeros((n_slots, H, K, V))
    p0 = rng.uniform(-2, 0.5, H)
    p1 = rng.standard_normal(H)
    steps = [[(2, 19), (0, 1), (3, 33)], [(0, 1), (2, 1), (3, 1)], [(3, 2), (2, 40)]]
    for si, step in enumerate(steps):
        rows = sum(n for _, n in step)
        q = rng.standard_normal((rows, G * K))
        k = rng.standard_normal((rows, G * K)) * 0.3
        v = rng.standard_normal((rows, H * V))
        d = rng.standard_normal((rows, H)) if kind == 2 else rng.standard_normal((rows, H * K)) + 2
        if kind == 0:
            d = 1 / (1 + np.exp(-d))
        single = all(n == 1 for _, n in step)
        row_slot, seg = _segments(step, n_slots, dev)
        # operands as column slices of a wider matrix, as the mixers pass them
        wide = torch.zeros(rows, 2 * G * K + H * V + 3, dtype=torch.float32, device=dev)
        wide[:, :G * K] = torch.from_numpy(q)
        wide[:, G * K:2 * G * K] = torch.from_numpy(k)
        wide[:, 2 * G * K:2 * G * K + H * V] = torch.from_numpy(v)
        dd = torch.from_numpy(d).to(dev, torch.float32)
        out = torch.full((rows, H * V), float("nan"), dtype=torch.float32, device=dev)
        kernels.linear_recurrence(
            wide[:, :G * K], wide[:, G * K:2 * G * K], wide[:, 2 * G * K:2 * G * K + H * V], dd,
            state, out, row_slot, None if single else seg, H, G, K, V, kind, q_scale=0.5,
            exponent=0.25, rate_log=torch.from_numpy(p0).to(dev, torch.float32),
            step_bias=torch.from_numpy(p1).to(dev, torch.float32), n_requests=len(step))
        ref = np.zeros((rows, H, V))
        r = 0
        for slot, n in step:
            for _ in range(n):
                for h in range(H):
                    g = h // (H // G)
                    qq, kk = q[r, g * K:(g + 1) * K] * 0.5, k[r, g * K:(g + 1) * K]
                    vv = v[r, h * V:(h + 1) * V]
                    if kind == 2:
                        dt = np.logaddexp(0, d[r, h] + p1[h])
                        a, vv = np.exp(-np.exp(p0[h]) * dt), vv * dt
                    else:
                        a = d[r, h * K:(h + 1) * K]
                        if kind == 1:
                            a = (1 / (1 + np.exp(-a))) ** 0.25
                        a = a[:, None]
                    S[slot, h] = a * S[slot, h] + np.outer(kk, vv)
                    ref[r, h] = S[slot, h].T @ qq
                r += 1
        assert_close(out.cpu().numpy(), ref.reshape(rows, H * V), "float32", f"step {si}", 1e-5)
    got = state[:, :H * V * K].cpu().numpy().reshape(n_slots, H, V, K).transpose(0, 1, 3, 2)
    assert_close(got, S, "float32", "state", 1e-5)
    assert float(state[:, H * V * K:].abs().max()) == 0.0       # nothing written past the state
    assert float(state[1].abs().max()) == 0.0                   # a slot without rows stays as it was


@pytest.mark.gpu
@pytest.mark.parametrize("taps", (1, 2, 3, 4, 5))
def test_causal_convolution_with_history(taps):
    from llmario_b200 import kernels

    dev, C, n_slots = "cuda:0", 70, 3
    rng = np.random.default_rng(taps)
    w, b = rng.standard_normal((C, taps)), rng.standard_normal(C)
    hist = torch.zeros(n_slots, 11 + C * (taps - 1), dtype=torch.float32, device=dev)
    seen = {s: np.zeros((taps - 1, C)) for s in range(n_slots)}    # inputs so far, zeros before
    for step in ([(1, 9), (0, 2)], [(0, 1), (1, 1)], [(1, 1), (0, 6)], [(0, 1)], [(1, 2), (0, 37)],
                 [(0, 3), (1, 290)], [(1, 1), (0, 1)]):        # (many rows: a thread walks a strip)
        rows = sum(n for _, n in step)
        x = rng.standard_normal((rows, C))
        row_slot, seg = _segments(step, n_slots, dev)
        single = all(n == 1 for _, n in step)
        src = torch.zeros(rows, C + 4, dtype=torch.float32, device=dev)
        src[:, 2:2 + C] = torch.from_numpy(x)
        out = torch.empty(rows, C, dtype=torch.float32, device=dev)
        kernels.causal_conv_silu(src[:, 2:2 + C], torch.from_numpy(w).to(dev, torch.float32),
                                 torch.from_numpy(b).to(dev, torch.float32), hist[:, 11:], out,
                                 row_slot, None if single else seg)
        ref = np.zeros((rows, C))
        r = 0
        for slot, n in step:
            for _ in range(n):
                seen[slot] = np.concatenate([seen[slot], x[r:r + 1]])
                z = b + sum(w[:, taps - 1 - j] * seen[slot][-1 - j] for j in range(taps))
                ref[r] = z / (1 + np.exp(-z))
                r += 1
        assert_close(out.cpu().numpy(), ref, "float32", "convolution", 1e-5)
    assert float(hist[:, :11].abs().max()) == 0.0 and float(hist[2].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
def test_elementwise_kernels_of_the_block(dtype):
    from llmario_b200 import kernels

    dev = "cuda:0"
    rng = np.random.default_rng(5)
    rows, width = 37, 100
    # norm of the sublayer's output, scale, residual sum
    y, w, s, x = (rng.standard_normal(sh) for sh in ((rows, width), width, width, (rows, width)))
    xt = torch.from_numpy(x).to(dev, torch.float32)
    h16 = torch.zeros(rows, width, dtype=torch.bfloat16, device=dev)
    kernels.norm_scale_add(torch.from_numpy(y).to(dev, torch.float32),
                           torch.from_numpy(w).to(dev, torch.float32),
                           torch.from_numpy(s).to(dev, torch.float32), xt, 1e-3, rounded=h16)
    assert_close(xt.cpu().numpy(), x + VP.rms_norm(y, w, 1e-3) * s, "float32", "norm_scale_add", 1e-5)
    assert torch.equal(h16, xt.to(torch.bfloat16))          # the next sublayer's input beside it
    # rounding a column slice
    out = torch.zeros(rows, 40, dtype=dtype, device=dev)
    kernels.cast_rows(xt[:, 13:53], out)
    assert torch.equal(out, xt[:, 13:53].to(dtype))
    # the decay of gated linear attention from its projection
    z, zb = rng.standard_normal((rows, 24)) * 3, rng.standard_normal(24)
    zt = torch.from_numpy(z).to(dev, torch.float32)
    kernels.bias_sigmoid_pow(zt, torch.from_numpy(zb).to(dev, torch.float32), 1 / 16)
    assert_close(zt.cpu().numpy(), VP.sigmoid(z + zb) ** (1 / 16), "float32", "bias_sigmoid_pow", 1e-6)
    # gate per head
    H, hd = 3, 20
    o = torch.from_numpy(rng.standard_normal((rows, H * hd))).to(dev, dtype)
    gate = torch.from_numpy(rng.standard_normal((rows, H + 5))).to(dev, torch.float32)
    ref = o.double().cpu().numpy().reshape(rows, H, hd) * VP.sigmoid(gate[:, 2:2 + H].double().cpu().numpy())[:, :, None]
    kernels.head_gate(o, gate[:, 2:2 + H], H, hd, clear=True)
    assert_close(o.float().cpu().numpy(), ref.reshape(rows, H * hd), "float32", "head_gate",
                 1e-5 if dtype == torch.float32 else 8e-3)
    assert float(gate[:, 2:2 + H].abs().max()) == 0.0 and float(gate[:, :2].abs().min()) > 0.0
    # gate and group norm behind the recurrence, both orders, with and without the direct path
    # (channels in fours and not: the kernel reads 16-byte pieces where it can; a group larger
    # than what a thread keeps in registers)
    for groups, group, head in ((4, 30, 24), (3, 64, 16), (1, 9 * 1024, 48)):
      ch = groups * group
      oo, xx, gg = (rng.standard_normal((rows, ch)) for _ in range(3))
      skip = rng.standard_normal(ch // head)
      for gate_first, wt, use_skip in ((True, rng.standard_normal(ch), True),
                                       (False, rng.standard_normal(group), False)):
          yy = oo + (np.repeat(skip, head) * xx if use_skip else 0)
          gate_v = gg / (1 + np.exp(-gg))
          if gate_first:
              ref = VP.rms_unit((yy * gate_v).reshape(rows, groups, group), 1e-4).reshape(rows, ch) * wt
          else:
              ref = VP.rms_unit(yy.reshape(rows, groups, group), 1e-4).reshape(rows, ch) \
                  * np.tile(wt, groups) * gate_v
          res = torch.empty(rows, ch, dtype=dtype, device=dev)
          f = lambda a: torch.from_numpy(a).to(dev, torch.float32)
          kernels.gated_group_norm(f(oo), f(gg), f(wt), res, group, 1e-4, gate_first,
                                   skip=f(skip) if use_skip else None,
                                   skip_input=f(xx) if use_skip else None, head=head)
          assert_close(res.float().cpu().numpy(), ref, "float32", "gated_group_norm",
                       1e-5 if dtype == torch.float32 else 8e-3)


# --------------------------------------------------------------------------------------------
# the model through the step function
# --------------------------------------------------------------------------------------------
def run_steps(runner, steps):
    """``steps``: lists of (request, tokens, wanted places).  Returns request -> {position: logits}."""
    from llmario_b200.engine.step import StepEntry

    got = {}
    for step in steps:
        entries = [StepEntry(r, list(t), list(w)) for r, t, w in step]
        starts = {r: (runner.length(r) if runner.cache.has(r) else 0) for r, _, _ in step}
        logits = runner.step(entries).cpu().numpy()
        i = 0
        for r, _, want in step:
            for wpos in want:
                got.setdefault(r, {})[starts[r] + wpos] = logits[i].copy()
                i += 1
    return got


def check_request(got, name, tokens, dtype, what, seed=0):
    ref = plain_logits(name, tokens, seed)
    pos = sorted(got)
    # 16-bit operands move the inputs of every layer by a rounding: a position gets, on top of
    # the bound, three times what such a move does to it in the plain implementation
    slack = 3.0 * sensitivity(name, tokens, seed)[pos] if dtype == "bfloat16" else None
    assert_close(np.stack([got[p] for p in pos]), ref[pos], dtype, what, slack=slack)


NAMES = sorted(CONFIGS)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt(name, dtype):
    """Every position of a prompt that spans several pages and chunks, the first tokens included."""
    toks = tokens_for(name, 110, 1)
    runner = runner_for(name, dtype)
    got = run_steps(runner, [[("a", toks, range(len(toks)))]])
    check_request(got["a"], name, toks, dtype, "whole prompt")
    runner.cache.check_invariants()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens(name, dtype):
    """A prompt, then tokens one by one through recorded steps: across page and chunk borders."""
    toks = tokens_for(name, 90, 2)
    n = 21
    runner = runner_for(name, dtype)
    steps = [[("a", toks[:n], [0, n - 1])]] + [[("a", [t], [0])] for t in toks[n:]]
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, "prompt, then single tokens")
    assert runner.counters["graph_replays"] > 40


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_many_sizes(name, dtype):
    """Portions cut in the middle of pages and chunks, down to two tokens; then single tokens."""
    toks = tokens_for(name, 120, 3)
    cuts = [2, 3, 2, 17, 2, 31, 5, 2, 29, 1, 2, 1, 1, 16, 2, 4]
    assert sum(cuts) == len(toks)
    steps, at = [], 0
    for c in cuts:
        steps.append([("a", toks[at:at + c], range(c))])
        at += c
    runner = runner_for(name, dtype)
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, "portions")
    # and the cut does not matter beyond rounding: the same prompt whole
    whole = run_steps(runner_for(name, dtype), [[("a", toks, range(len(toks)))]])
    a = np.stack([got["a"][p] for p in range(len(toks))])
    b = np.stack([whole["a"][p] for p in range(len(toks))])
    assert_close(a, b.astype(np.float64), dtype, "portions against whole",
                 1e-5 if dtype == "float32" else 2e-2,
                 slack=3.0 * sensitivity(name, toks) if dtype == "bfloat16" else None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("mix", "recurrent_only", "attn_tc", "ssm_groups"))
def test_mixed_batches_and_reused_slots(name, dtype):
    """Four request slots, six requests of unequal lengths: portions of some beside single tokens
    of others, requests that pause, requests that end and whose slot and pages the next one
    takes.  Every request must get what it gets alone (the plain implementation's logits)."""
    lengths = {"a": 70, "b": 9, "c": 41, "d": 33, "e": 52, "f": 2}
    toks = {r: tokens_for(name, n, 10 + i) for i, (r, n) in enumerate(lengths.items())}
    runner = runner_for(name, dtype, page_size=8, cache_tokens=208, max_requests=4)
    at = {r: 0 for r in toks}

    def take(r, n):
        n = min(n, lengths[r] - at[r])
        part = toks[r][at[r]:at[r] + n]
        at[r] += n
        return (r, part, range(n))

    plan = [[("a", 30), ("b", 2)], [("a", 1), ("b", 1), ("c", 17)], [("b", 6), ("c", 1), ("d", 2)],
            [("a", 1), ("c", 23), ("d", 1)], [("a", 38)], [("d", 30), ("e", 3)],
            [("e", 1), ("f", 2)], [("e", 48)]]
    got = {}
    for step in plan:
        entries = [take(r, n) for r, n in step]
        for r, res in run_steps(runner, [entries]).items():
            got.setdefault(r, {}).update(res)
        for r, _ in step:
            if at[r] == lengths[r]:
                runner.close(r)
        runner.cache.check_invariants()
    assert all(at[r] == lengths[r] for r in toks)
    for r in toks:
        assert sorted(got[r]) == list(range(lengths[r]))
        check_request(got[r], name, toks[r], dtype, f"request {r}", seed=0)
    assert runner.cache.free_slots() == 4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("attn_g8", "attn_g3", "attn_tc", "mix"))
def test_a_long_prompt_over_many_chunks_and_the_engine_page(name, dtype):
    """A prompt of several tensor-core tiles with the engine's default page of 64, then a second
    portion that starts inside a chunk and a page, then single tokens."""
    toks = tokens_for(name, 420, 6)
    runner = runner_for(name, dtype, page_size=64, cache_tokens=1024)
    steps = [[("a", toks[:333], range(333))], [("a", toks[333:410], range(77))]] \
        + [[("a", [t], [0])] for t in toks[410:]]
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, "long prompt")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_from_a_seed(seed, dtype):
    """Layers of any kind in any order with sizes drawn from a seed, the engine's page of 64:
    a prompt in portions, then single tokens, against the plain implementation."""
    name = random_config(seed)
    toks = tokens_for(name, 230, 7)
    runner = runner_for(name, dtype, page_size=64, cache_tokens=512)
    steps = [[("a", toks[:150], range(150))], [("a", toks[150:153], range(3))],
             [("a", toks[153:200], range(47))]] + [[("a", [t], [0])] for t in toks[200:]]
    got = run_steps(runner, steps)
    check_request(got["a"], name, toks, dtype, f"{name} {CONFIGS[name]['layers']}")


@pytest.mark.gpu
@pytest.mark.parametrize("name", ("mix", "recurrent_only", "gla_big_key"))
def test_long_decoding(name):
    """Hundreds of single tokens behind a one-token prompt: the state carries what no cache holds."""
    toks = tokens_for(name, 260, 4)
    runner = runner_for(name, "float32", page_size=32, cache_tokens=512)
    got = run_steps(runner, [[("a", [t], [0])] for t in toks])
    check_request(got["a"], name, toks, "float32", "long decoding")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk,page", [(40, 16), (64, 64), (24, 32)])
def test_a_key_that_stands_out_at_the_edges_of_chunks(dtype, chunk, page):
    """Needles at the first and last place of every chunk, probes on either side of the edges,
    in a whole prompt and decoded one by one, with pages smaller, equal and larger than a chunk."""
    name = needle_model(chunk)
    rng = np.random.default_rng(chunk)
    n = 4 * chunk + 9
    toks = [int(t) for t in rng.integers(2, 64, n)]
    for c in range(0, n, chunk):           # needles at the first and last place of every chunk,
        for p in (c, c + chunk - 1):       # probes right behind them on either side of the edge
            if p < n:
                toks[p] = 0
        for p in (c + 1, c + 2, c + chunk - 2, c + chunk // 2):
            if p < n:
                toks[p] = 1
    ref = plain_logits(name, toks)
    # the probes' logits do depend on the needles they see: moving the edge by one would show
    moved = json.loads(json.dumps(CONFIGS[name]))
    moved["layers"][0]["mixer"]["mask"]["size"] = chunk + 1
    other = VP.forward(moved, weights(name), toks)
    assert np.abs(other - ref).max() > 0.2 * np.abs(ref).max()
    runner = runner_for(name, dtype, page_size=page, cache_tokens=512)
    whole = run_steps(runner, [[("w", toks, range(n))]])
    check_request(whole["w"], name, toks, dtype, "needles, whole prompt")
    half = n // 2 + 3
    steps = [[("d", toks[:half], range(half))]] + [[("d", [t], [0])] for t in toks[half:]]
    dec = run_steps(runner, steps)
    check_request(dec["d"], name, toks, dtype, "needles, decoded")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_engine(dtype):
    """The engine's own entry point and scheduler: prompts of unequal lengths, more requests than
    slots, greedy tokens.  The plain implementation, reading the engine's sequence, must choose
    the same token wherever its two best logits are clearly apart."""
    from llmario_b200.engine.engine import Engine
    from llmario_b200.sampling import SamplingParams

    for name in ("mix", "recurrent_only"):
        eng = Engine(model_dir(name), dtype=dtype, page_size=16, cache_tokens=1024, max_requests=2,
                     token_budget=48, context=256)
        prompts = [tokens_for(name, n, 20 + i) for i, n in enumerate((5, 70, 33, 1, 18))]
        outs = eng.generate(prompts, SamplingParams.greedy_params(max_tokens=24, ignore_eos=True))
        margin = 1e-3 if dtype == "float32" else 8e-2
        clear = 0
        for p, o in zip(prompts, outs):
            assert len(o) == 24
            ref = plain_logits(name, list(p) + list(o))
            for j, tok in enumerate(o):
                l = ref[len(p) - 1 + j]
                top = np.sort(l)[-2:]
                if top[1] - top[0] > margin * np.abs(l).max():
                    clear += 1
                    assert tok == int(np.argmax(l)), f"{name}: token {j} of a request"
        assert clear > 60
        assert eng.stats()["graph_replays"] > 0
        eng.runner.cache.check_invariants()


@pytest.mark.gpu
def test_command_line_and_trace_runner(tmp_path):
    """The two programs a user starts: ``llmario-b200 run`` on a Vunasun model folder (greedy ids
    against the plain implementation) and ``bin/trace_run`` (given tokens in steps, logits in
    files), which choose the model class by ``config.json``."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "mix"
    prompt = tokens_for(name, 19, 40)
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "llmario-b200"), "run",
                        model_dir(name), "--tokens", ",".join(map(str, prompt)), "--max-tokens", "6",
                        "--dtype", "float32", "--page-size", "16", "--context", "128"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]
    assert len(out) == 6
    ref = plain_logits(name, prompt + out)
    for j, tok in enumerate(out):
        l = ref[len(prompt) - 1 + j]
        top = np.sort(l)[-2:]
        if top[1] - top[0] > 1e-3 * np.abs(l).max():
            assert tok == int(np.argmax(l))
    # a preset name gives a model with random weights
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "llmario-b200"), "run", "vunasun-tiny",
                        "--prompt-len", "5", "--n", "6", "--dtype", "bfloat16", "--page-size", "16",
                        "--context", "64"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len(p.stdout.strip().splitlines()[-1].split(",")) == 6
    # the trace runner: two requests, portions beside single tokens, a slot given back and taken
    a, b, c = (tokens_for(name, n, 50 + i) for i, n in enumerate((40, 7, 12)))
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [0, 24]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[25:26], "want": [0]},
                                {"id": "b", "tokens": b, "want": [6]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[26:], "want": [13]},
                                {"id": "c", "tokens": c[:2], "want": []}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "c", "tokens": c[2:], "want": [0, 9]}], "end": ["c"]},
    ]
    out_dir = tmp_path / "out"
    p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", model_dir(name), "--dtype",
                        "float32", "--out", str(out_dir), "--max-tokens", "192"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb, rc = plain_logits(name, a), plain_logits(name, b), plain_logits(name, c)
    want = {0: np.stack([ra[0], ra[24]]), 1: np.stack([ra[25], rb[6]]), 2: ra[39:40],
            3: np.stack([rc[2], rc[11]])}
    for i, ref in want.items():
        got = np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(ref.shape)
        assert_close(got, ref, "float32", f"trace step {i}")
