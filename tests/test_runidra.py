"""The Runidra decoder against the plain float64 implementation (tests/plain/runidra_plain.py):
every mechanism alone and together, in whole prompts, portions, single decoded tokens, mixed
batches, reused slots and pages, and through the engine's own entry point."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

from plain import runidra_plain as RP
from runidra_util import (CLOSE_CALL, CONFIGS, CUSTOM, _bf16_values, _weights, assert_close, config,
                          latent, model_dir, plain_logits, random_config, router_margins,
                          runner_for, slack_for, tokens_for, weights)

DTYPES = ("float32", "bfloat16")


# --------------------------------------------------------------------------------------------
# no GPU: configuration, and the plain implementation against itself
# --------------------------------------------------------------------------------------------
def test_configuration_round_trip_and_tensor_names():
    from llmario_b200.config import ConfigError, RunidraConfig, resolve_architecture
    from llmario_b200.weights.loader import check_tensors, expected_tensors

    for name, raw in CONFIGS.items():
        assert resolve_architecture(raw) == "Runidra"
        cfg = RunidraConfig.from_dict(raw)
        assert RunidraConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.to_dict() == raw, name
        spec = cfg.to_spec()
        want = expected_tensors(spec)
        have = {n: a.shape for n, a in weights(name).items()}
        assert set(want) == set(have), name
        check_tensors(spec, have)
        assert [c.layer for c in spec.run_order] == RP.run_order(raw)
        assert spec.residual_streams == raw.get("streams")
        for layer, entry in zip(spec.layers, raw["layers"]):
            assert layer.mixer.kind == entry["type"]
            assert (layer.feed_forward.kind == "none") == (entry["mlp"] is None)
    bad = json.loads(json.dumps(CONFIGS["mix"]))
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ConfigError, match="unsupported type"):
        RunidraConfig.from_dict(bad)
    bad = json.loads(json.dumps(CONFIGS["mix"]))
    bad["layers"][0]["mlp"]["kind"] = "routed"
    with pytest.raises(ConfigError, match="mlp kind"):
        RunidraConfig.from_dict(bad)
    bad = json.loads(json.dumps(CONFIGS["mix"]))
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        RunidraConfig.from_dict(bad)
    bad = json.loads(json.dumps(CONFIGS["experts"]))
    bad["layers"][0]["mlp"]["router"]["top"] = 7
    with pytest.raises(ConfigError, match="top"):
        RunidraConfig.from_dict(bad)
    bad = json.loads(json.dumps(CONFIGS["latent"]))
    del bad["norm"]
    with pytest.raises(ConfigError, match="eps"):
        RunidraConfig.from_dict(bad)


def test_plain_memory_keeps_its_gates_in_range():
    """The running maximum keeps the exponentials of the gates at or below one, and the matrix
    memory's answer does not change when a long prefix is replayed in front of a suffix."""
    cfg = CONFIGS["memory"]
    w = weights("memory")
    toks = tokens_for("memory", 300, 5)
    z = RP.forward(cfg, w, toks)
    assert np.isfinite(z).all() and np.abs(z).max() <= cfg["logit_softcap"]


def test_plain_sink_and_window_matter():
    """The plain statement itself: the sink and the window's edge move the logits."""
    name = needle_model(12)
    cfg, w = CONFIGS[name], weights(name)
    toks, probes = needle_tokens(12, 80)
    ref = RP.forward(cfg, w, toks)
    off = json.loads(json.dumps(cfg))
    off["layers"][0]["mixer"]["mask"]["size"] = 13
    moved = RP.forward(off, w, toks)
    d = np.abs(moved - ref).max(axis=1)
    assert d[probes["just_outside"]].min() > 0.15 * np.abs(ref).max()
    w2 = {k: v for k, v in w.items() if not k.endswith("sink")}
    assert np.abs(RP.forward(cfg, w2, toks) - ref).max() > 0.05 * np.abs(ref).max()


# --------------------------------------------------------------------------------------------
# kernels of the mechanisms, each against a few lines of NumPy
# --------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("S,width,rows", [(1, 40, 3), (2, 64, 70), (3, 100, 9), (4, 4096, 5), (8, 24, 2)])
@pytest.mark.parametrize("out_dtype", (torch.float32, torch.bfloat16))
def test_stream_step_kernel(S, width, rows, out_dtype):
    from llmario_b200 import kernels

    rng = np.random.default_rng(S * 100 + width)
    xs = rng.standard_normal((S, rows, width))
    y = rng.standard_normal((rows, width))
    mix, cout, cin = rng.standard_normal((S, S)), rng.standard_normal(S), rng.standard_normal(S)
    gain = 1 + 0.1 * rng.standard_normal(width)
    dev = lambda a: torch.tensor(a, dtype=torch.float32, device="cuda")
    new = np.einsum("st,srw->trw", mix, xs) + cout[:, None, None] * y[None]
    u = np.einsum("s,srw->rw", cin, new)
    normed = u / np.sqrt((u * u).mean(-1, keepdims=True) + 1e-5) * gain
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    # write and read in one launch
    x_d, y_d = dev(xs), dev(y)
    out = torch.empty(rows, width, dtype=out_dtype, device="cuda")
    kernels.stream_step(x_d, y=y_d, mix=dev(mix), out_coef=dev(cout), clear_y=True, in_coef=dev(cin),
                        weight=dev(gain), eps=1e-5, out=out)
    np.testing.assert_allclose(x_d.cpu().numpy(), new, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(out.float().cpu().numpy(), normed, rtol=tol, atol=tol)
    assert float(y_d.abs().max()) == 0.0
    # the two halves apart, the read at chosen rows
    x_d, y_d = dev(xs), dev(y)
    kernels.stream_step(x_d, y=y_d, mix=dev(mix), out_coef=dev(cout))
    np.testing.assert_allclose(x_d.cpu().numpy(), new, rtol=1e-5, atol=1e-5)
    assert float((y_d - dev(y)).abs().max()) == 0.0
    index = torch.tensor([rows - 1, 0], dtype=torch.int32, device="cuda")
    out = torch.empty(2, width, dtype=out_dtype, device="cuda")
    kernels.stream_step(x_d, in_coef=dev(cin), weight=dev(gain), eps=1e-5, out=out, rows_index=index)
    np.testing.assert_allclose(out.float().cpu().numpy(), normed[[rows - 1, 0]], rtol=tol, atol=tol)
    x_d = dev(xs)
    kernels.stream_fill(x_d)
    assert all(torch.equal(x_d[s], x_d[0]) for s in range(S))


@pytest.mark.gpu
@pytest.mark.parametrize("H,cap", [(1, 15.0), (3, 4.0), (6, 0.0)])
def test_log_gate_scan_kernel(H, cap):
    """Gates over steps of unequal requests, the running maximum carried in the state slot."""
    from llmario_b200 import kernels

    rng = np.random.default_rng(H)
    n_slots = 4
    m_state = torch.zeros(n_slots, H + 5, dtype=torch.float32, device="cuda")
    ref_m = np.zeros((n_slots, H))
    bi, bf = rng.standard_normal(H), rng.standard_normal(H) + 1
    soft = (lambda z: cap * np.tanh(z / cap)) if cap else (lambda z: z)
    for rows_per_slot in ([(2, 70), (0, 3)], [(0, 1), (2, 1), (3, 1)], [(3, 40), (2, 33), (0, 2)]):
        rows = sum(n for _, n in rows_per_slot)
        z = 3 * rng.standard_normal((rows, 2 * H + 3))
        row_slot = np.concatenate([[s] * n for s, n in rows_per_slot]).astype(np.int32)
        single = all(n == 1 for _, n in rows_per_slot)
        want = np.zeros((rows, 3 * H))
        r = 0
        for s, n in rows_per_slot:
            for _ in range(n):
                gi = soft(z[r, 1:1 + H] + bi)
                gf = RP.log_sigmoid(soft(z[r, 1 + H:1 + 2 * H] + bf))
                new = np.maximum(gf + ref_m[s], gi)
                want[r] = np.concatenate([np.exp(gf + ref_m[s] - new), np.exp(gi - new), new])
                ref_m[s] = new
                r += 1
        z_d = torch.tensor(z, dtype=torch.float32, device="cuda")
        slot_d = torch.tensor(row_slot, device="cuda")
        seg = None
        if not single:
            seg = torch.empty(n_slots, 3, dtype=torch.int32, device="cuda")
            kernels.segment_table(slot_d, seg)
        out = torch.empty(rows, 3 * H, dtype=torch.float32, device="cuda")
        kernels.log_gate_scan(z_d[:, 1:1 + H], z_d[:, 1 + H:1 + 2 * H],
                              torch.tensor(bi, dtype=torch.float32, device="cuda"),
                              torch.tensor(bf, dtype=torch.float32, device="cuda"), cap,
                              m_state[:, 5:], out, slot_d, seg, H, n_requests=len(rows_per_slot))
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=2e-5, atol=1e-6)
        np.testing.assert_allclose(m_state[:, 5:].cpu().numpy(), ref_m, rtol=1e-5, atol=1e-6)
    assert float(m_state[:, :5].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("E,top", [(3, 1), (6, 2), (16, 4), (70, 8), (5, 5)])
def test_route_kernel(E, top):
    from llmario_b200 import kernels

    rng = np.random.default_rng(E)
    rows = 37
    z = rng.standard_normal((rows, E + 2)) * 2
    z[3, :E] = 0.5                    # all equal: the lowest indices win
    z_d = torch.tensor(z, dtype=torch.float32, device="cuda")
    ids = torch.empty(rows, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(rows, top, dtype=torch.float32, device="cuda")
    kernels.moe_route(z_d[:, :E], E, top, ids, wts)
    zf = z_d[:, :E].cpu().numpy().astype(np.float64)
    for r in range(rows):
        chosen = np.argsort(-zf[r], kind="stable")[:top]
        assert ids[r].cpu().tolist() == chosen.tolist(), r
        w = np.exp(zf[r][chosen] - zf[r][chosen].max())
        np.testing.assert_allclose(wts[r].cpu().numpy(), w / w.sum(), rtol=1e-5)
    # the product and the choice in one launch: logits of 32-bit weights, one row more than experts
    for dtype, width in ((torch.float32, 50), (torch.bfloat16, 256)):
        h = torch.tensor(rng.standard_normal((rows, width)), dtype=dtype, device="cuda")
        w = torch.tensor(rng.standard_normal((E + 1, width)), dtype=torch.float32, device="cuda")
        b = torch.tensor(rng.standard_normal(E + 1), dtype=torch.float32, device="cuda")
        z2 = torch.empty(rows, E + 1, dtype=torch.float32, device="cuda")
        kernels.moe_router(h, w, b, E, top, z2, ids, wts)
        ref = h.double().cpu().numpy() @ w.double().cpu().numpy().T + b.double().cpu().numpy()
        np.testing.assert_allclose(z2.cpu().numpy(), ref, rtol=1e-4, atol=1e-4)
        zf = z2[:, :E].cpu().numpy().astype(np.float64)
        for r in range(rows):
            chosen = np.argsort(-zf[r], kind="stable")[:top]
            assert ids[r].cpu().tolist() == chosen.tolist(), r
            w_ = np.exp(zf[r][chosen] - zf[r][chosen].max())
            np.testing.assert_allclose(wts[r].cpu().numpy(), w_ / w_.sum(), rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
def test_head_linear_and_gated_activation(dtype):
    from llmario_b200 import kernels

    rng = np.random.default_rng(3)
    for rows, H, k, n in ((5, 3, 10, 7), (70, 4, 32, 96), (300, 2, 96, 48), (300, 3, 64, 128),
                          (1000, 16, 96, 96), (200, 5, 24, 256)):
        a = torch.tensor(rng.standard_normal((rows, H, k + 8)), dtype=dtype, device="cuda")
        w = torch.tensor(rng.standard_normal((H, n, k)), dtype=dtype, device="cuda")
        out = torch.zeros(rows, H, n + 8, dtype=dtype, device="cuda")
        kernels.head_linear(a[:, :, :k], w, out[:, :, :n])
        ref = np.einsum("rhk,hnk->rhn", a[:, :, :k].double().cpu().numpy(), w.double().cpu().numpy())
        tol = 1e-4 if dtype == torch.float32 else 0.1
        np.testing.assert_allclose(out[:, :, :n].double().cpu().numpy(), ref, rtol=tol, atol=tol)
        assert float(out[:, :, n:].abs().max()) == 0.0
    gu = torch.tensor(rng.standard_normal((9, 2 * 21)) * 2, dtype=torch.float32, device="cuda")
    bias = torch.tensor(rng.standard_normal(2 * 21), dtype=torch.float32, device="cuda")
    g, u = (gu + bias)[:, :21].double().cpu().numpy(), (gu + bias)[:, 21:].double().cpu().numpy()
    for act, fn in (("gelu_tanh", RP.gelu_tanh), ("silu", RP.silu)):
        out = torch.empty(9, 21, dtype=dtype, device="cuda")
        kernels.gated_act(gu, bias, out, act)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        np.testing.assert_allclose(out.double().cpu().numpy(), fn(g) * u, rtol=tol, atol=tol)
    z = torch.tensor(rng.standard_normal((4, 33)) * 20, dtype=torch.float32, device="cuda")
    ref = 7.0 * np.tanh(z.double().cpu().numpy() * 1.5 / 7.0)
    kernels.scale_soft_cap(z, 1.5, 7.0)
    np.testing.assert_allclose(z.cpu().numpy(), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,E,top,width,ff", [(3, 4, 2, 64, 32), (70, 6, 3, 96, 48), (700, 8, 2, 128, 80),
                                                 (40, 16, 1, 64, 16)])
def test_grouped_experts_against_numpy(rows, E, top, width, ff):
    """Sorting by expert, the two grouped tensor-core products and the weighted sum, against a
    few lines of NumPy on the same 16-bit values; the row-wise kernels against the same."""
    from llmario_b200 import kernels

    rng = np.random.default_rng(rows + E)
    b16 = lambda a: torch.tensor(a, dtype=torch.bfloat16, device="cuda")
    h, gu, dn = b16(rng.standard_normal((rows, width))), b16(rng.standard_normal((E, 2 * ff, width)) / 8), \
        b16(rng.standard_normal((E, width, ff)) / 8)
    ids = torch.tensor(np.stack([rng.permutation(E)[:top] for _ in range(rows)]), dtype=torch.int32,
                       device="cuda")
    wts = torch.tensor(rng.random((rows, top)), dtype=torch.float32, device="cuda")
    shared = torch.tensor(rng.standard_normal((rows, width)), dtype=torch.float32, device="cuda")
    gate = torch.tensor(rng.standard_normal((rows, 3)), dtype=torch.float32, device="cuda")
    hf, guf, dnf = h.double().cpu().numpy(), gu.double().cpu().numpy(), dn.double().cpu().numpy()
    ref = np.zeros((rows, width))
    for r in range(rows):
        for k in range(top):
            e = int(ids[r, k])
            a = RP.silu(guf[e, :ff] @ hf[r]) * (guf[e, ff:] @ hf[r])
            a = torch.tensor(a).to(torch.bfloat16).double().numpy()        # the activation is rounded
            ref[r] += float(wts[r, k]) * (dnf[e] @ a)
    ref += RP.sigmoid(gate[:, 1].double().cpu().numpy())[:, None] * shared.double().cpu().numpy()
    # grouped
    pairs = rows * top
    bn = kernels.moe_tile(pairs, E)
    tiles = -(-pairs // bn) + E
    pos = torch.empty(pairs, dtype=torch.int32, device="cuda")
    tile_group = torch.empty(tiles, dtype=torch.int32, device="cuda")
    kernels.moe_align(ids, E, bn, pos, tile_group)
    p, tg = pos.cpu().numpy(), tile_group.cpu().numpy()
    assert len(set(p.tolist())) == pairs and p.max() < tiles * bn
    assert all(tg[p[i] // bn] == int(ids.view(-1)[i]) for i in range(pairs))
    xp = torch.full((tiles * bn, width), float("nan"), dtype=torch.bfloat16, device="cuda")
    kernels.moe_gather(h, pos, xp, top)
    act = torch.empty(tiles * bn, ff, dtype=torch.bfloat16, device="cuda")
    kernels.gemm_grouped(xp, gu, act, tile_group, bn, gated=True)
    d = torch.empty(tiles * bn, width, dtype=torch.float32, device="cuda")
    kernels.gemm_grouped(act, dn, d, tile_group, bn, gated=False)
    y = torch.ones(rows, width, dtype=torch.float32, device="cuda")
    kernels.moe_combine(d, pos, wts, y, True, shared, gate[:, 1])
    tol = 0.03 * np.abs(ref).max()
    np.testing.assert_allclose(y.cpu().numpy() - 1.0, ref, atol=tol)
    kernels.check_tc_status(h.device)
    # row-wise
    act2 = torch.empty(rows, top, ff, dtype=torch.bfloat16, device="cuda")
    kernels.moe_gate_up_rows(h, gu, ids, act2)
    y2 = torch.empty(rows, width, dtype=torch.float32, device="cuda")
    kernels.moe_down_rows(act2, dn, ids, wts, y2, False, shared, gate[:, 1])
    np.testing.assert_allclose(y2.cpu().numpy(), ref, atol=tol)


# --------------------------------------------------------------------------------------------
# whole models through the step function
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
    # 16-bit operands move the inputs of every layer by a rounding: see slack_for
    slack = slack_for(name, tokens, dtype, seed)
    assert_close(np.stack([got[p] for p in pos]), ref[pos], dtype, what,
                 slack=None if slack is None else slack[pos])


NAMES = sorted(CONFIGS)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt(name, dtype):
    """Every position of a prompt that spans several pages and windows, the first tokens included."""
    toks = tokens_for(name, 110, 1)
    runner = runner_for(name, dtype)
    got = run_steps(runner, [[("a", toks, range(len(toks)))]])
    check_request(got["a"], name, toks, dtype, "whole prompt")
    runner.cache.check_invariants()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens(name, dtype):
    """A prompt, then tokens one by one through recorded steps: across page and window borders."""
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
    """Portions cut in the middle of pages and windows, down to two tokens; then single tokens."""
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
                 1e-5 if dtype == "float32" else 2e-2, slack=slack_for(name, toks, dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("mix", "loop_all", "latent_tc", "latent_h16", "odd", "experts_tc"))
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
@pytest.mark.parametrize("name", ("latent_tc", "mix", "experts", "experts_tc"))
def test_a_long_prompt_over_many_windows_and_the_engine_page(name, dtype):
    """A prompt of several hundred tokens with the engine's default page of 64, then a second
    portion that starts inside a window and a page, then single tokens."""
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
@pytest.mark.parametrize("name", ("mix", "memory_big_key", "loop_all"))
def test_long_decoding(name):
    """Hundreds of single tokens behind a one-token prompt: the state carries what no cache
    holds, and windows pass over decoded tokens many times."""
    toks = tokens_for(name, 260, 4)
    runner = runner_for(name, "float32", page_size=32, cache_tokens=512)
    got = run_steps(runner, [[("a", [t], [0])] for t in toks])
    check_request(got["a"], name, toks, "float32", "long decoding")


# --------------------------------------------------------------------------------------------
# a key that stands out: the window's edges and the sink
# --------------------------------------------------------------------------------------------
def needle_model(window: int) -> str:
    """A latent-attention layer whose weights make one score stand out.  Token 0 is the needle:
    its latent is one large direction, which head 0's key map turns into a key that the probe's
    (token 1's) query points along; every other token has neither.  A probe's output is then
    decided by whether its window still holds a needle, so an edge that is off by one shows as a
    large error.  The sinks are large enough to take visible weight."""
    name = f"needle{window}"
    if name not in CONFIGS:
        CONFIGS[name] = config([latent(heads=2, dim=16, rot_dim=8, vdim=24, q_rank=16, kv_rank=32,
                                       window=window, scale=1.0)], width=64, vocab=64, streams=2)
        w = {n: a.copy() for n, a in _weights(CONFIGS[name], 7).items()}
        w["embed"][:, :2] = 0.0
        w["embed"][0, 0] = 8.0
        w["embed"][1, 1] = 8.0
        x = "l0.mix."
        for m in ("dq", "dkv"):
            w[x + m] *= 0.25
            w[x + m][:, :2] = 0.0
        w[x + "dkv"][5, 0] = 6.0        # the needle's latent: channel 5
        w[x + "dq"][3, 1] = 6.0         # the probe's query latent: channel 3
        w[x + "uk"] *= 0.3
        w[x + "uq"] *= 0.3
        w[x + "uk"][7, 5] = 2.0         # head 0, key channel 7 <- latent channel 5
        w[x + "uq"][7, 3] = 2.0         # head 0, plain query channel 7 <- query latent channel 3
        w[x + "sink"][:] = [3.0, 1.0]
        w["l0.hc1.in"][:] = [0.6, 0.5]
        CUSTOM[name] = _bf16_values(w)
    return name


def needle_tokens(window: int, n: int, seed: int = 3):
    """Tokens 2.. at random with needles (0) and probes (1) placed so that probes sit exactly
    ``window - 1`` (the last key inside) and ``window`` (the first outside) behind a needle."""
    rng = np.random.default_rng(seed)
    toks = [int(t) for t in rng.integers(2, 64, n)]
    probes = {"just_inside": [], "just_outside": []}
    at = 1
    while at + 2 * window + 2 < n:
        toks[at] = 0
        toks[at + window - 1] = 1
        probes["just_inside"].append(at + window - 1)
        at += window + 3
        toks[at] = 0
        toks[at + window] = 1
        probes["just_outside"].append(at + window)
        at += window + 5
    return toks, probes


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,page", [(12, 16), (40, 16), (64, 64), (24, 32), (33, 8)])
def test_a_key_that_stands_out_at_the_edges_of_windows(dtype, window, page):
    """Needles just inside and just outside the window of a probe, in a whole prompt, in
    portions whose cuts fall between needle and probe, and with the probes decoded one by one,
    over pages smaller than, equal to and larger than the window."""
    name = needle_model(window)
    n = 6 * window + 40
    toks, probes = needle_tokens(window, n)
    assert len(probes["just_inside"]) >= 2 and len(probes["just_outside"]) >= 2
    ref = plain_logits(name, toks)
    runner = runner_for(name, dtype, page_size=page, cache_tokens=1024)
    got = run_steps(runner, [[("a", toks, range(n))]])
    check_request(got["a"], name, toks, dtype, "needles, whole prompt")
    cuts, at = [], 0
    for c in [window - 1, 2, window + 1, 3, 2 * window - 1]:
        cuts.append((at, at + c))
        at += c
    steps = [[("b", toks[a:b], range(b - a))] for a, b in cuts] + [[("b", [t], [0])] for t in toks[at:]]
    got = run_steps(runner, steps)
    check_request(got["b"], name, toks, dtype, "needles, portions and single tokens")
    # the test has teeth: with the window one longer the probes just outside see their needle
    off = json.loads(json.dumps(CONFIGS[name]))
    off["layers"][0]["mixer"]["mask"]["size"] = window + 1
    moved = RP.forward(off, weights(name), toks)
    assert np.abs(moved - ref).max(axis=1)[probes["just_outside"]].min() > 0.15 * np.abs(ref).max()


# --------------------------------------------------------------------------------------------
# the engine's own entry point, the command line, the trace runner
# --------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_engine(dtype):
    """The engine's own entry point and scheduler: prompts of unequal lengths, more requests than
    slots, greedy tokens.  The plain implementation, reading the engine's sequence, must choose
    the same token wherever its two best logits are clearly apart."""
    from llmario_b200.engine.engine import Engine
    from llmario_b200.sampling import SamplingParams

    for name in ("mix", "loop_all"):
        eng = Engine(model_dir(name), dtype=dtype, page_size=16, cache_tokens=1024, max_requests=2,
                     token_budget=48, context=256)
        prompts = [tokens_for(name, n, 20 + i) for i, n in enumerate((5, 70, 33, 1, 18))]
        outs = eng.generate(prompts, SamplingParams.greedy_params(max_tokens=24, ignore_eos=True))
        margin = 1e-3 if dtype == "float32" else 8e-2
        clear = 0
        for p, o in zip(prompts, outs):
            assert len(o) == 24
            ref = plain_logits(name, list(p) + list(o))
            # (the engine chose these tokens: behind a router's close call in the sequence the
            # two computations may have gone different ways)
            close = np.nonzero(router_margins(name, list(p) + list(o)) < CLOSE_CALL)[0]
            until = int(close[0]) if len(close) and dtype == "bfloat16" else len(ref)
            for j, tok in enumerate(o):
                if len(p) - 1 + j >= until:
                    break
                l = ref[len(p) - 1 + j]
                top = np.sort(l)[-2:]
                if top[1] - top[0] > margin * np.abs(l).max():
                    clear += 1
                    assert tok == int(np.argmax(l)), f"{name}: token {j} of a request"
        assert clear > (60 if dtype == "float32" else 5)
        assert eng.stats()["graph_replays"] > 0
        eng.runner.cache.check_invariants()


@pytest.mark.gpu
def test_command_line_and_trace_runner(tmp_path):
    """The two programs a user starts: ``llmario-b200 run`` on a Runidra model folder (greedy ids
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
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "llmario-b200"), "run", "runidra-tiny",
                        "--prompt-len", "5", "--n", "6", "--dtype", "bfloat16", "--page-size", "16",
                        "--context", "64"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len(p.stdout.strip().splitlines()[-1].split(",")) == 6
    # the trace runner: three requests, portions beside single tokens, a slot given back and taken
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
