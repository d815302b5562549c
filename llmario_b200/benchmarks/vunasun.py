"""Vunasun beside Qwen3 at equal sizes: prompt and decode rates of whole models with random
weights, and the design's own kernels one by one against the memory roofline.

    python -m llmario_b200.benchmarks.vunasun [--sizes 0.6b,8b] [--layers 8] [--kernels]

A Vunasun model of a size has the width, feed-forward width, attention heads and number of
layers of the Qwen3 preset of that name; its layers repeat (gla, gla, mamba2, attention), every
one with a feed-forward, so that the two models stream about the same weights.  ``bench.py
--workload vunasun`` prints the same record as its JSON line.
"""
from __future__ import annotations

import argparse
import json
import random
import statistics
import sys
from typing import Any, Dict, List

SIZES = {"0.6b": "qwen3-0.6b", "8b": "qwen3-8b"}


def vunasun_config(preset: Dict[str, Any], layers: int, vocab: int = 32768):
    """The Vunasun configuration with the sizes of a Qwen3 preset."""
    from ..config.vunasun import sized_like

    return sized_like(preset["hidden_size"], preset["intermediate_size"],
                      preset["num_attention_heads"], preset["num_key_value_heads"],
                      preset["head_dim"], layers, vocab)


def _rates(model, page_size: int, batch: int, prompt_len: int, prefill_tokens: int, steps: int,
           warmup: int) -> Dict[str, Any]:
    """Prompt and decode rates of ``model`` through the step function, timed on the device."""
    import torch

    from .. import kernels
    from ..engine.step import ModelRunner, StepEntry

    rng = random.Random(0)
    vocab = model.vocab_size
    per_req = prompt_len + warmup + steps + 2 * page_size
    runner = ModelRunner(model, page_size=page_size,
                         n_pages=-(-max(batch * per_req, prefill_tokens + page_size) // page_size),
                         max_requests=batch, max_context=max(per_req, prefill_tokens + page_size),
                         token_budget=max(prefill_tokens, prompt_len))
    times = []
    for r in range(4):
        toks = [rng.randrange(vocab) for _ in range(prefill_tokens)]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.step([StepEntry(f"p{r}", toks, [prefill_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.close(f"p{r}")
        if r:
            times.append(a.elapsed_time(b))
    prefill_ms = statistics.median(times)
    ids = [f"d{i}" for i in range(batch)]
    for rid in ids:
        runner.step([StepEntry(rid, [rng.randrange(vocab) for _ in range(prompt_len)], [])])

    def one():
        runner.step([StepEntry(rid, [rng.randrange(vocab)], [0]) for rid in ids])

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    l0 = kernels.launches
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        one()
    b.record()
    torch.cuda.synchronize()
    decode_ms = a.elapsed_time(b) / steps
    launches = (kernels.launches - l0) / steps
    state = sum(t.numel() * t.element_size() for t in runner.cache.state.values()) \
        // max(1, runner.cache.max_requests)
    for rid in ids:
        runner.close(rid)
    return {"prefill_tok_s": round(prefill_tokens / (prefill_ms / 1e3)), "prefill_ms": round(prefill_ms, 3),
            "decode_tok_s": round(batch / (decode_ms / 1e3)), "decode_ms": round(decode_ms, 4),
            "launches_per_decode_step": round(launches, 1), "weight_bytes": model.weight_bytes(),
            "state_bytes_per_request": int(state),
            "graph_replays": runner.counters["graph_replays"]}


def compare(sizes: List[str], layers: int, batch: int = 8, prompt_len: int = 1024,
            prefill_tokens: int = 2048, steps: int = 64, warmup: int = 24,
            page_size: int = 64) -> Dict[str, Any]:
    import torch

    from ..cli import PRESETS, preset_config
    from ..engine.model import Model
    from .roofline import peaks

    pk = peaks()
    out: Dict[str, Any] = {}
    for size in sizes:
        preset = dict(PRESETS[SIZES[size]], vocab_size=32768)
        rec: Dict[str, Any] = {}
        for which in ("qwen3", "vunasun"):
            if which == "qwen3":
                from ..config import Qwen3Config

                cfg = Qwen3Config.from_dict(dict(preset, num_hidden_layers=layers,
                                                 tie_word_embeddings=False,
                                                 architectures=["Qwen3ForCausalLM"]))
            else:
                cfg = vunasun_config(preset, layers)
            model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            r = _rates(model, page_size, batch, prompt_len, prefill_tokens, steps, warmup)
            # a decode step streams the weights once and every live request's state twice
            moved = r["weight_bytes"] + 2 * batch * r["state_bytes_per_request"]
            r["decode_frac_of_copy_peak"] = round(moved / (r["decode_ms"] / 1e3) / (pk["hbm_gbs"] * 1e9), 3)
            rec[which] = r
            del model
            torch.cuda.empty_cache()
        out[size] = rec
    return {"layers": layers, "batch": batch, "prompt_len": prompt_len,
            "prefill_tokens": prefill_tokens, "page_size": page_size, "peaks": pk["source"],
            "sizes": out}


# ---------------------------------------------------------------------------------------------
def _time(fn, reps: int = 20, flush=None) -> float:
    """Median microseconds of ``fn`` timed with CUDA events, the L2 flushed before every run."""
    import torch

    for _ in range(3):
        fn()
    ts = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    return statistics.median(ts)


def kernel_table(width: int = 4096, tokens: int = 2048, batch: int = 64) -> List[Dict[str, Any]]:
    """The design's own kernels, each alone at the sizes of ``vunasun_config`` for ``width``,
    with the bytes they must move and the fraction of the measured copy rate; beside them the
    like kernels of the Qwen3 path (the norm, decode attention over as many bytes)."""
    import torch

    from .. import kernels
    from .roofline import peaks

    dev = "cuda:0"
    pk = peaks()
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    rows_out: List[Dict[str, Any]] = []

    def rec(name, us, nbytes, note=""):
        rows_out.append({"kernel": name, "us": round(us, 2), "bytes": int(nbytes),
                         "gb_s": round(nbytes / us / 1e3, 1),
                         "frac_of_copy_peak": round(nbytes / (us * 1e-6) / (pk["hbm_gbs"] * 1e9), 3),
                         "note": note})

    f32 = lambda *s: torch.randn(*s, dtype=torch.float32, device=dev)
    slots = batch
    for label, rows, single in ((f"prompt of {tokens}", tokens, False), (f"decode, batch {batch}", batch, True)):
        row_slot = (torch.arange(rows, dtype=torch.int32, device=dev) if single
                    else torch.zeros(rows, dtype=torch.int32, device=dev))
        seg = None
        if not single:
            seg = torch.empty(slots, 3, dtype=torch.int32, device=dev)
            kernels.segment_table(row_slot, seg)
        # gated linear attention: heads of 128 key and 256 value channels
        H, K, V = max(1, width // 256), 128, 256
        proj = f32(rows, 2 * H * K + 2 * H * V + 64) * 0.1
        z = torch.sigmoid(f32(rows, H * K) + 2)
        zb = f32(H * K)
        us = _time(lambda: kernels.bias_sigmoid_pow(z, zb, 1 / 16), flush=flush)
        rec(f"bias_sigmoid_pow ({label})", us, rows * H * K * 8)
        z = torch.sigmoid(f32(rows, H * K) + 2)
        state = torch.zeros(slots, H * V * K, dtype=torch.float32, device=dev)
        o = torch.empty(rows, H * V, dtype=torch.float32, device=dev)
        us = _time(lambda: kernels.linear_recurrence(
            proj[:, :H * K], proj[:, H * K:2 * H * K], proj[:, 2 * H * K:2 * H * K + H * V], z, state, o,
            row_slot, seg, H, H, K, V, kernels.DECAY_VECTOR, q_scale=K ** -0.5, n_requests=1), flush=flush)
        live = rows if single else 1
        moved = rows * (3 * H * K + 2 * H * V) * 4 + 2 * live * H * V * K * 4
        rec(f"linear_recurrence gla ({label})", us, moved,
            "a prompt is one request: its tokens are walked in order" if not single else "")
        gated = torch.empty(rows, H * V, dtype=torch.bfloat16, device=dev)
        w = f32(V)
        us = _time(lambda: kernels.gated_group_norm(o, proj[:, 2 * H * K + H * V:2 * H * K + 2 * H * V], w, gated,
                                                    V, 1e-6, False), flush=flush)
        rec(f"gated_group_norm gla ({label})", us, rows * H * V * (4 + 4 + 2))
        # state-space mixer: heads of 64 channels, 128 state rows, one group
        H2, P, N, G = 2 * width // 64, 64, 128, 1
        inner, C = H2 * P, H2 * P + 2 * N
        proj2 = f32(rows, 2 * inner + 2 * N + H2) * 0.1
        st2 = torch.zeros(slots, H2 * P * N + C * 3, dtype=torch.float32, device=dev)
        xbc = torch.empty(rows, C, dtype=torch.float32, device=dev)
        cw, cb = f32(C, 4) * 0.3, f32(C) * 0.1
        us = _time(lambda: kernels.causal_conv_silu(proj2[:, inner:inner + C], cw, cb, st2[:, H2 * P * N:], xbc,
                                                    row_slot, seg), flush=flush)
        rec(f"causal_conv_silu + history ({label})", us, rows * C * 8 + 2 * live * C * 3 * 4, "two launches")
        o2 = torch.empty(rows, inner, dtype=torch.float32, device=dev)
        a_log, dtb = f32(H2) * 0.1, f32(H2) * 0.1
        us = _time(lambda: kernels.linear_recurrence(
            xbc[:, inner + N:], xbc[:, inner:inner + N], xbc[:, :inner], proj2[:, 2 * inner + 2 * N:], st2, o2,
            row_slot, seg, H2, G, N, P, kernels.DECAY_RATE_STEP, rate_log=a_log, step_bias=dtb, n_requests=1),
            flush=flush)
        moved = rows * (2 * N + 2 * inner + H2) * 4 + 2 * live * H2 * P * N * 4
        rec(f"linear_recurrence mamba2 ({label})", us, moved)
        g2 = torch.empty(rows, inner, dtype=torch.bfloat16, device=dev)
        w2, skip = f32(inner), f32(H2)
        us = _time(lambda: kernels.gated_group_norm(o2, proj2[:, :inner], w2, g2, inner, 1e-6, True, skip=skip,
                                                    skip_input=xbc[:, :inner], head=P), flush=flush)
        rec(f"gated_group_norm mamba2 ({label})", us, rows * inner * (4 + 4 + 4 + 2))
        # the block's own kernels, and the norm of the Qwen3 path beside them
        x, y, wn, ls = f32(rows, width), f32(rows, width), f32(width), f32(width)
        h16 = torch.empty(rows, width, dtype=torch.bfloat16, device=dev)
        us = _time(lambda: kernels.norm_scale_add(y, wn, ls, x, 1e-6, rounded=h16), flush=flush)
        rec(f"norm_scale_add ({label})", us, rows * width * 14)
        us = _time(lambda: kernels.cast_rows(x, h16), flush=flush)
        rec(f"cast_rows ({label})", us, rows * width * 6)
        us = _time(lambda: kernels.rms_norm(x, wn, h16, 1e-6), flush=flush)
        rec(f"rms_norm, the Qwen3 path's ({label})", us, rows * width * 6)
    return rows_out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--sizes", default="0.6b,8b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--kernels", action="store_true", help="time the design's kernels one by one")
    ap.add_argument("--only-kernels", action="store_true", help="leave the whole models out")
    ap.add_argument("--width", type=int, default=4096, help="--kernels: the models' width")
    ap.add_argument("--tokens", type=int, default=2048, help="--kernels: tokens of the prompt")
    a = ap.parse_args(argv)
    out = {} if a.only_kernels else compare([s for s in a.sizes.split(",") if s], a.layers,
                                            batch=a.batch, steps=a.steps)
    if a.kernels or a.only_kernels:
        out["kernels"] = kernel_table(a.width, a.tokens)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
