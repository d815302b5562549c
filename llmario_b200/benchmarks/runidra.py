"""Runidra beside Qwen3 at equal sizes: prompt and decode rates of whole models with random
weights, and the design's own kernels one by one against the memory roofline.

    python -m llmario_b200.benchmarks.runidra [--sizes 0.6b,8b] [--layers 8] [--kernels]

A Runidra model of a size has the width, feed-forward width, attention heads and number of
layers of the Qwen3 preset of that name; its layers repeat (latent attention + dense, matrix
memory + routed experts, latent attention + dense, latent attention + routed experts) on two
residual streams (``config.runidra.sized_like``).  A token uses two of eight experts of half the
feed-forward width beside a shared one, so a prompt does 1.5 times the feed-forward work of the
dense layer and a decode step of few rows streams up to all experts.  ``bench.py --workload
runidra`` prints the same record as its JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Dict, List

from .vunasun import SIZES, _rates, _time


def runidra_config(preset: Dict[str, Any], layers: int, vocab: int = 32768, window: int = 1024):
    """The Runidra configuration with the sizes of a Qwen3 preset."""
    from ..config.runidra import sized_like

    return sized_like(preset["hidden_size"], preset["intermediate_size"],
                      preset["num_attention_heads"], preset["head_dim"], layers, vocab,
                      window=window)


def compare(sizes: List[str], layers: int, batch: int = 8, prompt_len: int = 1024,
            prefill_tokens: int = 2048, steps: int = 64, warmup: int = 24,
            page_size: int = 64) -> Dict[str, Any]:
    import torch

    from ..cli import PRESETS
    from ..engine.model import Model
    from .roofline import peaks

    pk = peaks()
    out: Dict[str, Any] = {}
    for size in sizes:
        preset = dict(PRESETS[SIZES[size]], vocab_size=32768)
        rec: Dict[str, Any] = {}
        for which in ("qwen3", "runidra"):
            if which == "qwen3":
                from ..config import Qwen3Config

                cfg = Qwen3Config.from_dict(dict(preset, num_hidden_layers=layers,
                                                 tie_word_embeddings=False,
                                                 architectures=["Qwen3ForCausalLM"]))
            else:
                cfg = runidra_config(preset, layers)
            model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            r = _rates(model, page_size, batch, prompt_len, prefill_tokens, steps, warmup)
            # a decode step streams the weights once (all experts counted) and every live
            # request's recurrent state twice
            moved = r["weight_bytes"] + 2 * batch * r["state_bytes_per_request"]
            r["decode_frac_of_copy_peak"] = round(moved / (r["decode_ms"] / 1e3) / (pk["hbm_gbs"] * 1e9), 3)
            rec[which] = r
            del model
            torch.cuda.empty_cache()
        out[size] = rec
    return {"layers": layers, "batch": batch, "prompt_len": prompt_len,
            "prefill_tokens": prefill_tokens, "page_size": page_size, "peaks": pk["source"],
            "sizes": out}


def kernel_table(width: int = 4096, tokens: int = 2048, batch: int = 64, heads: int = 32,
                 ff: int = 12288, window: int = 1024) -> List[Dict[str, Any]]:
    """The design's own kernels, each alone at the sizes of ``runidra_config`` for ``width``,
    with the bytes they must move (or the operations they must do) and the fraction of the
    measured copy rate (or tensor rate); beside them the like kernels of the Qwen3 path."""
    import torch

    from .. import kernels
    from .roofline import peaks

    dev = "cuda:0"
    pk = peaks()
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    rows_out: List[Dict[str, Any]] = []

    def rec(name, us, nbytes, flops=0, note=""):
        r = {"kernel": name, "us": round(us, 2), "bytes": int(nbytes),
             "gb_s": round(nbytes / us / 1e3, 1),
             "frac_of_copy_peak": round(nbytes / (us * 1e-6) / (pk["hbm_gbs"] * 1e9), 3), "note": note}
        if flops:
            r["tflops"] = round(flops / us / 1e6, 1)
            r["frac_of_tensor_peak"] = round(flops / (us * 1e-6) / (pk["bf16_tflops"] * 1e12), 3)
        rows_out.append(r)

    f32 = lambda *s: torch.randn(*s, dtype=torch.float32, device=dev)
    b16 = lambda *s: torch.randn(*s, dtype=torch.bfloat16, device=dev)
    slots = batch
    S = 2
    for label, rows, single in ((f"prompt of {tokens}", tokens, False), (f"decode, batch {batch}", batch, True)):
        row_slot = (torch.arange(rows, dtype=torch.int32, device=dev) if single
                    else torch.zeros(rows, dtype=torch.int32, device=dev))
        seg = None
        if not single:
            seg = torch.empty(slots, 3, dtype=torch.int32, device=dev)
            kernels.segment_table(row_slot, seg)
        live = rows if single else 1
        # ---- the residual streams: a sublayer's write with the next one's read and norm
        xs, y, wn = f32(S, rows, width), f32(rows, width), f32(width)
        mix, cout, cin = f32(S, S), f32(S), f32(S)
        h16 = torch.empty(rows, width, dtype=torch.bfloat16, device=dev)
        us = _time(lambda: kernels.stream_step(xs, y=y, mix=mix * 0.1, out_coef=cout * 0.1, in_coef=cin,
                                               weight=wn, eps=1e-6, out=h16), flush=flush)
        rec(f"stream_step: write + read + norm, {S} streams ({label})", us, rows * width * (8 * S + 4 + 2))
        x1 = f32(rows, width)
        us = _time(lambda: kernels.rms_norm(x1, wn, h16, 1e-6), flush=flush)
        rec(f"rms_norm, the Qwen3 path's ({label})", us, rows * width * 6)
        # ---- matrix memory: heads of 128 x 128
        H, K, V = max(1, width // 256), 128, 128
        proj = f32(rows, 2 * H * K + 2 * H * V + 2 * H) * 0.1
        ci = 2 * H * K + 2 * H * V
        state = torch.zeros(slots, H * (V + 1) * K + H, dtype=torch.float32, device=dev)
        gates = torch.empty(rows, 3 * H, dtype=torch.float32, device=dev)
        bi, bf = f32(H), f32(H) + 2
        us = _time(lambda: kernels.log_gate_scan(proj[:, ci:ci + H], proj[:, ci + H:ci + 2 * H], bi, bf, 15.0,
                                                 state[:, H * (V + 1) * K:], gates, row_slot, seg, H,
                                                 n_requests=1), flush=flush)
        rec(f"log_gate_scan ({label})", us, rows * H * 20,
            note="a chain of maxima per request and head: latency, not bytes")
        o = torch.empty(rows, H * (V + 1), dtype=torch.float32, device=dev)
        us = _time(lambda: kernels.linear_recurrence(
            proj[:, :H * K], proj[:, H * K:2 * H * K], proj[:, 2 * H * K:2 * H * K + H * V], gates[:, :H],
            state, o, row_slot, seg, H, H, K, V + 1, kernels.DECAY_SCALAR_INPUT, q_scale=K ** -0.5,
            n_requests=1, input_weight=gates[:, H:2 * H], ones=True), flush=flush)
        moved = rows * (2 * H * K + 2 * H * V) * 4 + 2 * live * H * (V + 1) * K * 4
        rec(f"linear_recurrence, matrix memory ({label})", us, moved,
            note="a prompt is one request: its tokens are walked in order" if not single else "")
        gated = torch.empty(rows, H * V, dtype=torch.bfloat16, device=dev)
        wv = f32(H * V)
        us = _time(lambda: kernels.memory_out_norm(o, gates[:, 2 * H:], proj[:, 2 * H * K + H * V:ci], wv, gated,
                                                   H, V, 1e-6, 1e-6), flush=flush)
        rec(f"memory_out_norm ({label})", us, rows * H * V * (4 + 4 + 2))
        # ---- attention through latents: key rows of 64 + 64 channels, one key head
        C, R, D, Vd, Rq = 64, 64, 64, 128, max(64, width // 4)
        hd = C + R
        page, n_pages = 64, -(-(window + tokens) // 64) + 1
        ctx_len = window if single else 0
        store = b16(n_pages * max(1, live if single else 1), 1, 2, 1, page, hd) * 0.3
        table = torch.arange(store.shape[0], dtype=torch.int32, device=dev).view(max(1, live if single else 1), -1)
        row_pos = (torch.full((rows,), ctx_len, dtype=torch.int32, device=dev) if single
                   else torch.arange(rows, dtype=torch.int32, device=dev))
        slot_of = (torch.arange(rows, dtype=torch.int32, device=dev) if single else row_slot)
        down = f32(rows, Rq + C + R)
        cq = torch.empty(rows, Rq, dtype=torch.bfloat16, device=dev)
        angles = f32(rows, R // 2, 2)

        class View:
            k, v = store[0, 0, 0], store[0, 0, 1]
            page_stride, block_table, page_size = store.stride(0), table, page

        us = _time(lambda: kernels.latent_store(down, f32(Rq), f32(C), angles, cq, View, slot_of, row_pos, Rq, C,
                                                R, 1e-6), flush=flush)
        rec(f"latent_store: two norms, rotation, cache write ({label})", us,
            rows * ((Rq + C + R) * 4 + Rq * 2 + (2 * C + R) * 2))
        q32 = f32(rows, heads * (D + R))
        q_plain = torch.empty(rows, heads * D, dtype=torch.bfloat16, device=dev)
        q_full = torch.empty(rows, heads * hd, dtype=torch.bfloat16, device=dev)
        us = _time(lambda: kernels.latent_query(q32, angles, q_plain, q_full, heads, D, R, C), flush=flush)
        rec(f"latent_query: rounding and rotation ({label})", us, rows * heads * ((D + R) * 4 + (D + R) * 2))
        maps = b16(heads, C, D) * 0.1
        us = _time(lambda: kernels.head_linear(q_plain.view(rows, heads, D), maps,
                                               q_full.view(rows, heads, hd)[:, :, :C]), flush=flush)
        rec(f"head_linear: the heads' key maps on the queries ({label})", us,
            rows * heads * (D + C) * 2 + heads * C * D * 2, flops=2.0 * rows * heads * C * D,
            note="one launch per head on the tensor-core product")
        sink = f32(heads)
        mixed = torch.empty(rows, heads * C, dtype=torch.bfloat16, device=dev)
        keys = (min(window, ctx_len + 1) * rows if single
                else sum(min(window, p + 1) for p in range(rows)))
        us = _time(lambda: kernels.attention_generic(q_full, mixed, View.k, View.v, View.page_stride, table,
                                                     slot_of, row_pos, heads, 1, hd, page, hd ** -0.5, window,
                                                     sink=sink, value_dim=C), reps=5, flush=flush)
        rec(f"attention over latents, generic kernel ({label})", us,
            (live * min(window, (ctx_len if single else rows)) * (hd + C) * 2 + rows * heads * (hd + C) * 2),
            flops=2.0 * keys * heads * (hd + C),
            note="one warp per (row, head); every head reads the shared key rows again")
        # ---- routed experts, row-wise form
        E, top, eff = 8, 2, ff // 2
        z = f32(rows, E + 1)
        ids = torch.empty(rows, top, dtype=torch.int32, device=dev)
        wts = torch.empty(rows, top, dtype=torch.float32, device=dev)
        us = _time(lambda: kernels.moe_route(z, E, top, ids, wts), flush=flush)
        rec(f"moe_route ({label})", us, rows * ((E + 1) * 4 + top * 8))
        if single:
            hrow = b16(rows, width)
            gu, dn = b16(E, 2 * eff, width) * 0.02, b16(E, width, eff) * 0.02
            act = torch.empty(rows, top, eff, dtype=torch.bfloat16, device=dev)
            used = len(set(ids.flatten().tolist()))
            us = _time(lambda: kernels.moe_gate_up_rows(hrow, gu, ids, act), reps=5, flush=flush)
            rec(f"moe_gate_up_rows ({label})", us, used * 2 * eff * width * 2,
                note=f"{used} of {E} experts in use: each is read from memory once, again from L2 per row")
            yo = torch.zeros(rows, width, dtype=torch.float32, device=dev)
            us = _time(lambda: kernels.moe_down_rows(act, dn, ids, wts, yo, False), reps=5, flush=flush)
            rec(f"moe_down_rows ({label})", us, used * eff * width * 2)
            del gu, dn
        gu32 = f32(rows, 2 * ff)
        act16 = torch.empty(rows, ff, dtype=torch.bfloat16, device=dev)
        us = _time(lambda: kernels.gated_act(gu32, f32(2 * ff), act16, "gelu_tanh"), flush=flush)
        rec(f"gated_act: biases, gelu, product ({label})", us, rows * ff * (8 + 2))
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
