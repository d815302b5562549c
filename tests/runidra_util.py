"""Small Runidra configurations with seeded weights for the tests, the plain implementation's
logits for them, and the error bounds.  Every configuration here is the tests' own: sizes are
chosen to differ from one another (heads, ranks, key and value sizes that are not multiples of
the kernels' tiles, windows that straddle pages, one to four streams, layers with and without a
feed-forward, loops)."""
from __future__ import annotations

import functools
import json
import os
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from plain import runidra_plain as RP


def mlstm(heads=2, dim=24, vdim=40, cap=15.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": mlp}


def latent(heads=3, dim=16, rot_dim=16, vdim=24, q_rank=40, kv_rank=48, window=20, base=10000.0,
           scale=None, dims=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
         "kv_rank": kv_rank, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if rot_dim:
        m["rot"] = {"dims": dims or rot_dim, "base": base}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=40, shared=56):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(layers, width=64, vocab=96, eps=1e-5, streams=2, loop=None, scale=1.5, cap=12.0):
    c = {"architecture": "Runidra", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": layers, "logit_scale": scale, "logit_softcap": cap}
    if streams is not None:
        c["streams"] = streams
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


CONFIGS: Dict[str, dict] = {
    # one mechanism each
    "memory": config([mlstm(mlp=dense(96))]),
    "memory_wide": config([mlstm(heads=1, dim=72, vdim=16, cap=6.0)], width=48, streams=1),
    "memory_big_key": config([mlstm(heads=3, dim=136, vdim=20)], streams=3),
    "latent": config([latent(mlp=dense(80))]),
    "latent_tc": config([latent(heads=4, dim=48, rot_dim=16, vdim=32, q_rank=64, kv_rank=112,
                                window=40)], width=128),
    # sixteen heads on the one key row of 64 channels: in 16 bits the sixteen-row decode kernel
    "latent_h16": config([latent(heads=16, dim=16, rot_dim=32, vdim=8, q_rank=32, kv_rank=32,
                                 window=24, mlp=dense(64))], streams=2),
    "latent_whole": config([latent(heads=2, dim=24, rot_dim=8, vdim=16, window=None, scale=0.2,
                                   dims=4)], streams=None),
    "latent_odd": config([latent(heads=5, dim=6, rot_dim=10, vdim=7, q_rank=9, kv_rank=13,
                                 window=7)], width=60, vocab=77, streams=4),
    "latent_one": config([latent(heads=1, dim=40, rot_dim=24, vdim=40, q_rank=32, kv_rank=64,
                                 window=1)], streams=1),
    "experts": config([latent(mlp=moe())]),
    "experts_top1": config([mlstm(mlp=moe(experts=3, top=1, ff=24, shared=None))], streams=None),
    # expert widths in steps of 16: in 16-bit the grouped tensor-core products
    "experts_tc": config([latent(mlp=moe(experts=5, top=2, ff=48, shared=64)),
                          mlstm(mlp=moe(experts=3, top=1, ff=32, shared=None))], streams=2),
    "experts_all": config([mlstm(heads=1, dim=16, vdim=16, mlp=moe(experts=4, top=4, ff=16, shared=8))]),
    # sizes that are multiples of nothing: every kernel's plain path
    "odd": config([mlstm(heads=3, dim=6, vdim=10, cap=3.0, mlp=moe(experts=5, top=3, ff=11, shared=13)),
                   latent(heads=2, dim=10, rot_dim=6, vdim=9, q_rank=7, kv_rank=11, window=5,
                          mlp=dense(34))], width=50, vocab=33, streams=3),
    # all of them, in an order of their own, with a loop
    "mix": config([latent(window=48, mlp=moe()), mlstm(mlp=dense(96)), mlstm(heads=4, dim=16, vdim=16),
                   latent(heads=2, dim=32, rot_dim=32, vdim=48, kv_rank=32, window=16, base=500.0,
                          mlp=dense(64))], width=64, vocab=128, loop=(1, 3, 2)),
    "loop_all": config([mlstm(mlp=moe(experts=4, top=2, ff=32)), latent(window=33)], loop=(0, 2, 3)),
}


def random_config(seed: int) -> str:
    """A configuration drawn from a seed: two to five layers of any kind in any order, with or
    without a loop.  Registered under the returned name."""
    name = f"random{seed}"
    if name in CONFIGS:
        return name
    rng = np.random.default_rng(7000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        mlp = pick(None, dense(pick(128, 160, 320)),
                   moe(experts=pick(4, 8, 12), top=pick(1, 2, 3), ff=pick(32, 64, 80),
                       shared=pick(None, 64, 96)))
        if rng.random() < 0.4:
            layers.append(mlstm(heads=pick(1, 2, 4, 6), dim=pick(16, 32, 40, 64),
                                vdim=pick(16, 24, 64), cap=pick(8.0, 15.0, 30.0), mlp=mlp))
        else:
            rot = pick(8, 16, 32, 64)
            layers.append(latent(heads=pick(2, 3, 4, 8), dim=pick(16, 32, 64), rot_dim=rot,
                                 vdim=pick(16, 32, 48), q_rank=pick(24, 48, 80),
                                 kv_rank=pick(32, 64, 96, 128), window=pick(24, 48, 64, 100),
                                 base=pick(1e4, 5e4, 1e6), mlp=mlp))
    n = len(layers)
    loop = None
    if rng.random() < 0.6:
        a = int(rng.integers(0, n))
        loop = (a, int(rng.integers(a + 1, n + 1)), int(rng.integers(2, 4)))
    CONFIGS[name] = config(layers, width=pick(96, 128, 160, 224), vocab=int(rng.integers(200, 700)),
                           streams=pick(None, 1, 2, 3, 4), loop=loop, scale=pick(1.0, 2.0, 0.5),
                           cap=pick(0.0, 10.0, 30.0))
    return name


def _weights(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    """Seeded weights, already rounded to bfloat16 values so that both precisions and the
    plain implementation compute with the same numbers."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    S = cfg.get("streams")
    t: Dict[str, np.ndarray] = {}

    def mat(name, out, inn, gain=1.0):
        t[name] = rng.standard_normal((out, inn)) * gain / np.sqrt(inn)

    def vec(name, n, mean=0.0, std=1.0):
        t[name] = mean + std * rng.standard_normal(n)

    def gated(p, ff, biases):
        mat(p + "gate", ff, W), mat(p + "up", ff, W), mat(p + "down", W, ff)
        if biases:
            vec(p + "gate.b", ff, 0.0, 0.3), vec(p + "up.b", ff, 0.0, 0.3), vec(p + "down.b", W, 0.0, 0.3)

    t["embed"] = rng.standard_normal((cfg["vocab"], W))
    for i, layer in enumerate(cfg["layers"]):
        p, x, m = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        vec(p + "norm1", W, 1.0, 0.1)
        subs = ["1"] + (["2"] if layer["mlp"] is not None else [])
        if S is not None:
            for q in subs:
                vec(f"{p}hc{q}.in", S, 1.0 / S, 0.2)
                vec(f"{p}hc{q}.out", S, 0.8, 0.3)
                t[f"{p}hc{q}.mix"] = np.eye(S) * 0.9 + 0.15 * rng.standard_normal((S, S))
        if layer["type"] == "mlstm":
            H, K, V = m["heads"], m["dim"], m["vdim"]
            mat(x + "q", H * K, W, 2.0), mat(x + "k", H * K, W), mat(x + "v", H * V, W)
            mat(x + "g", H * V, W), mat(x + "o", W, H * V)
            mat(x + "i", H, W, 2.0), mat(x + "f", H, W, 2.0)
            vec(x + "i.b", H, 0.0, 1.0), vec(x + "f.b", H, 2.0, 1.0)
            vec(x + "norm", H * V, 1.0, 0.1)
        else:
            H, D, R, V = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"]
            Rq, Rkv = m["q_rank"], m["kv_rank"]
            mat(x + "dq", Rq, W), vec(x + "dq.norm", Rq, 1.0, 0.2)
            mat(x + "uq", H * (D + R), Rq, 2.0)
            mat(x + "dkv", Rkv + R, W, 2.0), vec(x + "dkv.norm", Rkv, 1.0, 0.2)
            mat(x + "uk", H * D, Rkv, 2.0), mat(x + "uv", H * V, Rkv)
            vec(x + "sink", H, 0.5, 1.0), mat(x + "o", W, H * V)
        mlp = layer["mlp"]
        if mlp is not None:
            vec(p + "norm2", W, 1.0, 0.1)
            f = p + "mlp."
            if mlp["kind"] == "dense":
                gated(f, mlp["ff"], True)
            else:
                E = mlp["router"]["experts"]
                for e in range(E):
                    gated(f"{f}e{e}.", mlp["expert"]["ff"], False)
                # logits far enough apart that rounding does not change who is chosen
                mat(f + "router", E, W, 4.0), vec(f + "router.b", E, 0.0, 1.0)
                if mlp.get("shared"):
                    gated(f + "shared.", mlp["shared"]["ff"], False)
                    mat(f + "shared.sg", 1, W, 2.0)
    vec("final.norm", W, 1.0, 0.1)
    mat("head", cfg["vocab"], W)
    return _bf16_values(t)


def _bf16_values(t: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    return {n: torch.from_numpy(np.asarray(a, dtype=np.float64)).to(torch.bfloat16)
            .to(torch.float64).numpy() for n, a in t.items()}


CUSTOM: Dict[str, Dict[str, np.ndarray]] = {}     # configurations whose weights a test has made


@functools.lru_cache(maxsize=None)
def weights(name: str, seed: int = 0) -> Dict[str, np.ndarray]:
    return CUSTOM[name] if name in CUSTOM else _weights(CONFIGS[name], seed)


_dirs: Dict[tuple, str] = {}


def model_dir(name: str, seed: int = 0) -> str:
    """A folder with config.json and model.safetensors (bfloat16) of the configuration."""
    from llmario_b200.weights.safetensors_io import write_safetensors

    key = (name, seed)
    if key not in _dirs:
        d = tempfile.mkdtemp(prefix=f"runidra_{name}_")
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CONFIGS[name], f)
        write_safetensors(os.path.join(d, "model.safetensors"),
                          {n: torch.from_numpy(a).to(torch.bfloat16)
                           for n, a in weights(name, seed).items()})
        _dirs[key] = d
    return _dirs[key]


@functools.lru_cache(maxsize=None)
def _plain(name: str, seed: int, tokens: tuple):
    margins: List[np.ndarray] = []
    logits = RP.forward(CONFIGS[name], weights(name, seed), list(tokens), margins=margins)
    closest = np.min(np.stack(margins), axis=0) if margins else np.full(len(tokens), np.inf)
    return logits, closest


def plain_logits(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    return _plain(name, seed, tuple(int(t) for t in tokens))[0]


# A router's choice between two experts whose logits lie closer than this can fall either way
# once the router's input is rounded to 16 bits (logits of a size of about 4 then move by a
# hundredth or two); the 16-bit tests do not compare the positions of such calls.
CLOSE_CALL = 0.08


def router_margins(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    """Per position, the smallest gap over all routed layer runs between the last chosen
    expert's logit and the best one not chosen (infinite for a model without routed layers)."""
    return _plain(name, seed, tuple(int(t) for t in tokens))[1]


@functools.lru_cache(maxsize=None)
def _sensitivity(name: str, seed: int, tokens: tuple) -> np.ndarray:
    """Per position, how far the logits move when the inputs move by about one bfloat16
    rounding or two: the plain implementation run again with the embedding rows scaled by
    1 + 2^-7 N(0, 1) (the largest of four such moves)."""
    w = dict(weights(name, seed))
    rng = np.random.default_rng(99)
    embed, ref = w["embed"], _plain(name, seed, tokens)[0]
    worst = np.zeros(len(tokens))
    for _ in range(4):
        w["embed"] = embed * (1 + 2.0 ** -7 * rng.standard_normal(embed.shape))
        moved = RP.forward(CONFIGS[name], w, list(tokens))
        worst = np.maximum(worst, np.abs(moved - ref).max(axis=1))
    return worst


def sensitivity(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    return _sensitivity(name, seed, tuple(int(t) for t in tokens))


def tokens_for(name: str, n: int, seed: int) -> List[int]:
    rng = np.random.default_rng(1000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[name]["vocab"], n)]


def slack_for(name: str, tokens: Sequence[int], dtype: str, seed: int = 0) -> Optional[np.ndarray]:
    """What a position is allowed on top of the bound.  float32: nothing.  bfloat16: three times
    what a move of the inputs by a rounding or two does to it in the plain implementation, and
    everything at a position where a router makes a close call (the other expert may run)."""
    if dtype != "bfloat16":
        return None
    slack = 3.0 * sensitivity(name, tokens, seed)
    slack[router_margins(name, tokens, seed) < CLOSE_CALL] = np.inf
    return slack


def runner_for(name: str, dtype: str, page_size: int = 16, cache_tokens: int = 1024,
               max_requests: int = 4, seed: int = 0, use_graphs: bool = True):
    from llmario_b200.engine.model import Model
    from llmario_b200.engine.step import ModelRunner

    model = Model.from_folder(model_dir(name, seed), dtype, "cuda:0")
    return ModelRunner(model, page_size=page_size, n_pages=-(-cache_tokens // page_size),
                       max_requests=max_requests, max_context=cache_tokens,
                       token_budget=cache_tokens, use_graphs=use_graphs)


# Largest error as a fraction of the largest logit.  float32: rounding of 32-bit sums only.
# bfloat16: 16-bit operands of the matrix products (the weights are exact in both).
# (float32: through several passes of a loop over streams that are mixed again and again, a few
# positions of a few sequences reach 3e-4; one request alone and in a batch give the same bits)
BOUND = {"float32": 5e-4, "bfloat16": 4e-2}


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str = "",
                 bound: Optional[float] = None, slack: Optional[np.ndarray] = None) -> None:
    """``slack``: per row, an allowance on top of the bound (16-bit runs: a multiple of the
    row's :func:`sensitivity`)."""
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    err = np.abs(got.astype(np.float64) - ref)
    tol = (bound if bound is not None else BOUND[dtype]) * max(1e-6, float(np.abs(ref).max()))
    if slack is not None:
        with np.errstate(invalid="ignore"):
            err = np.maximum(0.0, err - slack.reshape((-1,) + (1,) * (err.ndim - 1)))
        assert len(slack) < 20 or np.isfinite(slack).mean() > 0.7, f"{what}: too few positions are compared"
    worst = np.unravel_index(np.argmax(err), err.shape)
    assert err.max() <= tol, (f"{what} ({dtype}): max |diff| {err.max():.3e} > {tol:.3e} at "
                              f"{tuple(int(w) for w in worst)}")
