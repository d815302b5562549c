"""Small Vunasun configurations with seeded weights for the tests, the plain implementation's
logits for them, and the error bounds.  Every configuration here is the tests' own: sizes are
chosen to differ from one another (heads, groups, key and value sizes that are not multiples of
the kernels' tiles, chunk sizes that straddle pages, layers with and without a feed-forward)."""
from __future__ import annotations

import functools
import json
import os
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from plain import vunasun_plain as VP


def gla(heads=2, dim=24, vdim=40, tau=4.0, rank=8, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau,
                                     "rank": rank}, "mlp": mlp}


def mamba2(heads=4, vdim=24, state=16, groups=2, conv=4, norm_groups=1, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state,
                                        "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp}


def attention(heads=4, kv_heads=2, dim=32, chunk=24, rot=16, base=10000.0, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
         "scale": scale if scale is not None else dim ** -0.5}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(layers, width=64, vocab=96, eps=1e-5):
    return {"architecture": "Vunasun", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


CONFIGS: Dict[str, dict] = {
    # one mechanism each
    "gla": config([gla(mlp=dense(96))]),
    "gla_wide": config([gla(heads=1, dim=72, vdim=16, tau=1.0, rank=16)], width=48),
    "gla_big_key": config([gla(heads=2, dim=136, vdim=24, tau=32.0)], width=64),
    "ssm": config([mamba2()]),
    "ssm_groups": config([mamba2(heads=6, vdim=16, state=40, groups=6, conv=2, norm_groups=3,
                                 mlp=dense(80))], width=72),
    "ssm_one_tap": config([mamba2(heads=2, vdim=40, state=8, groups=1, conv=1, norm_groups=2)]),
    "attn": config([attention(mlp=dense(128))]),
    "attn_tc": config([attention(heads=4, kv_heads=1, dim=64, chunk=40, rot=64)], width=128),
    "attn_whole": config([attention(heads=2, kv_heads=2, dim=40, chunk=None, rot=None,
                                    scale=0.2)]),
    "attn_odd": config([attention(heads=3, kv_heads=1, dim=20, chunk=7, rot=10)], width=60,
                       vocab=77),
    # three query heads to a key head (no tensor-core tile takes it), and eight with whole heads
    # of 128 rotated and a chunk that is no multiple of a page
    "attn_g3": config([attention(heads=6, kv_heads=2, dim=64, chunk=36, rot=16)], width=96),
    "attn_g8": config([attention(heads=8, kv_heads=1, dim=128, chunk=100, rot=128,
                                 mlp=dense(64))], width=64),
    # sixteen query heads to a key head
    "attn_g16": config([attention(heads=16, kv_heads=1, dim=64, chunk=30, rot=32)], width=64),
    # sizes that are multiples of nothing: every kernel's plain path
    "odd": config([gla(heads=3, dim=6, vdim=10, tau=2.0, rank=5),
                   mamba2(heads=3, vdim=5, state=6, groups=3, conv=3, norm_groups=3, mlp=dense(34)),
                   attention(heads=2, kv_heads=2, dim=10, chunk=5, rot=4)], width=50, vocab=33),
    # all of them, in an order of their own
    "mix": config([attention(chunk=48, mlp=dense(96)), mamba2(norm_groups=2), gla(),
                   attention(heads=2, kv_heads=1, dim=64, chunk=16, rot=32, base=500.0),
                   gla(heads=4, dim=16, vdim=16, tau=8.0, mlp=dense(64))], width=64, vocab=128),
    "recurrent_only": config([gla(), mamba2(mlp=dense(64))]),
}


def random_config(seed: int) -> str:
    """A configuration drawn from a seed: three to six layers of any kind in any order, sizes of
    the kind a small model has.  Registered under the returned name."""
    name = f"random{seed}"
    if name in CONFIGS:
        return name
    rng = np.random.default_rng(4000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    layers = []
    for _ in range(int(rng.integers(3, 7))):
        mlp = dense(pick(128, 160, 320)) if rng.random() < 0.5 else None
        kind = pick("gla", "mamba2", "attention")
        if kind == "gla":
            layers.append(gla(heads=pick(1, 2, 4), dim=pick(16, 32, 40, 64), vdim=pick(16, 24, 64),
                              tau=pick(4.0, 8.0, 16.0, 32.0), rank=pick(8, 16, 32), mlp=mlp))
        elif kind == "mamba2":
            heads = pick(2, 4, 8)
            vdim = pick(16, 32, 64)
            layers.append(mamba2(heads=heads, vdim=vdim, state=pick(16, 32, 64),
                                 groups=pick(*[g for g in (1, 2, 4, 8) if heads % g == 0]),
                                 conv=pick(2, 3, 4), norm_groups=pick(1, 2, 4), mlp=mlp))
        else:
            heads = pick(2, 4, 8)
            dim = pick(32, 64, 128)
            layers.append(attention(heads=heads, kv_heads=pick(*[g for g in (1, 2, 4, 8) if heads % g == 0]),
                                    dim=dim, chunk=pick(32, 48, 64, 128), rot=pick(dim // 2, dim),
                                    base=pick(1e4, 2e5, 1e6), scale=pick(dim ** -0.5, 0.1), mlp=mlp))
    CONFIGS[name] = config(layers, width=pick(96, 128, 160, 224, 256), vocab=int(rng.integers(200, 700)))
    return name


def _weights(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    """Seeded weights, already rounded to bfloat16 values so that both precisions and the
    plain implementation compute with the same numbers."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    t: Dict[str, np.ndarray] = {}

    def mat(name, out, inn, gain=1.0):
        t[name] = rng.standard_normal((out, inn)) * gain / np.sqrt(inn)

    def vec(name, n, mean=0.0, std=1.0):
        t[name] = mean + std * rng.standard_normal(n)

    t["embed"] = rng.standard_normal((cfg["vocab"], W))
    for i, layer in enumerate(cfg["layers"]):
        p, x, m = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        vec(p + "norm1", W, 1.0, 0.1)
        vec(p + "ls1", W, 0.7, 0.1)
        if layer["type"] == "gla":
            H, K, V, r = m["heads"], m["dim"], m["vdim"], m["rank"]
            mat(x + "q", H * K, W, 2.0), mat(x + "k", H * K, W), mat(x + "v", H * V, W)
            mat(x + "g", H * V, W), mat(x + "o", W, H * V)
            mat(x + "a1", r, W), mat(x + "a2", H * K, r, 2.0)
            vec(x + "a2.b", H * K, 1.5, 1.0), vec(x + "norm", V, 1.0, 0.1)
        elif layer["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner = H * P
            mat(x + "in", 2 * inner + 2 * G * N + H, W)
            t[x + "conv"] = rng.standard_normal((inner + 2 * G * N, m["conv"])) * 0.5
            vec(x + "conv.b", inner + 2 * G * N, 0.0, 0.2)
            vec(x + "dt_bias", H, -1.0, 0.5)
            t[x + "A_log"] = rng.uniform(-2.0, 0.5, H)
            vec(x + "D", H, 1.0, 0.3), vec(x + "norm", inner, 1.0, 0.1)
            mat(x + "o", W, inner)
        else:
            H, G, D = m["heads"], m["kv_heads"], m["dim"]
            mat(x + "q", H * D, W, 2.0), mat(x + "k", G * D, W, 2.0)
            vec(x + "q.b", H * D, 0.0, 0.3), vec(x + "k.b", G * D, 0.0, 0.3)
            vec(x + "q.norm", D, 1.0, 0.2), vec(x + "k.norm", D, 1.0, 0.2)
            mat(x + "g", H, W), mat(x + "o", W, H * D)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            vec(p + "norm2", W, 1.0, 0.1), vec(p + "ls2", W, 0.7, 0.1)
            mat(p + "mlp.gate", ff, W), mat(p + "mlp.up", ff, W), mat(p + "mlp.down", W, ff)
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


def needle_model(chunk: int) -> str:
    """An attention layer whose weights make one score stand out: the key of token 0 (the
    needle) and the query of token 1 (the probe) share one large direction outside the rotated
    dimensions, every other token has none of it.  A probe's output is then decided by which
    needles its chunk lets it see, and an edge that is off by one shows as a large error."""
    name = f"needle{chunk}"
    if name not in CONFIGS:
        CONFIGS[name] = config([attention(heads=2, kv_heads=1, dim=64, chunk=chunk, rot=32,
                                          scale=1.0)], width=64, vocab=64)
        w = {n: a.copy() for n, a in _weights(CONFIGS[name], 7).items()}
        w["embed"][:, :2] = 0.0
        w["embed"][0, 0] = 8.0
        w["embed"][1, 1] = 8.0
        for m in ("l0.mix.q", "l0.mix.k"):
            w[m] *= 0.25
            w[m][:, :2] = 0.0
        w["l0.mix.k"][63, 0] = 4.0
        w["l0.mix.q"][63, 1] = 4.0
        w["l0.mix.q"][64 + 63, 1] = 4.0
        CUSTOM[name] = _bf16_values(w)
    return name


_dirs: Dict[tuple, str] = {}


def model_dir(name: str, seed: int = 0) -> str:
    """A folder with config.json and model.safetensors (bfloat16) of the configuration."""
    from llmario_b200.weights.safetensors_io import write_safetensors

    key = (name, seed)
    if key not in _dirs:
        d = tempfile.mkdtemp(prefix=f"vunasun_{name}_")
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CONFIGS[name], f)
        write_safetensors(os.path.join(d, "model.safetensors"),
                          {n: torch.from_numpy(a).to(torch.bfloat16)
                           for n, a in weights(name, seed).items()})
        _dirs[key] = d
    return _dirs[key]


@functools.lru_cache(maxsize=None)
def _plain(name: str, seed: int, tokens: tuple) -> np.ndarray:
    return VP.forward(CONFIGS[name], weights(name, seed), list(tokens))


def plain_logits(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    return _plain(name, seed, tuple(int(t) for t in tokens))


@functools.lru_cache(maxsize=None)
def _sensitivity(name: str, seed: int, tokens: tuple) -> np.ndarray:
    """Per position, how far the logits move when the inputs move by about one bfloat16
    rounding or two: the plain implementation run again with the embedding rows scaled by
    1 + 2^-7 N(0, 1).  Some positions are ill-conditioned by design: the first token of a
    sequence leaves a linear-attention head with the rank-one state k v^T, whose output
    (k . q) v is divided by its own size in the head's norm, so that a small k . q decides the
    sign of the whole head."""
    w = dict(weights(name, seed))
    rng = np.random.default_rng(99)
    embed, ref = w["embed"], _plain(name, seed, tokens)
    worst = np.zeros(len(tokens))
    for _ in range(4):           # the largest of four moves: one draw can miss a sign that flips
        w["embed"] = embed * (1 + 2.0 ** -7 * rng.standard_normal(embed.shape))
        moved = VP.forward(CONFIGS[name], w, list(tokens))
        worst = np.maximum(worst, np.abs(moved - ref).max(axis=1))
    return worst


def sensitivity(name: str, tokens: Sequence[int], seed: int = 0) -> np.ndarray:
    return _sensitivity(name, seed, tuple(int(t) for t in tokens))


def tokens_for(name: str, n: int, seed: int) -> List[int]:
    rng = np.random.default_rng(1000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[name]["vocab"], n)]


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
BOUND = {"float32": 2e-4, "bfloat16": 4e-2}


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str = "",
                 bound: Optional[float] = None, slack: Optional[np.ndarray] = None) -> None:
    """``slack``: per row, an allowance on top of the bound (16-bit runs: a multiple of the
    row's :func:`sensitivity`)."""
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    err = np.abs(got.astype(np.float64) - ref)
    tol = (bound if bound is not None else BOUND[dtype]) * max(1e-6, float(np.abs(ref).max()))
    if slack is not None:
        err = np.maximum(0.0, err - slack.reshape((-1,) + (1,) * (err.ndim - 1)))
    worst = np.unravel_index(np.argmax(err), err.shape)
    assert err.max() <= tol, (f"{what} ({dtype}): max |diff| {err.max():.3e} > {tol:.3e} at "
                              f"{tuple(int(w) for w in worst)}")
