"""Typed configuration of the Runidra decoder, read from the keys of its ``config.json``.

A Runidra model is a list of layers, each with one mixer (``mlstm``: a matrix memory with
exponential gates; ``latent_attention``: attention whose queries, keys and values pass through
low-rank latents, with one rotated key part for all heads, a sliding window and a sink in the
softmax) and an optional feed-forward (``dense``: gated, tanh-form gelu, biases; ``moe``: routed
experts with a gated shared expert).  Sublayers are pre-norm.  With the key ``streams`` the residual is kept as that many streams
that every sublayer reads through learned weights and writes through a learned mixing matrix.
``loop`` repeats a range of layers (shared weights, a cache or state per repetition).  The logits are scaled and soft-capped.  Every size and constant that can differ
between two models of the design is read here and nowhere else; tensor names follow ``l<i>.<part>``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .vunasun import _freeze, _get, _thaw

MIXERS = ("mlstm", "latent_attention")
MEMORY_FLOOR = 1e-6        # added to the matrix memory's normaliser: fixed by the design


@dataclass(frozen=True)
class RunidraLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]       # the mixer's sizes and constants, as given
    mlp: Optional[Tuple[Tuple[str, Any], ...]]   # the feed-forward's, None: the layer has none

    def m(self) -> Dict[str, Any]:
        return _thaw(dict(self.mixer))

    def f(self) -> Optional[Dict[str, Any]]:
        return None if self.mlp is None else _thaw(dict(self.mlp))


@dataclass(frozen=True)
class RunidraConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[RunidraLayer, ...]
    streams: Optional[int] = None             # None: one residual stream and the plain sum
    loop: Optional[Tuple[int, int, int]] = None    # (start, stop, times)
    logit_scale: float = 1.0
    logit_softcap: float = 0.0                # 0: none
    max_positions: int = 1 << 17      # the design has no limit of its own: the engine's default

    architecture = "Runidra"
    model_type = "runidra"

    # ---------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "RunidraConfig":
        vocab = _get(raw, "vocab", int, "model")
        width = _get(raw, "width", int, "model")
        eps = _get(raw.get("norm"), "eps", float, "norm")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            kind = e.get("type") if isinstance(e, dict) else None
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: unsupported type {kind!r} "
                                  f"(known: {', '.join(MIXERS)})")
            m = e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}: missing 'mixer'")
            cls._check_mixer(kind, m, where + ".mixer")
            mlp = e.get("mlp")
            if mlp is not None:
                cls._check_mlp(mlp, where + ".mlp")
            layers.append(RunidraLayer(kind, tuple(sorted(_freeze(m).items())),
                                       None if mlp is None else tuple(sorted(_freeze(mlp).items()))))
        streams = None
        if raw.get("streams") is not None:
            streams = _get(raw, "streams", int, "model")
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            for key in ("start", "stop", "times"):
                if not isinstance(lp.get(key), int) or isinstance(lp.get(key), bool):
                    raise ConfigError(f"config.json: loop: key '{key}' must be an integer")
            loop = (lp["start"], lp["stop"], lp["times"])
            if not (0 <= loop[0] <= loop[1] <= len(layers)) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {lp} does not fit {len(layers)} layers")
        cap = raw.get("logit_softcap")
        max_pos = int(raw.get("max_positions") or cls.max_positions)
        return cls(vocab, width, eps, tuple(layers), streams, loop,
                   float(raw.get("logit_scale", 1.0)), float(cap) if cap else 0.0, max_pos)

    @staticmethod
    def _check_mixer(kind: str, m: Dict[str, Any], where: str) -> None:
        if kind == "mlstm":
            for key in ("heads", "dim", "vdim"):
                _get(m, key, int, where)
            if m.get("gate_cap") is not None and _get(m, "gate_cap", float, where) <= 0:
                raise ConfigError(f"config.json: {where}: gate_cap must be positive")
        else:
            for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                _get(m, key, int, where)
            _get(m, "scale", float, where)
            rot_dim = m.get("rot_dim") or 0
            if not isinstance(rot_dim, int) or rot_dim < 0:
                raise ConfigError(f"config.json: {where}: rot_dim {rot_dim!r}")
            rot = m.get("rot")
            if rot is not None:
                dims = _get(rot, "dims", int, where + ".rot")
                _get(rot, "base", float, where + ".rot")
                if dims % 2 or dims > rot_dim:
                    raise ConfigError(f"config.json: {where}.rot: dims {dims} must be even and at "
                                      f"most rot_dim {rot_dim}")
            if m.get("mask") is not None:
                _get(m["mask"], "size", int, where + ".mask")

    @staticmethod
    def _check_mlp(mlp: Dict[str, Any], where: str) -> None:
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            _get(mlp, "ff", int, where)
        elif kind == "moe":
            _get(mlp.get("expert"), "ff", int, where + ".expert")
            n = _get(mlp.get("router"), "experts", int, where + ".router")
            top = _get(mlp.get("router"), "top", int, where + ".router")
            if top > n:
                raise ConfigError(f"config.json: {where}: top {top} of {n} experts")
            if mlp.get("shared") is not None:
                _get(mlp["shared"], "ff", int, where + ".shared")
        else:
            raise ConfigError(f"config.json: {where}: unsupported mlp kind {kind!r} "
                              "(known: dense, moe)")

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` that reads back as this configuration."""
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.eps}, "layers": []}
        for layer in self.layers:
            out["layers"].append({"type": layer.type, "mixer": _deep(layer.m()),
                                  "mlp": None if layer.mlp is None else _deep(layer.f())})
        if self.streams is not None:
            out["streams"] = self.streams
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.logit_scale != 1.0:
            out["logit_scale"] = self.logit_scale
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != type(self).max_positions:
            out["max_positions"] = self.max_positions
        return out

    def run_order(self) -> Tuple[int, ...]:
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b, times = self.loop
        return tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))

    # ---------------------------------------------------------------------------------------
    def to_spec(self) -> ModelSpec:
        c = self
        W = c.width

        def norm(width: int, name: str) -> PartSpec:
            return PartSpec("rms_norm", {"width": width, "eps": c.eps,
                                         "tensors": {"weight": (name, (width,))}})

        def gated(prefix: str, ff: int, activation: str, biases: bool) -> PartSpec:
            t = {"gate": (prefix + "gate", (ff, W)), "up": (prefix + "up", (ff, W)),
                 "down": (prefix + "down", (W, ff))}
            if biases:
                t.update(gate_bias=(prefix + "gate.b", (ff,)), up_bias=(prefix + "up.b", (ff,)),
                         down_bias=(prefix + "down.b", (W,)))
            return PartSpec("gated", {"hidden_size": W, "intermediate_size": ff,
                                      "activation": activation, "tensors": t})

        layers = []
        for i, layer in enumerate(c.layers):
            p = f"l{i}."
            x = p + "mix."
            m = layer.m()
            if layer.type == "mlstm":
                H, K, V = m["heads"], m["dim"], m["vdim"]
                mixer = PartSpec("mlstm", {
                    "hidden_size": W, "num_heads": H, "key_dim": K, "value_dim": V,
                    "gate_cap": float(m["gate_cap"]) if m.get("gate_cap") else 0.0,
                    "eps": c.eps, "floor": MEMORY_FLOOR,
                    "tensors": {
                        "q": (x + "q", (H * K, W)), "k": (x + "k", (H * K, W)),
                        "v": (x + "v", (H * V, W)), "g": (x + "g", (H * V, W)),
                        "i": (x + "i", (H, W)), "i_bias": (x + "i.b", (H,)),
                        "f": (x + "f", (H, W)), "f_bias": (x + "f.b", (H,)),
                        "norm": (x + "norm", (H * V,)), "o": (x + "o", (W, H * V)),
                    },
                })
            else:
                H, D, V = m["heads"], m["dim"], m["vdim"]
                R, Rq, Rkv = int(m.get("rot_dim") or 0), m["q_rank"], m["kv_rank"]
                rot = m.get("rot")
                mixer = PartSpec("latent_attention", {
                    "hidden_size": W, "num_heads": H, "head_dim": D, "rot_dim": R, "value_dim": V,
                    "q_rank": Rq, "kv_rank": Rkv, "scale": float(m["scale"]), "eps": c.eps,
                    "window": int(m["mask"]["size"]) if m.get("mask") else None,
                    "position": None if rot is None or not R else PartSpec("rope_normal", {
                        "rot_dim": int(rot["dims"]), "theta": float(rot["base"]),
                        "freq_scale": 1.0, "attn_factor": 1.0}),
                    "tensors": {
                        "dq": (x + "dq", (Rq, W)), "dq_norm": (x + "dq.norm", (Rq,)),
                        "uq": (x + "uq", (H * (D + R), Rq)),
                        "dkv": (x + "dkv", (Rkv + R, W)), "dkv_norm": (x + "dkv.norm", (Rkv,)),
                        "uk": (x + "uk", (H * D, Rkv)), "uv": (x + "uv", (H * V, Rkv)),
                        "sink": (x + "sink", (H,)), "o": (x + "o", (W, H * V)),
                    },
                })
            f = p + "mlp."
            mlp = layer.f()
            if mlp is None:
                ffn = PartSpec("none", {})
            elif mlp.get("kind", "dense") == "dense":
                ffn = gated(f, int(mlp["ff"]), "gelu_tanh", True)
            else:
                E, top, ff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
                t = {"router": (f + "router", (E, W)), "router_bias": (f + "router.b", (E,))}
                for e in range(E):
                    t[f"gate{e}"] = (f"{f}e{e}.gate", (ff, W))
                    t[f"up{e}"] = (f"{f}e{e}.up", (ff, W))
                    t[f"down{e}"] = (f"{f}e{e}.down", (W, ff))
                params: Dict[str, Any] = {"hidden_size": W, "intermediate_size": ff,
                                          "experts": E, "top": top, "tensors": t}
                if mlp.get("shared") is not None:
                    params["shared"] = gated(f + "shared.", int(mlp["shared"]["ff"]), "silu",
                                             False)
                    t["shared_gate"] = (f + "shared.sg", (1, W))
                ffn = PartSpec("moe", params)
            if c.streams is None:
                block = PartSpec("pre_norm_residual", {
                    "mixer_norm": norm(W, p + "norm1"),
                    "feed_forward_norm": norm(W, p + "norm2") if mlp is not None else None})
            else:
                S = c.streams
                t = {"mixer_in": (p + "hc1.in", (S,)), "mixer_out": (p + "hc1.out", (S,)),
                     "mixer_mix": (p + "hc1.mix", (S, S))}
                bp: Dict[str, Any] = {"streams": S, "mixer_norm": norm(W, p + "norm1"),
                                      "tensors": t}
                if mlp is not None:
                    bp["feed_forward_norm"] = norm(W, p + "norm2")
                    t.update(feed_forward_in=(p + "hc2.in", (S,)),
                             feed_forward_out=(p + "hc2.out", (S,)),
                             feed_forward_mix=(p + "hc2.mix", (S, S)))
                block = PartSpec("hyper_connection", bp)
            layers.append(LayerSpec(block, mixer, ffn, p))

        spec = ModelSpec(
            architecture=c.architecture, vocab_size=c.vocab, hidden_size=W,
            max_positions=c.max_positions,
            embedding=PartSpec("token_embedding", {
                "vocab_size": c.vocab, "hidden_size": W,
                "tensors": {"table": ("embed", (c.vocab, W))}}),
            layers=tuple(layers), run_order=tuple(LayerCall(i) for i in c.run_order()),
            final_norm=norm(W, "final.norm"),
            head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": W, "tied": False,
                                          "scale": c.logit_scale, "soft_cap": c.logit_softcap,
                                          "tensors": {"weight": ("head", (c.vocab, W))}}),
            residual_streams=c.streams)
        spec.validate()
        return spec


def sized_like(width: int, ff: int, heads: int, head_dim: int, layers: int, vocab: int,
               window: int = 1024, experts: int = 8, top: int = 2) -> RunidraConfig:
    """A configuration for models with random weights at the sizes of a transformer: layers
    repeating (latent attention + dense, matrix memory + routed experts, latent attention +
    dense, latent attention + routed experts) on two residual streams.  The attention keeps a
    latent of 64 and a rotated part of 64 per token (one key row of 128; smaller for heads below
    64), queries through a latent of a quarter of the width; the memory has heads of 128 x 128
    (at most half the width); at most 16 attention heads; the routed experts are
    `experts` of width ff / top with `top` chosen, beside a shared one of the same width."""
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // top}, "router": {"experts": experts, "top": top},
           "shared": {"ff": ff // top}}
    rot = min(64, head_dim // 2)
    heads = min(heads, 16)      # the tensor-core decode kernels take up to 16 query heads per key head
    att = {"heads": heads, "dim": head_dim - rot, "rot_dim": rot, "vdim": head_dim,
           "q_rank": max(64, width // 4), "kv_rank": 128 - rot if head_dim >= 64 else 2 * head_dim,
           "scale": head_dim ** -0.5, "mask": {"size": window}, "rot": {"dims": rot, "base": 1e6}}
    mem = {"heads": max(1, width // 256), "dim": min(128, width // 2), "vdim": min(128, width // 2),
           "gate_cap": 15.0}
    pattern = [{"type": "latent_attention", "mixer": att, "mlp": dense},
               {"type": "mlstm", "mixer": mem, "mlp": moe},
               {"type": "latent_attention", "mixer": att, "mlp": dense},
               {"type": "latent_attention", "mixer": att, "mlp": moe}]
    return RunidraConfig.from_dict({
        "architecture": "Runidra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
        "streams": 2, "logit_scale": 1.0, "logit_softcap": 30.0,
        "layers": [copy.deepcopy(pattern[i % 4]) for i in range(layers)]})


def _deep(v):
    if isinstance(v, dict):
        return {k: _deep(x) for k, x in v.items()}
    if isinstance(v, tuple) and all(isinstance(x, tuple) and len(x) == 2 for x in v) and v:
        return {k: _deep(x) for k, x in v}
    return v
