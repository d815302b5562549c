"""Typed configuration of the Vunasun decoder, read from the keys of its ``config.json``.

A Vunasun model is a list of layers, each with one mixer (``gla``: gated linear attention;
``mamba2``: a state-space mixer; ``attention``: grouped-query attention inside chunks, whose values
are its keys) and an optional dense gated feed-forward.  The norm sits on a sublayer's output:
``x += ls1 * norm1(mixer(x)); x += ls2 * norm2(ff(x))``.  Every size and every constant that can
differ between two models of the design is read here and nowhere else; tensor names follow
``l<i>.<part>`` as the weight files store them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec

MIXERS = ("gla", "mamba2", "attention")


def _get(d: Dict[str, Any], key: str, kind, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where}: missing key '{key}'")
    try:
        v = kind(d[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: {where}: key '{key}' has value {d[key]!r}, expected "
                          f"{kind.__name__}") from None
    if kind is int and (v <= 0 or v != d[key]):
        raise ConfigError(f"config.json: {where}: key '{key}' must be a positive integer, "
                          f"not {d[key]!r}")
    return v


@dataclass(frozen=True)
class VunasunLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]       # the mixer's sizes and constants, as given
    ff: Optional[int]                        # width of the feed-forward, None: the layer has none

    def m(self) -> Dict[str, Any]:
        return dict(self.mixer)


@dataclass(frozen=True)
class VunasunConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[VunasunLayer, ...]
    max_positions: int = 1 << 17      # the design has no limit of its own: the engine's default

    architecture = "Vunasun"
    model_type = "vunasun"

    # ---------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "VunasunConfig":
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
            ff = None
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}: unsupported mlp kind "
                                      f"{mlp.get('kind')!r} (known: dense)")
                ff = _get(mlp, "ff", int, where + ".mlp")
            layers.append(VunasunLayer(kind, tuple(sorted(_freeze(m).items())), ff))
        max_pos = int(raw.get("max_positions") or cls.max_positions)
        return cls(vocab, width, eps, tuple(layers), max_pos)

    @staticmethod
    def _check_mixer(kind: str, m: Dict[str, Any], where: str) -> None:
        if kind == "gla":
            for key in ("heads", "dim", "vdim"):
                _get(m, key, int, where)
            if _get(m, "tau", float, where) <= 0:
                raise ConfigError(f"config.json: {where}: tau must be positive")
        elif kind == "mamba2":
            for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                _get(m, key, int, where)
            if m["heads"] % m["groups"]:
                raise ConfigError(f"config.json: {where}: {m['heads']} heads in {m['groups']} groups")
            if (m["heads"] * m["vdim"]) % m["norm_groups"]:
                raise ConfigError(f"config.json: {where}: {m['heads'] * m['vdim']} channels in "
                                  f"{m['norm_groups']} norm groups")
        else:
            for key in ("heads", "kv_heads", "dim"):
                _get(m, key, int, where)
            _get(m, "scale", float, where)
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: {where}: {m['heads']} query heads on "
                                  f"{m['kv_heads']} key heads")
            if m.get("vdim") is not None and int(m["vdim"]) != int(m["dim"]):
                raise ConfigError(f"config.json: {where}: the values are the keys, so vdim "
                                  f"{m['vdim']} must equal dim {m['dim']}")
            rot = m.get("rot")
            if rot is not None:
                dims = _get(rot, "dims", int, where + ".rot")
                _get(rot, "base", float, where + ".rot")
                if dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"config.json: {where}.rot: dims {dims} must be even and at "
                                      f"most dim {m['dim']}")
            mask = m.get("mask")
            if mask is not None:
                _get(mask, "size", int, where + ".mask")

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` that reads back as this configuration."""
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.eps}, "layers": []}
        for layer in self.layers:
            out["layers"].append({"type": layer.type, "mixer": _thaw(layer.m()),
                                  "mlp": None if layer.ff is None
                                  else {"kind": "dense", "ff": layer.ff}})
        if self.max_positions != type(self).max_positions:
            out["max_positions"] = self.max_positions
        return out

    # ---------------------------------------------------------------------------------------
    def to_spec(self) -> ModelSpec:
        c = self
        W = c.width

        def norm(width: int, name: str) -> PartSpec:
            return PartSpec("rms_norm", {"width": width, "eps": c.eps,
                                         "tensors": {"weight": (name, (width,))}})

        layers = []
        for i, layer in enumerate(c.layers):
            p = f"l{i}."
            x = p + "mix."
            m = _thaw(layer.m())
            if layer.type == "gla":
                H, K, V = m["heads"], m["dim"], m["vdim"]
                # the decay's low rank is no configuration key: the stored tensors decide it
                # (an optional key "rank" pins it, for models made without files)
                rank = int(m["rank"]) if m.get("rank") else None
                mixer = PartSpec("gla", {
                    "hidden_size": W, "num_heads": H, "key_dim": K, "value_dim": V,
                    "tau": float(m["tau"]), "eps": c.eps,
                    "tensors": {
                        "q": (x + "q", (H * K, W)), "k": (x + "k", (H * K, W)),
                        "v": (x + "v", (H * V, W)), "g": (x + "g", (H * V, W)),
                        "o": (x + "o", (W, H * V)), "norm": (x + "norm", (V,)),
                        "a1": (x + "a1", (rank, W)),
                        "a2": (x + "a2", (H * K, rank)),
                        "a2_bias": (x + "a2.b", (H * K,)),
                    },
                })
            elif layer.type == "mamba2":
                H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
                inner, conv = H * P, H * P + 2 * G * N
                mixer = PartSpec("mamba2", {
                    "hidden_size": W, "num_heads": H, "head_dim": P, "state_dim": N, "groups": G,
                    "conv_taps": m["conv"], "norm_groups": m["norm_groups"], "eps": c.eps,
                    "tensors": {
                        "in": (x + "in", (2 * inner + 2 * G * N + H, W)),
                        "conv": (x + "conv", (conv, m["conv"])),
                        "conv_bias": (x + "conv.b", (conv,)),
                        "dt_bias": (x + "dt_bias", (H,)), "A_log": (x + "A_log", (H,)),
                        "D": (x + "D", (H,)), "norm": (x + "norm", (inner,)),
                        "o": (x + "o", (W, inner)),
                    },
                })
            else:
                H, G, D = m["heads"], m["kv_heads"], m["dim"]
                rot = m.get("rot")
                mixer = PartSpec("attention", {
                    "hidden_size": W, "num_heads": H, "num_kv_heads": G, "head_dim": D,
                    "scale": float(m["scale"]), "window": None,
                    "chunk": int(m["mask"]["size"]) if m.get("mask") else None,
                    "values": "keys",
                    "position": None if rot is None else PartSpec("rope_neox", {
                        "rot_dim": int(rot["dims"]), "theta": float(rot["base"]),
                        "freq_scale": 1.0, "attn_factor": 1.0}),
                    "q_norm": norm(D, x + "q.norm"), "k_norm": norm(D, x + "k.norm"),
                    "tensors": {
                        "q": (x + "q", (H * D, W)), "q_bias": (x + "q.b", (H * D,)),
                        "k": (x + "k", (G * D, W)), "k_bias": (x + "k.b", (G * D,)),
                        "gate": (x + "g", (H, W)), "o": (x + "o", (W, H * D)),
                    },
                })
            block_params: Dict[str, Any] = {
                "mixer_norm": norm(W, p + "norm1"),
                "tensors": {"mixer_scale": (p + "ls1", (W,))},
            }
            if layer.ff is None:
                ffn = PartSpec("none", {})
            else:
                f = p + "mlp."
                ffn = PartSpec("swiglu", {
                    "hidden_size": W, "intermediate_size": layer.ff,
                    "tensors": {"gate": (f + "gate", (layer.ff, W)), "up": (f + "up", (layer.ff, W)),
                                "down": (f + "down", (W, layer.ff))},
                })
                block_params["feed_forward_norm"] = norm(W, p + "norm2")
                block_params["tensors"]["feed_forward_scale"] = (p + "ls2", (W,))
            layers.append(LayerSpec(PartSpec("output_norm_residual", block_params), mixer, ffn, p))

        spec = ModelSpec(
            architecture=c.architecture, vocab_size=c.vocab, hidden_size=W,
            max_positions=c.max_positions,
            embedding=PartSpec("token_embedding", {
                "vocab_size": c.vocab, "hidden_size": W,
                "tensors": {"table": ("embed", (c.vocab, W))}}),
            layers=tuple(layers), run_order=tuple(LayerCall(i) for i in range(len(layers))),
            final_norm=norm(W, "final.norm"),
            head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": W, "tied": False,
                                          "tensors": {"weight": ("head", (c.vocab, W))}}))
        spec.validate()
        return spec


def sized_like(width: int, ff: int, heads: int, kv_heads: int, head_dim: int, layers: int,
               vocab: int) -> VunasunConfig:
    """A configuration for models with random weights at the sizes of a transformer: layers
    repeating (gla, gla, mamba2, attention), every one with a feed-forward of ``ff``; the linear
    attention with key channels of half and value channels of the whole width in heads of 128 x
    256, the state-space mixer with twice the width in heads of 64 over 128 state rows, the
    attention with the given heads, half of each rotated, in chunks of 1,024."""
    mlp = {"kind": "dense", "ff": ff}
    gla = {"type": "gla", "mlp": mlp,
           "mixer": {"heads": max(1, width // 256), "dim": 128, "vdim": 256, "tau": 16.0, "rank": 64}}
    ssm = {"type": "mamba2", "mlp": mlp,
           "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4,
                     "norm_groups": 1}}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
                     "scale": head_dim ** -0.5, "mask": {"size": 1024},
                     "rot": {"dims": head_dim // 2, "base": 1e6}}}
    pattern = [gla, gla, ssm, att]
    return VunasunConfig.from_dict({
        "architecture": "Vunasun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
        "layers": [pattern[i % 4] for i in range(layers)]})


def _freeze(v):
    if isinstance(v, dict):
        return {k: _freeze_value(x) for k, x in v.items()}
    return v


def _freeze_value(v):
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze_value(x)) for k, x in v.items()))
    return v


def _thaw(m: Dict[str, Any]) -> Dict[str, Any]:
    return {k: (dict((a, b) for a, b in v) if isinstance(v, tuple) else v) for k, v in m.items()}
