"""A plain, slow statement of the Runidra decoder in float64 NumPy: one function per mechanism,
whole sequences from position 0, the recurrence token by token.  It shares nothing with the
package: it reads the raw ``config.json`` dictionary and a dictionary of arrays by tensor name.

Notation: ``h`` [T, width] is a sublayer's input, ``W`` [out, in] is applied as ``h @ W.T``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def soft_cap(z, cap):
    return cap * np.tanh(z / cap)


# --------------------------------------------------------------------------------------------
def mlstm_mixer(h, t: Dict[str, np.ndarray], p: str, m: dict, eps: float):
    """Matrix memory with exponential gates kept in range by a running maximum ``mx``:
    mx_t = max(f_t + mx_{t-1}, i_t);  S_t = e^(f_t + mx_{t-1} - mx_t) S_{t-1} + e^(i_t - mx_t) k_t v_t^T
    (z_t the same with k_t alone);  o_t = S_t^T q_t / (max(|z_t . q_t|, e^(-mx_t)) + 1e-6)."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ t[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ t[p + "k"].T).reshape(T, H, dk)
    v = (h @ t[p + "v"].T).reshape(T, H, dv)
    gi = soft_cap(h @ t[p + "i"].T + t[p + "i.b"], cap)
    gf = log_sigmoid(soft_cap(h @ t[p + "f"].T + t[p + "f.b"], cap))
    S = np.zeros((H, dk, dv), F)
    z = np.zeros((H, dk), F)
    mx = np.zeros(H, F)
    o = np.zeros((T, H, dv), F)
    for i in range(T):
        new = np.maximum(gf[i] + mx, gi[i])
        keep, take = np.exp(gf[i] + mx - new), np.exp(gi[i] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[i][:, :, None] * v[i][:, None, :]
        z = keep[:, None] * z + take[:, None] * k[i]
        mx = new
        den = np.maximum(np.abs(np.einsum("hk,hk->h", z, q[i])), np.exp(-mx)) + 1e-6
        o[i] = np.einsum("hkv,hk->hv", S, q[i]) / den[:, None]
    o = rms_unit(o, eps).reshape(T, H * dv) * t[p + "norm"]
    o = o * sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def rotate_adjacent(x, pos, dims: int, base: float):
    """Turn the pairs (2i, 2i+1), i < dims/2, of the last axis by pos * base^(-2i/dims)."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = pos[:, None].astype(F) * base ** (-2.0 * i / dims)          # [T, dims/2]
    c, s = np.cos(ang), np.sin(ang)
    while c.ndim < x.ndim:
        c, s = c[:, None], s[:, None]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_attention_mixer(h, t: Dict[str, np.ndarray], p: str, m: dict, eps: float):
    """Queries and keys/values through low-rank latents; one rotated key part for all heads;
    a window of the last ``mask.size`` keys; a sink logit per head in the softmax's sum."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    cq = rms_norm(h @ t[p + "dq"].T, t[p + "dq.norm"], eps)
    q = (cq @ t[p + "uq"].T).reshape(T, H, dn + dr)
    kv = h @ t[p + "dkv"].T
    c = rms_norm(kv[:, :r], t[p + "dkv.norm"], eps)
    rot = m.get("rot")
    k_rot, q_rot = kv[:, r:], q[..., dn:]
    if rot is not None:
        k_rot = rotate_adjacent(k_rot, pos, int(rot["dims"]), float(rot["base"]))
        q_rot = rotate_adjacent(q_rot, pos, int(rot["dims"]), float(rot["base"]))
    k_nope = (c @ t[p + "uk"].T).reshape(T, H, dn)
    val = (c @ t[p + "uv"].T).reshape(T, H, dv)
    s = np.einsum("ihd,jhd->hij", q[..., :dn], k_nope) + np.einsum("ihd,jd->hij", q_rot, k_rot)
    s = s * float(m["scale"])
    d = pos[:, None] - pos[None, :]
    seen = d >= 0
    if m.get("mask") is not None:
        seen &= d < int(m["mask"]["size"])
    s = np.where(seen[None], s, -np.inf)
    sink = t.get(p + "sink")
    top = s.max(axis=-1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink[:, None, None])
    e = np.exp(s - top)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink[:, None, None] - top)
    o = np.einsum("hij,jhd->ihd", e / den, val).reshape(T, H * dv)
    return o @ t[p + "o"].T


# --------------------------------------------------------------------------------------------
def dense_ff(h, t, p: str):
    g = h @ t[p + "gate"].T + t[p + "gate.b"]
    u = h @ t[p + "up"].T + t[p + "up.b"]
    return (gelu_tanh(g) * u) @ t[p + "down"].T + t[p + "down.b"]


def expert_ff(h, t, p: str):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def routed_ff(h, t, p: str, mlp: dict, margins: Optional[list] = None):
    """``margins`` collects, per token, how far the last chosen logit lies above the best one
    that was not chosen (a close call there decides which expert runs)."""
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ t[p + "router"].T + t[p + "router.b"]
    out = np.zeros((h.shape[0], t[p + "e0.down"].shape[0]), F)
    if margins is not None and top < n:
        ordered = -np.sort(-z, axis=1)
        margins.append(ordered[:, top - 1] - ordered[:, top])
    for i in range(h.shape[0]):
        chosen = np.argsort(-z[i], kind="stable")[:top]
        w = np.exp(z[i][chosen] - z[i][chosen].max())
        w = w / w.sum()
        for e, we in zip(chosen, w):
            out[i] += we * expert_ff(h[i:i + 1], t, f"{p}e{int(e)}.")[0]
    if mlp.get("shared") is not None:
        out += expert_ff(h, t, p + "shared.") * sigmoid(h @ t[p + "shared.sg"].T)
    assert n == z.shape[1]
    return out


def feed_forward(h, t, p: str, mlp: dict, margins: Optional[list] = None):
    if mlp.get("kind", "dense") == "dense":
        return dense_ff(h, t, p)
    return routed_ff(h, t, p, mlp, margins)


# --------------------------------------------------------------------------------------------
def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, tensors: Dict[str, np.ndarray], tokens, layers_out: Optional[list] = None,
            margins: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence from position 0.  ``layers_out`` collects the
    residual stream (the sum of the streams) behind every layer run, ``margins`` the routers'
    margins per token (see :func:`routed_ff`), one array per routed layer run."""
    t = {k: np.asarray(v, F) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x0 = t["embed"][np.asarray(tokens)]
    streams = cfg.get("streams")
    xs = [x0.copy() for _ in range(int(streams))] if streams else [x0.copy()]
    for li in run_order(cfg):
        layer = cfg["layers"][li]
        p = f"l{li}."
        subs = [("1", lambda a, L=layer, P=p: (mlstm_mixer if L["type"] == "mlstm" else
                                                latent_attention_mixer)(a, t, P + "mix.", L["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append(("2", lambda a, L=layer, P=p: feed_forward(a, t, P + "mlp.", L["mlp"], margins)))
        for q, fn in subs:
            if streams:
                cin, cout, mix = t[f"{p}hc{q}.in"], t[f"{p}hc{q}.out"], t[f"{p}hc{q}.mix"]
                u = sum(cin[s] * xs[s] for s in range(len(xs)))
                y = fn(rms_norm(u, t[f"{p}norm{q}"], eps))
                xs = [sum(mix[s, k] * xs[s] for s in range(len(xs))) + cout[k] * y
                      for k in range(len(xs))]
            else:
                xs[0] = xs[0] + fn(rms_norm(xs[0], t[f"{p}norm{q}"], eps))
        if layers_out is not None:
            layers_out.append(sum(xs))
    x = rms_norm(sum(xs), t["final.norm"], eps)
    z = (x @ t["head"].T) * float(cfg.get("logit_scale", 1.0))
    if cfg.get("logit_softcap"):
        z = soft_cap(z, float(cfg["logit_softcap"]))
    return z
