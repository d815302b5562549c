"""A plain, slow statement of the Vunasun decoder in float64 NumPy: one function per mechanism,
whole sequences from position 0, recurrences token by token.  It shares nothing with the
package: it reads the raw ``config.json`` dictionary and a dictionary of arrays by tensor name.

Notation: ``h`` [T, width] is a sublayer's input, ``W`` [out, in] is applied as ``h @ W.T``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


# --------------------------------------------------------------------------------------------
def gla_mixer(h, t: Dict[str, np.ndarray], p: str, m: dict, eps: float, state=None):
    """Gated linear attention with a decay per key channel.
    S_t = diag(alpha_t) S_{t-1} + k_t v_t^T ;  o_t = S_t^T q_t."""
    T = h.shape[0]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ t[p + "q"].T) * dk ** -0.5
    k = h @ t[p + "k"].T
    v = h @ t[p + "v"].T
    z = (h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "a2.b"]
    alpha = sigmoid(z) ** (1.0 / tau)
    q, k, alpha = (a.reshape(T, H, dk) for a in (q, k, alpha))
    v = v.reshape(T, H, dv)
    S = np.zeros((H, dk, dv), F) if state is None else state
    o = np.zeros((T, H, dv), F)
    for i in range(T):
        S = alpha[i][:, :, None] * S + k[i][:, :, None] * v[i][:, None, :]
        o[i] = np.einsum("hkv,hk->hv", S, q[i])
    o = rms_norm(o, t[p + "norm"], eps).reshape(T, H * dv)
    o = o * silu(h @ t[p + "g"].T)
    return o @ t[p + "o"].T, S


def mamba2_mixer(h, t: Dict[str, np.ndarray], p: str, m: dict, eps: float):
    """State-space mixer with a scalar decay per head.
    S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T ;  y_t = S_t^T C_t + D x_t."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    taps, ng = m["conv"], m["norm_groups"]
    inner = H * P
    u = h @ t[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    # causal convolution per channel: the last column of the kernel meets the current token
    cw, cb = t[p + "conv"], t[p + "conv.b"]
    padded = np.concatenate([np.zeros((taps - 1, xbc.shape[1]), F), xbc], axis=0)
    conv = np.zeros_like(xbc)
    for j in range(taps):
        conv += padded[j:j + T] * cw[:, j]
    xbc = silu(conv + cb)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + t[p + "dt_bias"])
    A = -np.exp(t[p + "A_log"])
    D = t[p + "D"]
    S = np.zeros((H, N, P), F)
    y = np.zeros((T, H, P), F)
    per = H // G
    for i in range(T):
        for hd in range(H):
            g = hd // per
            S[hd] = np.exp(A[hd] * dt[i, hd]) * S[hd] + dt[i, hd] * np.outer(B[i, g], x[i, hd])
            y[i, hd] = S[hd].T @ C[i, g] + D[hd] * x[i, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * t[p + "norm"]
    return y @ t[p + "o"].T


def rotate_half_split(x, pos, dims: int, base: float):
    """x [T, heads, dim]: dimension i < dims/2 is paired with i + dims/2; the rest pass."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half, dtype=F) / dims)
    a = pos[:, None].astype(F) * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def attention_mixer(h, t: Dict[str, np.ndarray], p: str, m: dict, eps: float):
    """Grouped-query softmax attention whose values are the keys as projected; per-head norm
    of q and k, partial rotation, keys visible only inside the query's own chunk, and a
    sigmoid gate per head on the output."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).reshape(T, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).reshape(T, G, d)
    v = k.copy()
    q = rms_norm(q, t[p + "q.norm"], eps)
    k = rms_norm(k, t[p + "k.norm"], eps)
    pos = np.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_half_split(q, pos, rot["dims"], float(rot["base"]))
        k = rotate_half_split(k, pos, rot["dims"], float(rot["base"]))
    size = m["mask"]["size"] if m.get("mask") else None
    i, j = pos[:, None], pos[None, :]
    visible = j <= i
    if size:
        visible &= (i // size) == (j // size)
    gate = sigmoid(h @ t[p + "g"].T)            # [T, H]
    out = np.zeros((T, H, d), F)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        s = np.where(visible, s, -np.inf)
        w = np.exp(s - s.max(axis=1, keepdims=True))
        w /= w.sum(axis=1, keepdims=True)
        out[:, hd] = (w @ v[:, g]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * d) @ t[p + "o"].T


def dense_feed_forward(h, t: Dict[str, np.ndarray], p: str):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


# --------------------------------------------------------------------------------------------
def forward(config: dict, tensors: Dict[str, np.ndarray], tokens, layers_out: Optional[List] = None):
    """Logits [T, vocab] of a whole sequence.  ``layers_out``: the residual stream after every
    layer is appended to it."""
    t = {n: np.asarray(a, dtype=F) for n, a in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = t["embed"][np.asarray(tokens)]
    for i, layer in enumerate(config["layers"]):
        L = f"l{i}."
        kind, m = layer["type"], layer["mixer"]
        if kind == "gla":
            y, _ = gla_mixer(x, t, L + "mix.", m, eps)
        elif kind == "mamba2":
            y = mamba2_mixer(x, t, L + "mix.", m, eps)
        elif kind == "attention":
            y = attention_mixer(x, t, L + "mix.", m, eps)
        else:
            raise ValueError(kind)
        x = x + rms_norm(y, t[L + "norm1"], eps) * t[L + "ls1"]
        if layer.get("mlp") is not None:
            y = dense_feed_forward(x, t, L + "mlp.")
            x = x + rms_norm(y, t[L + "norm2"], eps) * t[L + "ls2"]
        if layers_out is not None:
            layers_out.append(x.copy())
    x = rms_norm(x, t["final.norm"], eps)
    return x @ t["head"].T
