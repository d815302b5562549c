"""Attention whose queries, keys and values pass through low-rank latents.

With ``h`` the mixer's input, per token:

* ``c_q = norm(W_dq h)`` (gain ``dq_norm``), ``q = W_uq c_q``; every head's slice of q is
  [``head_dim`` plain | ``rot_dim`` rotated];
* ``W_dkv h`` = [``kv_rank`` numbers, normed with gain ``dkv_norm``: the latent ``c`` | ``rot_dim``
  numbers, not normed: one rotated key part shared by all heads];
* head h's plain key is ``U_k,h c`` and its value ``U_v,h c``; the score of a query and a key is
  ``(q_plain . k_plain + q_rot . k_rot) * scale``;
* the rotation turns adjacent pairs (2i, 2i + 1) of the rotated parts by ``pos * base^(-2i/dims)``;
* a query at position p sees the keys at p - window + 1 .. p; an optional ``sink`` per head adds
  ``exp(sink)`` to the softmax's sum (a key without a value);
* the heads' outputs, concatenated, are projected by ``W_o``.

The cache holds ``c`` and the rotated key part, nothing per head: one key row of ``kv_rank +
rot_dim`` channels per token.  The heads' key maps are applied to the queries (``U_k,h^T q_plain``) and their value maps
to the attention's output (``U_v,h sum_j p_j c_j``), so the attention itself runs as one shared key
head whose values are the first ``kv_rank`` channels of its keys.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import driver, kernels
from ..cache import PagedKV
from ..config.spec import ConfigError, PartSpec
from .base import (BoundCall, StepContext, build_part, optional_tensor_of, register_part,
                   tensor_of)
from .linear import Linear
from .recurrent import _f32, _padded_rows


class LatentAttention:
    graph_safe = True

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], dtype, device):
        self.hidden = int(spec["hidden_size"])
        self.heads = H = int(spec["num_heads"])
        self.dim = D = int(spec["head_dim"])
        self.rot_dim = R = int(spec.get("rot_dim") or 0)
        self.value_dim = V = int(spec["value_dim"])
        self.q_rank = int(spec["q_rank"])
        self.kv_rank = C = int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        self.window = spec.get("window")
        self.mask = kernels.mask_code(self.window, None)
        self.key_dim = C + R                     # channels of a cached key row
        if self.key_dim > kernels.ATTENTION_MAX_HEAD_DIM:
            raise ConfigError(f"latent attention: a key row of {C} + {R} channels; the attention "
                              f"kernels take up to {kernels.ATTENTION_MAX_HEAD_DIM}")
        self.position = (build_part("position", spec["position"], weights, dtype, device)
                         if spec.get("position") is not None else None)
        if self.position is not None and (not hasattr(self.position, "step_angles")
                                          or self.position.rot_dim > R):
            raise ConfigError("latent attention rotates pairs of its rotated part: it needs a "
                              "rotary position part of at most rot_dim dimensions")
        t = {r: tensor_of(spec, r, weights) for r in ("dq", "uq", "dkv", "uk", "uv", "o")}
        if tuple(t["dkv"].shape) != (C + R, self.hidden) or tuple(t["uq"].shape) != (H * (D + R), self.q_rank):
            raise ConfigError("latent attention: the projections do not have the sizes of the spec")
        self.down_proj = _padded_rows([t["dq"], t["dkv"]], self.hidden)   # [c_q | c | k_rot]
        self.q_proj = Linear(t["uq"])
        # head h's key map, transposed: it is applied to the query's plain part
        self.key_maps = t["uk"].view(H, D, C).transpose(1, 2).contiguous()        # [H, C, D]
        self.value_maps = t["uv"].view(H, V, C).contiguous()                      # [H, V, C]
        self.o_proj = Linear(t["o"])
        self.q_gain = _f32(tensor_of(spec, "dq_norm", weights), device)
        self.c_gain = _f32(tensor_of(spec, "dkv_norm", weights), device)
        sink = optional_tensor_of(spec, "sink", weights)
        self.sink = None if sink is None else _f32(sink, device)

    def cache_need(self):
        return PagedKV(1, self.key_dim, self.window)

    def streamed_weights(self):
        return [self.down_proj.weight, self.q_proj.weight, self.key_maps, self.value_maps,
                self.o_proj.weight]

    def forward(self, ctx: StepContext, call: BoundCall, h: torch.Tensor, x: torch.Tensor,
                accumulate: bool = True) -> None:
        rows, H, D, R, C, V = ctx.rows, self.heads, self.dim, self.rot_dim, self.kv_rank, self.value_dim
        view = ctx.cache.view(call.cache_entry)
        if view is None:
            raise RuntimeError(f"run-order entry {call.index}: attention needs a cache")
        # With few rows the products are cut along K and add partial sums: their destinations are
        # then buffers that are created as zeros and that the kernels which consume them clear
        # again, so no clearing launch runs.
        kept_zero = rows <= kernels.SPLIT_K_MAX_ROWS
        z = ".z" if kept_zero else ""
        proj = ctx.buffer("latent.proj" + z, (rows, self.down_proj.out_features), torch.float32,
                          zero=kept_zero)
        self.down_proj(h, proj, out_is_zero=kept_zero)
        angles = self.position.step_angles(ctx) if self.position is not None else None
        cq = ctx.buffer("latent.cq", (rows, self.q_rank))
        kernels.latent_store(proj, self.q_gain, self.c_gain, angles, cq, view, ctx.row_slot,
                             ctx.row_pos, self.q_rank, C, R, self.eps, call.writes_cache,
                             clear=kept_zero)
        q = ctx.buffer("latent.q" + z, (rows, H * (D + R)), torch.float32, zero=kept_zero)
        self.q_proj(cq, q, out_is_zero=kept_zero)
        q_plain = ctx.buffer("latent.q_plain", (rows, H * D))
        q_full = ctx.buffer("latent.q_full", (rows, H * self.key_dim))
        kernels.latent_query(q, angles, q_plain, q_full, H, D, R, C, clear=kept_zero)
        kernels.head_linear(q_plain.view(rows, H, D), self.key_maps,
                            q_full.view(rows, H, self.key_dim)[:, :, :C])
        # sum_j p_j c_j per head.  The tensor-core kernels work on whole value rows (what lies
        # behind the latent in a value row of the cache is zero and never written); the generic
        # kernel is told to stop at the latent's end.
        whole = driver.tensor_core_attention(ctx.dtype, view, H, 1, self.key_dim)
        vd = self.key_dim if whole else C
        mixed = ctx.buffer("latent.mixed", (rows, H * vd))
        driver.attention(ctx, q_full, mixed, view, H, 1, self.key_dim, self.scale, self.mask,
                         sink=self.sink, value_dim=None if whole else C)
        out = ctx.buffer("latent.out", (rows, H * V))
        kernels.head_linear(mixed.view(rows, H, vd)[:, :, :C], self.value_maps,
                            out.view(rows, H, V))
        self.o_proj(out, x, accumulate=accumulate)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
