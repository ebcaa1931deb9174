"""Grouped-query sliding-window attention with per-head q / k norms around a rotate-half rotation, on ragged rows and the paged cache.

What this adds to :class:`ConvWindowAttention` (row-wide norms, interleaved rotation, convolved projections), each a constructor
parameter so that other stacks can combine them:

* ``norm_at``: every q and k head is RMS-normalised over its own ``head_dim`` channels, ``"pre"`` the rotation or ``"post"`` it
  (``None``: not at all); ``norm_weight`` adds a learned weight ``[head_dim]`` shared by the heads (``q_norm_weight`` / ``k_norm_weight``);
* ``rot_dims`` / ``rot_base`` / ``rot_scaling``: rotary positions on the first ``rot_dims`` channels of a head in the rotate-half layout
  (channel ``i`` pairs with ``i + rot_dims / 2``); ``rot_scaling = {factor, low, high, original}`` divides low frequencies by
  ``factor`` with a smooth band between the wavelengths ``original / high`` and ``original / low`` (the Llama-3 rule,
  :func:`modules.rope.compute_inv_freq`); angles are formed in fp64;
* ``head_temp``: the score of head ``h`` is multiplied by a learned number ``head_temp[h]`` besides ``scale``;
* ``sink``: ``exp(sinks[h])`` is one more term of head ``h``'s softmax denominator (nothing is read for it and ``scale`` does not apply);
* ``out_gate``: the concatenated heads are multiplied by ``sigmoid(W_g x)`` before the output projection;
* ``value_from_key``: there is no value projection; the raw k slice of the projection doubles as the value (untouched by norm or
  rotation) and is kept in the value cache beside the normalised, rotated key;
* ``window``: key ``j`` is visible from position ``i`` when ``i - window < j <= i`` (``None``: every ``j <= i``).

``own_in_proj=False``: the module owns no input projection and :meth:`forward_projected` takes rows ``q | k | [v] | [gate]`` that
someone else projected (mixers that sit side by side on one input share one GEMM); ``in_width`` is the number of such channels.

Data flow (CUDA: csrc/seqmix.cu, one kernel per line after the first):

    p = W_in x                          q | k | v | gate in ONE GEMM
    q = head_norm_rope_append(p)        per-head norms + rotation + paged cache write of k and v
    o = paged_window_attention(q)       fp32 scores / softmax over the cache (window, sink, per-head temperature), times sigmoid(gate)
    y = W_o o
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import ops
from ...parallel.layers import ColumnParallelLinear, RowParallelLinear
from ..rope import compute_inv_freq
from .conv_window_attention import ragged_rope_tables

_NORM_AT = {None: 0, "pre": 1, "post": 2}


class HeadNormWindowAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, *, rot_dims: int, rot_base: float,
                 rot_scaling: Optional[dict] = None, scale: float, window: Optional[int], eps: float, layer_idx: int, norm_at: Optional[str] = "pre",
                 norm_weight: bool = True, head_temp: bool = False, sink: bool = False, out_gate: bool = False, value_from_key: bool = False,
                 own_in_proj: bool = True, dtype=torch.bfloat16, device=None, tp_group=None):
        super().__init__()
        if tp_group is not None and tp_group.size != 1:
            raise NotImplementedError("head-norm window attention: tensor parallel degree 1")
        if num_heads % num_kv_heads:
            raise ValueError("query heads must be a multiple of key / value heads")
        if value_from_key and v_head_dim != head_dim:
            raise ValueError("values taken from the keys have the keys' size")
        if rot_dims % 2 or rot_dims > head_dim:
            raise ValueError("rotated channels: an even number, at most the head size")
        self.n_q, self.n_kv, self.head_dim, self.v_head_dim = num_heads, num_kv_heads, head_dim, v_head_dim
        self.rot_dims, self.scale, self.eps, self.layer_idx = int(rot_dims), float(scale), float(eps), layer_idx
        self.window = int(window) if window else None
        self.norm_at, self.value_from_key = _NORM_AT[norm_at], bool(value_from_key)
        self.Cq, self.Ck = num_heads * head_dim, num_kv_heads * head_dim
        self.Cv = 0 if value_from_key else num_kv_heads * v_head_dim
        self.Co = num_heads * v_head_dim
        self.Cg = self.Co if out_gate else 0
        self.in_width = self.Cq + self.Ck + self.Cv + self.Cg
        self.in_proj = ColumnParallelLinear(hidden_size, self.in_width, bias=False, gather_output=False, dtype=dtype, device=device,
                                            tensor_model_parallel_group=tp_group) if own_in_proj else None
        self.o_proj = RowParallelLinear(self.Co, hidden_size, bias=False, input_is_parallel=True, dtype=dtype, device=device,
                                        tensor_model_parallel_group=tp_group)
        f32 = dict(dtype=torch.float32, device=device)
        with_w = bool(norm_weight) and self.norm_at != 0
        self.q_norm_weight = nn.Parameter(torch.ones(head_dim, **f32), requires_grad=False) if with_w else None
        self.k_norm_weight = nn.Parameter(torch.ones(head_dim, **f32), requires_grad=False) if with_w else None
        self.head_temp = nn.Parameter(torch.ones(num_heads, **f32), requires_grad=False) if head_temp else None
        self.sinks = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False) if sink else None
        if self.rot_dims:
            sc = None
            if rot_scaling:
                sc = dict(rope_type="llama3", factor=float(rot_scaling["factor"]), low_freq_factor=float(rot_scaling["low"]),
                          high_freq_factor=float(rot_scaling["high"]), original_max_position_embeddings=rot_scaling["original"])
            inv, _ = compute_inv_freq(self.rot_dims, float(rot_base), sc, dtype=torch.float64)
            self.register_buffer("rope_inv_freq", inv.to(device=device, dtype=torch.float64), persistent=False)
            self.rope_tag = ("half", self.rot_dims, float(rot_base), tuple(sorted(sc.items())) if sc else None)

    def state_specs(self, cache_index=None):
        return {}

    def kv_shape(self):
        return (self.n_kv, self.head_dim, self.v_head_dim)

    def forward(self, x, meta, kv_mgr, cache_index=None):
        return self.forward_projected(self.in_proj(x), meta, kv_mgr, cache_index)

    def forward_projected(self, p, meta, kv_mgr, cache_index=None):
        B, T = p.shape[:2]
        ex = meta.extras
        ctx, qlen = ex["ctx_len"], ex["q_len"]
        cos, sin = ragged_rope_tables(meta, T, self.rot_dims, 0.0, self.rope_inv_freq, 1.0, self.rope_tag) if self.rot_dims else (None, None)
        k_cache, v_cache = kv_mgr.get_kv_by_layer_id(self.layer_idx if cache_index is None else cache_index)
        q = ops.head_norm_rope_append(p, self.n_q, self.n_kv, self.head_dim, self.v_head_dim, cos, sin, self.q_norm_weight, self.k_norm_weight,
                                      self.norm_at, self.eps, self.value_from_key, k_cache, v_cache, meta.block_table, ctx, qlen)
        gate = p[..., self.Cq + self.Ck + self.Cv:self.in_width] if self.Cg else None
        o = ops.paged_window_attention(q, k_cache, v_cache, meta.block_table, ctx, qlen, self.scale, None, self.window, 0, gate, self.sinks,
                                       head_scale=self.head_temp)
        return self.o_proj(o)
