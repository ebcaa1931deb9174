"""Recurrent mixers on ragged rows with carried state (chunked prompts, mixed prefill / decode batches): Mamba-2 and the gated delta rule.

``in_proj`` rows are ``[z: inner | x: inner | B: G N | C: G N | dt: heads]``.  x, B and C pass a depthwise causal convolution (+bias)
and SiLU; ``dt = softplus(dt + dt_bias)``; per head ``S <- exp(-exp(A_log) dt) S + dt B x^T`` (fp32, ``[N, head_dim]``),
``y = S^T C + D x``; the heads are gated by ``silu(z)`` FIRST and then RMS-normalised in ``norm_groups`` equal parts, times a weight.
Decays, step sizes, the state and the norm are fp32 whatever the activation dtype.  The convolution tail and the state of a
sequence live in its state line (``RecurrentStateCache``), so a prompt may arrive in portions of any size and rows of one batch may be
at different places of their sequences.  The per-token PyTorch loop of ``contrib/models/hybrid_family.py::Mamba2Mixer`` serves
whole-prompt prefill only; this module is the kernel path (csrc/seqmix.cu: short_conv, ssd_scan, group_rmsnorm).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear


class RaggedMamba2Mixer(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, state_size: int, groups: int, norm_groups: int,
                 conv_taps: int, eps: float, layer_idx: int, dtype=torch.bfloat16, device=None, tp_group=None, own_in_proj: bool = True):
        """``own_in_proj=False``: the module owns no input projection and :meth:`forward_projected` takes rows someone else projected
        (``in_width`` channels: mixers side by side on one input share one GEMM)."""
        super().__init__()
        if num_heads % groups or (num_heads * head_dim) % norm_groups:
            raise ValueError("Mamba-2: heads must divide into groups and the inner width into norm groups")
        if tp_group is not None and tp_group.size != 1:
            raise NotImplementedError("ragged Mamba-2 mixer: tensor parallel degree 1")
        self.nh, self.P, self.N, self.G, self.norm_groups = num_heads, head_dim, state_size, groups, norm_groups
        self.taps, self.eps, self.layer_idx = conv_taps, eps, layer_idx
        self.inner = num_heads * head_dim
        self.conv_dim = self.inner + 2 * groups * state_size
        self.in_width = self.inner + self.conv_dim + num_heads
        self.in_proj = ColumnParallelLinear(hidden_size, self.in_width, bias=False, gather_output=False,
                                            dtype=dtype, device=device, tensor_model_parallel_group=tp_group) if own_in_proj else None
        self.out_proj = RowParallelLinear(self.inner, hidden_size, bias=False, input_is_parallel=True, dtype=dtype, device=device,
                                          tensor_model_parallel_group=tp_group)
        f32 = dict(dtype=torch.float32, device=device)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_dim, conv_taps, **f32), requires_grad=False)
        self.conv_bias = nn.Parameter(torch.zeros(self.conv_dim, **f32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False)
        self.D = nn.Parameter(torch.ones(num_heads, **f32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(self.inner, **f32), requires_grad=False)
        self.conv_state, self.ssm_state = f"ssm_conv{layer_idx}", f"ssm_state{layer_idx}"

    def state_specs(self, cache_index=None):
        return {self.conv_state: (self.taps - 1, self.conv_dim), self.ssm_state: ((self.nh, self.N, self.P), torch.float32)}

    def forward(self, x, meta, kv_mgr, cache_index=None):
        return self.forward_projected(self.in_proj(x), meta, kv_mgr, cache_index)

    def forward_projected(self, p, meta, kv_mgr, cache_index=None):
        ex = meta.extras
        ctx, qlen, lines = ex["ctx_len"], ex["q_len"], ex["state_lines"]
        I, Cd = self.inner, self.conv_dim
        z, u, dt = p[..., :I], p[..., I:I + Cd], p[..., I + Cd:I + Cd + self.nh]
        states = kv_mgr.states
        cst = states.tensor(self.conv_state)
        sst = states.tensor(self.ssm_state)
        xBC = ops.short_conv(u, self.conv_weight, self.conv_bias, cst, lines, ctx, qlen, silu=True)
        ops.short_conv_update(u, cst, lines, ctx, qlen)
        y = ops.ssd_scan(xBC, dt, z, self.A_log, self.dt_bias, self.D, sst, lines, ctx, qlen, self.nh, self.P, self.N, self.G)
        y = ops.group_rmsnorm(y, self.norm_weight, self.norm_groups, self.eps, out_dtype=p.dtype)
        return self.out_proj(y)


class RaggedGatedDeltaMixer(nn.Module):
    """Gated delta rule on ragged rows.  Projection rows are ``[q: n_qk D | k: n_qk D | v: heads Dv | beta: heads | a: heads | gate: heads Dv]``
    (head ``h`` reads q / k head ``h // (heads / n_qk)``).  q, k and v pass a depthwise causal convolution (no bias) and SiLU; q and k
    are scaled to unit length per head (``UNIT_EPS`` under the root), q also by ``D^-1/2``; the write strength is ``b = sigmoid(beta)``
    and the decay has ``log decay = -exp(A_log) * softplus(a + dt_bias)``.  Per head the fp32 state ``M [D, Dv]`` is first shrunk,
    ``M *= decay``, then corrected along ``k`` towards ``v``: ``e = b * (v - M' k)``, ``M += outer(k, e)``; the output reads the corrected
    state, ``y = M' q``.  Every head of ``y`` is RMS-normalised over ``Dv`` with a weight shared by the heads, multiplied by ``silu(gate)``,
    and projected out.  Unit norms, ``beta``, decays and the state are fp32 whatever
    the activation dtype.  The convolution tail and the state of a sequence live in its state line (csrc/seqmix.cu: short_conv,
    gated_delta_scan, head_rmsnorm_gate)."""
    UNIT_EPS = 1e-6      # inside the root of the q / k unit norms (fixed by the rule)

    def __init__(self, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, v_head_dim: int, conv_taps: int, eps: float,
                 layer_idx: int, dtype=torch.bfloat16, device=None, tp_group=None, own_in_proj: bool = True):
        super().__init__()
        if num_heads % num_qk_heads:
            raise ValueError("gated delta rule: value heads must be a multiple of q / k heads")
        if tp_group is not None and tp_group.size != 1:
            raise NotImplementedError("ragged gated-delta mixer: tensor parallel degree 1")
        self.nh, self.n_qk, self.D, self.Dv = num_heads, num_qk_heads, head_dim, v_head_dim
        self.taps, self.eps, self.layer_idx = conv_taps, eps, layer_idx
        self.Cqk, self.inner = num_qk_heads * head_dim, num_heads * v_head_dim
        self.conv_dim = 2 * self.Cqk + self.inner
        self.in_width = self.conv_dim + 2 * num_heads + self.inner
        self.in_proj = ColumnParallelLinear(hidden_size, self.in_width, bias=False, gather_output=False, dtype=dtype, device=device,
                                            tensor_model_parallel_group=tp_group) if own_in_proj else None
        self.out_proj = RowParallelLinear(self.inner, hidden_size, bias=False, input_is_parallel=True, dtype=dtype, device=device,
                                          tensor_model_parallel_group=tp_group)
        f32 = dict(dtype=torch.float32, device=device)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_dim, conv_taps, **f32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(v_head_dim, **f32), requires_grad=False)
        self.conv_state, self.delta_state = f"delta_conv{layer_idx}", f"delta_state{layer_idx}"

    def state_specs(self, cache_index=None):
        return {self.conv_state: (self.taps - 1, self.conv_dim), self.delta_state: ((self.nh, self.D, self.Dv), torch.float32)}

    def forward(self, x, meta, kv_mgr, cache_index=None):
        return self.forward_projected(self.in_proj(x), meta, kv_mgr, cache_index)

    def forward_projected(self, p, meta, kv_mgr, cache_index=None):
        ex = meta.extras
        ctx, qlen, lines = ex["ctx_len"], ex["q_len"], ex["state_lines"]
        Cd, H = self.conv_dim, self.nh
        u, beta, a, gate = p[..., :Cd], p[..., Cd:Cd + H], p[..., Cd + H:Cd + 2 * H], p[..., Cd + 2 * H:Cd + 2 * H + self.inner]
        states = kv_mgr.states
        cst, sst = states.tensor(self.conv_state), states.tensor(self.delta_state)
        qkv = ops.short_conv(u, self.conv_weight, None, cst, lines, ctx, qlen, silu=True)
        ops.short_conv_update(u, cst, lines, ctx, qlen)
        o = ops.gated_delta_scan(qkv, beta, a, self.A_log, self.dt_bias, sst, lines, ctx, qlen, H, self.n_qk, self.D, self.Dv, self.UNIT_EPS)
        return self.out_proj(ops.head_rmsnorm_gate(o, self.norm_weight, H, self.eps, gate, "silu", out_dtype=p.dtype))
