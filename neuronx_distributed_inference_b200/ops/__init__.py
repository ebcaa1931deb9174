"""Op dispatch: hand-written sm_100a kernels on CUDA tensors, PyTorch reference on CPU.

There is exactly one accelerated backend (the in-tree ``_C`` extension built from ``csrc/``);
there is no multi-backend layer.  A CUDA tensor with the extension missing is an error (set
``NXDI_B200_ALLOW_TORCH_FALLBACK=1`` to run the PyTorch definitions on GPU for debugging).
``stats`` counts kernel launches issued through this module (bench.py reports them).
"""
from __future__ import annotations

import os
from collections import Counter
from typing import Optional

import torch

from . import reference as ref
from ._ext import load_extension, extension_available

stats = Counter()
_ALLOW_FALLBACK = os.environ.get("NXDI_B200_ALLOW_TORCH_FALLBACK", "0") == "1"
GEMV_MAX_TOKENS = 8      # CUDA-core weight-streaming kernel up to here
_KERNELS_ENABLED = True
_TCGEN05_GEMM = os.environ.get("NXDI_B200_TCGEN05_GEMM", "1") == "1"   # 0: cuBLAS for T > 8 (A/B baseline)


def set_kernels_enabled(flag: bool):
    """Debug switch: run the PyTorch definitions on CUDA tensors (accuracy triage)."""
    global _KERNELS_ENABLED
    _KERNELS_ENABLED = flag


def _C():
    return load_extension()


def _use_cuda(x: torch.Tensor) -> bool:
    if not x.is_cuda or not _KERNELS_ENABLED:
        return False
    if extension_available():
        return True
    if _ALLOW_FALLBACK:
        return False
    raise RuntimeError("CUDA tensor but the sm_100a extension is not built: run "
                       "`python -c 'import __graft_entry__ as g; g.build()'` "
                       "(or set NXDI_B200_ALLOW_TORCH_FALLBACK=1)")


_FAST_DTYPES = (torch.bfloat16,)


# --------------------------------------------------------------------------------------------
def rmsnorm(x, weight, eps: float, offset: float = 0.0, residual=None):
    if _use_cuda(x) and x.dtype in _FAST_DTYPES and x.shape[-1] % 8 == 0 and weight is not None \
            and weight.dtype == x.dtype:
        stats["rmsnorm"] += 1
        x2 = x.reshape(-1, x.shape[-1]).contiguous()        # (a slice of a wider projection arrives strided)
        if residual is not None:
            r2 = residual.reshape(-1, x.shape[-1]).contiguous()
            y, r = _C().rmsnorm(x2, weight, eps, offset, r2)
            return y.view(x.shape), r.view(x.shape)
        y, _ = _C().rmsnorm(x2, weight, eps, offset, None)
        return y.view(x.shape)
    return ref.rmsnorm(x, weight, eps, offset, residual)


_ACT_CODES = {None: 0, "silu_mul": 1, "gelu_tanh_mul": 2, "gelu_mul": 3}


def staging_for(group, x, w):
    """Output tensor for a row-parallel GEMM inside the group's symmetric staging area (partial sums that an in-switch collective
    consumes next), or None when the group has no heap / the shape does not qualify."""
    heap = getattr(group, "heap", None)
    if heap is None or not x.is_cuda or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return None
    shape = tuple(x.shape[:-1]) + (w.shape[0],)
    T = x.numel() // x.shape[-1]
    if T <= GEMV_MAX_TOKENS or not heap.usable(torch.empty(0, dtype=torch.bfloat16, device=x.device), None, shape):
        return None
    return heap.staging(shape)


def linear(x, w, bias=None, norm_weight=None, norm_eps: float = 1e-6, norm_offset: float = 0.0,
           act: Optional[str] = None, scale=None, residual=None, out=None):
    """y = act(rmsnorm(x) @ w^T + bias) (+ residual).  w: [N,K] bf16, or int8/fp8 with per-channel ``scale``.
    ``out``: preallocated result (tcgen05 GEMM path only; used to land partial sums in the symmetric heap)."""
    if _use_cuda(x) and x.dtype in _FAST_DTYPES:
        K = x.shape[-1]
        T = x.numel() // K
        N = w.shape[0]
        wq = w.dtype in (torch.int8, torch.float8_e4m3fn)
        ok_w = (w.dtype == x.dtype and scale is None) or (wq and scale is not None and scale.dim() == 1)
        if ok_w and act in _ACT_CODES and w.is_contiguous():
            x2 = x.reshape(T, K)
            if wq and T <= GEMV_MAX_TOKENS and K % 16 == 0 and w.dim() == 2:
                stats["qgemv"] += 1
                r2 = residual.reshape(T, -1).contiguous() if (residual is not None and act is None) else None
                y = _C().gemv(x2, w, bias, norm_weight, norm_eps, norm_offset, _ACT_CODES[act], scale.float().contiguous(), r2)
                y = y.view(*x.shape[:-1], y.shape[-1])
                return y if (residual is None or r2 is not None) else y + residual
            if not wq and T <= GEMV_MAX_TOKENS and K % 64 == 0 and (K % 256 == 0 or _C().gemv2_supported(T, K)):
                stats["gemv"] += 1
                r2 = residual.reshape(T, -1) if (residual is not None and act is None) else None
                y = _C().gemv(x2, w, bias, norm_weight, norm_eps, norm_offset, _ACT_CODES[act], scale, r2)
                y = y.view(*x.shape[:-1], y.shape[-1])
                return y if (residual is None or r2 is not None) else y + residual
            n_out = N // 2 if act is not None else N
            if (wq and _ACT_QUANT and w.dtype == torch.float8_e4m3fn and T > GEMV_MAX_TOKENS and K % 128 == 0 and n_out % 8 == 0
                    and w.dim() == 2 and K <= 16384):
                # W8A8: RMSNorm + per-token fp8 quantisation in one kernel, then the fp8 tensor-core GEMM (2x the bf16 rate);
                # acc * a_scale[row] * w_scale[col] in the epilogue
                stats["gemm_fp8"] += 1
                xq, a_s = _C().rmsnorm_quant(x2.contiguous(), norm_weight, float(norm_eps), float(norm_offset), float("inf"))
                r2 = residual.reshape(T, -1).contiguous() if (residual is not None and act is None) else None
                y = _C().gemm_fp8(xq, a_s, w, scale.float().contiguous(), bias, _ACT_CODES[act], r2)
                y = y.view(*x.shape[:-1], y.shape[-1])
                return y if (residual is None or r2 is not None) else y + residual
            if (wq and T > GEMV_MAX_TOKENS and w.dim() == 2 and K % 64 == 0 and n_out % 8 == 0 and _TCGEN05_GEMM
                    and x.dtype == torch.bfloat16):
                # weight-only 8-bit prefill: one expansion pass into a shared bf16 scratch (stays in L2), then the bf16 tensor-core GEMM
                stats["dequant_gemm"] += 1
                w, scale, wq = _C().dequant_bf16(w, scale.float().contiguous(), _dequant_scratch(w)), None, False
            if not wq and n_out % 8 == 0 and K % 64 == 0 and _TCGEN05_GEMM and (T > GEMV_MAX_TOKENS or K % 64 != 0):
                if norm_weight is not None:
                    x2 = rmsnorm(x2, norm_weight, norm_eps, norm_offset)
                stats["gemm_tcgen05"] += 1
                r2 = residual.reshape(T, -1) if (residual is not None and act is None) else None
                o2 = out.view(T, -1) if out is not None else None
                y = _C().gemm(x2.contiguous(), w, bias, _ACT_CODES[act], r2, o2)
                y = out if out is not None else y.view(*x.shape[:-1], y.shape[-1])
                return y if (residual is None or r2 is not None) else y + residual
    y = ref.linear(x, w, bias, norm_weight, norm_eps, norm_offset, act, scale)
    y = y if residual is None else y + residual
    if out is not None:
        out.copy_(y)
        return out
    return y


_DEQ_SCRATCH = {}
_DEQ_RETIRED = []


def _dequant_scratch(w):
    """One bf16 scratch per device, grown to the largest 8-bit weight seen (consumed by the GEMM enqueued right after the expansion;
    stream order makes the reuse by the next layer safe)."""
    buf = _DEQ_SCRATCH.get(w.device)
    if buf is None or buf.numel() < w.numel():
        if buf is not None:
            _DEQ_RETIRED.append(buf)      # never freed: CUDA graphs captured with the smaller scratch still hold its address
        buf = torch.empty(w.numel(), dtype=torch.bfloat16, device=w.device)
        _DEQ_SCRATCH[w.device] = buf
    return buf


def linear_allreduce(x, w, bias, group, residual=None, reduce_dtype=None, scale=None):
    """Row-parallel GEMM -> all-reduce (+bias, +residual).  T <= 8 tokens on CUDA with a
    symmetric workspace attached to the group: ONE kernel (GEMV, P2P stores of partials into every
    peer, flag wait, reduce, residual add).  Otherwise GEMM then NCCL/gloo all-reduce."""
    from ..parallel import mappings
    K = x.shape[-1]
    T = x.numel() // K
    wq = w.dtype in (torch.int8, torch.float8_e4m3fn) and scale is not None and scale.dim() == 1 and w.dim() == 2
    if (_use_cuda(x) and x.dtype in _FAST_DTYPES and group.symm is not None and T <= GEMV_MAX_TOKENS
            and w.shape[0] <= group.symm.n_max
            and K % 64 == 0 and w.is_contiguous() and ((w.dtype == x.dtype and scale is None) or wq)
            and _C().gemv2_supported(T, K, (1 if w.dtype == torch.int8 else 2) if wq else 0)
            and reduce_dtype in (None, torch.float32)):
        stats["gemv_allreduce"] += 1
        y = group.symm.gemv_allreduce(x.reshape(T, K), w, bias, residual.reshape(T, -1) if residual is not None else None,
                                      scale.float().contiguous() if wq else None)
        return y.view(*x.shape[:-1], y.shape[-1])
    heap = getattr(group, "heap", None)
    if heap is not None and scale is None and reduce_dtype in (None, torch.float32, x.dtype) and T > GEMV_MAX_TOKENS \
            and heap.gemm_ar_usable(x, w):
        # prefill: tcgen05 GEMM -> per-tile hand-off -> in-switch reduce of the owned tiles -> multicast of the result, ONE kernel
        stats["gemm_all_reduce"] += 1
        y = heap.gemm_all_reduce(x.reshape(T, K), w, bias if group.rank == 0 else None, residual)
        return y.view(*x.shape[:-1], w.shape[0])
    if heap is not None and scale is None:
        # prefill: partial sums land in the symmetric staging area (bias on rank 0 only), one in-switch all-reduce adds the residual
        y = linear(x, w, bias if group.rank == 0 else None, out=staging_for(group, x, w))
        return mappings.all_reduce(y, group, reduce_dtype=reduce_dtype, residual=residual)
    y = linear(x, w, None, scale=scale)
    y = mappings.all_reduce(y, group, reduce_dtype=reduce_dtype)
    if bias is not None:
        y = y + bias
    if residual is not None:
        y = y + residual
    return y


def apply_rope(x, cos, sin, interleaved: bool = False):
    return ref.apply_rope(x, cos, sin, interleaved)


def rope_kv_append(qkv, cos, sin, k_cache, v_cache, seq_ids, positions, n_q, n_kv, head_dim,
                   interleaved: bool = False, q_norm=None, k_norm=None, norm_eps: float = 1e-6):
    """Split fused qkv [B,T,(n_q+2n_kv)*D], optional per-head q/k RMSNorm (Qwen3), RoPE on q,k,
    write k,v into the contiguous cache at (seq_ids[b], positions[b,t]).  Returns q [B,T,n_q,D].
    ONE kernel on CUDA (csrc/rope_kv.cu)."""
    B, T = positions.shape
    D = head_dim
    if (_use_cuda(qkv) and qkv.dtype in _FAST_DTYPES and k_cache.dtype == qkv.dtype and D in (64, 128, 256)
            and cos.shape[-1] * 2 == D and not interleaved):
        stats["rope_kv_append"] += 1
        return _C().rope_kv_append(qkv.reshape(B, T, -1), cos.contiguous(), sin.contiguous(), k_cache, v_cache,
                                   seq_ids.to(torch.int32), positions.to(torch.int32), n_q, n_kv, D,
                                   q_norm, k_norm, norm_eps)
    q, k, v = qkv.reshape(B, T, n_q + 2 * n_kv, D).split([n_q, n_kv, n_kv], dim=2)
    if q_norm is not None:
        q = ref.rmsnorm(q, q_norm, norm_eps)
        k = ref.rmsnorm(k, k_norm, norm_eps)
    q = ref.apply_rope(q, cos, sin, interleaved)
    k = ref.apply_rope(k, cos, sin, interleaved)
    kv_append(k_cache, v_cache, k, v, seq_ids, positions)
    return q


def rope_kv_split_append(qkv, cos, sin, k_cache, v_cache, seq_ids, positions, n_q, n_kv, head_dim, q_norm=None, k_norm=None,
                         norm_eps: float = 1e-6):
    """Prefill: split the fused QKV projection, per-head q/k RMSNorm, RoPE, cache write AND the contiguous rotated k / v of the new
    tokens for the flash kernel — ONE kernel (csrc/rope_kv.cu) instead of the split / rotate / cat / append chain.
    -> (q [B,T,n_q,D], k [B,T,n_kv,D], v [B,T,n_kv,D]) or None when the kernel does not apply."""
    B, T = positions.shape
    D = head_dim
    if (_use_cuda(qkv) and qkv.dtype == torch.bfloat16 and k_cache.dtype == qkv.dtype and D in (64, 128, 256) and cos is not None
            and cos.shape[-1] * 2 == D):
        stats["rope_kv_split_append"] += 1
        return _C().rope_kv_split_append(qkv.reshape(B, T, -1).contiguous(), cos.contiguous(), sin.contiguous(), k_cache, v_cache,
                                         seq_ids.to(torch.int32), positions.to(torch.int32).contiguous(), n_q, n_kv, D, q_norm, k_norm,
                                         norm_eps)
    return None


def kv_append(k_cache, v_cache, k_new, v_new, seq_ids, positions):
    if (_use_cuda(k_new) and k_new.dtype in _FAST_DTYPES and k_cache.dtype == k_new.dtype
            and (k_new.shape[-1] * k_new.element_size()) % 16 == 0 and v_new.shape[-1] == k_new.shape[-1]):
        stats["kv_append"] += 1
        _C().kv_append(k_cache, v_cache, k_new.contiguous(), v_new.contiguous(), seq_ids.to(torch.int32),
                       positions.to(torch.int32))
        return
    ref.kv_append(k_cache, v_cache, k_new, v_new, seq_ids, positions)


def attention_decode(q, k_cache, v_cache, seq_ids, positions, scale, window=None, chunk=None, sinks=None,
                     active_mask=None, softcap=None, k_scale=None, v_scale=None, seq_hint: int = 0, active_base=None):
    """``seq_hint``: upper bound on the live context (the TKG bucket) used only to size the split-KV grid."""
    D = q.shape[-1]
    if (_use_cuda(q) and q.dtype in _FAST_DTYPES and k_cache.dtype == q.dtype and D in (64, 128)
            and active_mask is None and chunk is None and softcap is None
            and q.shape[1] * (q.shape[2] // k_cache.shape[1]) <= 64):
        stats["attn_decode"] += 1
        return _C().attention_decode(q.contiguous(), k_cache, v_cache, seq_ids.to(torch.int32),
                                     positions.to(torch.int32).contiguous(), float(scale), int(window or 0), sinks,
                                     int(seq_hint))
    return ref.attention_decode(q, k_cache, v_cache, seq_ids, positions, scale, window, chunk, sinks,
                                active_mask, softcap, k_scale, v_scale, active_base)


def rope_attention_decode(qkv, cos, sin, k_cache, v_cache, seq_ids, write_positions, positions, n_q, n_kv, head_dim, scale,
                          window=None, sinks=None, q_norm=None, k_norm=None, norm_eps: float = 1e-6, seq_hint: int = 0):
    """Decode attention straight from the QKV projection: per-head q/k RMSNorm, RoPE, cache append and split-KV flash
    decode in ONE kernel (the append is the attention kernel's prologue).  qkv [B,T,(n_q+2n_kv)D] -> [B,T,n_q,D].
    Falls back to ``rope_kv_append`` + ``attention_decode`` where the fused kernel does not apply."""
    B, T = positions.shape
    D = head_dim
    if (_use_cuda(qkv) and qkv.dtype in _FAST_DTYPES and k_cache.dtype == qkv.dtype and D in (64, 128) and cos.shape[-1] * 2 == D
            and T * (n_q // n_kv) <= 64 and os.environ.get("NXDI_B200_FUSED_ROPE_ATTN", "1") != "0"):
        stats["rope_attn_decode"] += 1
        return _C().rope_attention_decode(qkv.reshape(B, T, -1), cos.contiguous(), sin.contiguous(), k_cache, v_cache,
                                          seq_ids.to(torch.int32), write_positions.to(torch.int32).contiguous(),
                                          positions.to(torch.int32).contiguous(), n_q, n_kv, D, float(scale), int(window or 0),
                                          sinks, q_norm, k_norm, norm_eps, int(seq_hint))
    q = rope_kv_append(qkv, cos, sin, k_cache, v_cache, seq_ids, write_positions, n_q, n_kv, D, False, q_norm, k_norm, norm_eps)
    return attention_decode(q, k_cache, v_cache, seq_ids, positions, scale, window, None, sinks, seq_hint=seq_hint)


_ATTN_TC = os.environ.get("NXDI_B200_ATTN_TC", "1") != "0"   # 0: the mma.sync flash kernel for head_dim 128 too (A/B baseline)


def attention_prefill(q, k, v, scale, causal: bool = True, window=None, chunk=None, key_valid=None,
                      q_pos=None, sinks=None, softcap=None):
    D = q.shape[-1]
    if (_use_cuda(q) and q.dtype in _FAST_DTYPES and D == 128 and _ATTN_TC and chunk is None and (causal or not window)
            and key_valid is None and q_pos is None and q.shape[1] == k.shape[1] and k.dtype == q.dtype):
        # Blackwell path: tcgen05 QK^T / PV with TMEM accumulators, TMA tiles (csrc/attention_tc.cu); soft-cap is an argument
        stats["attn_prefill_tc"] += 1
        return _C().attention_prefill_tc(q.contiguous(), k.contiguous(), v.contiguous(), float(scale), int(window or 0), sinks,
                                         bool(causal), float(softcap or 0.0))
    if (_use_cuda(q) and q.dtype in _FAST_DTYPES and D in (64, 128) and chunk is None and (causal or not window)
            and key_valid is None and q_pos is None and softcap is None and q.shape[1] == k.shape[1]):
        stats["attn_prefill"] += 1
        return _C().attention_prefill(q.contiguous(), k.contiguous(), v.contiguous(), float(scale),
                                      int(window or 0), sinks, bool(causal))
    return ref.attention_prefill(q, k, v, scale, causal, window, chunk, key_valid, q_pos, sinks, softcap)


def paged_kv_append(k_cache, v_cache, k_new, v_new, slot_mapping):
    if _use_cuda(k_new) and k_new.dtype in _FAST_DTYPES and k_cache.dtype == k_new.dtype:
        stats["paged_kv_append"] += 1
        _C().paged_kv_append(k_cache, v_cache, k_new.contiguous(), v_new.contiguous(),
                             slot_mapping.to(torch.int32).contiguous())
        return
    ref.paged_kv_append(k_cache, v_cache, k_new, v_new, slot_mapping)


def paged_attention_decode(q, k_cache, v_cache, block_table, positions, scale, window=None, sinks=None):
    D = q.shape[-1]
    if (_use_cuda(q) and q.dtype in _FAST_DTYPES and k_cache.dtype == q.dtype and D in (64, 128)
            and q.shape[1] * (q.shape[2] // k_cache.shape[2]) <= 64):
        stats["paged_attn_decode"] += 1
        return _C().paged_attention_decode(q.contiguous(), k_cache, v_cache, block_table.to(torch.int32).contiguous(),
                                           positions.to(torch.int32), float(scale), int(window or 0), sinks)
    return ref.paged_attention_decode(q, k_cache, v_cache, block_table, positions, scale, window, sinks)


def argmax(logits):
    if _use_cuda(logits) and logits.dim() == 2 and logits.dtype in (torch.float32, torch.bfloat16):
        stats["argmax"] += 1
        return _C().argmax(logits.contiguous(), [], None, 0, 0, 0, 0)
    return ref.argmax(logits)


def argmax_sharded(logits, group):
    """Arg-max over a vocabulary-sharded logits row block [B, V_local] -> GLOBAL token ids [B], ONE kernel: the per-rank
    winners are exchanged through the group's symmetric workspace inside the arg-max kernel (csrc/sampling.cu).  Returns None
    when the fused path does not apply (CPU, no workspace): the caller falls back to all-gather + glue."""
    symm = getattr(group, "symm", None)
    if (symm is None or not _use_cuda(logits) or logits.dim() != 2 or logits.dtype not in (torch.float32, torch.bfloat16)
            or logits.shape[0] > symm.ARGMAX_ROWS):
        return None
    stats["argmax_exchange"] += 1
    return symm.argmax(logits.contiguous())


def sample(logits, top_k, top_p, temperature, rand=None, global_topk: int = 256):
    if _use_cuda(logits) and logits.dim() == 2 and logits.dtype in (torch.float32, torch.bfloat16) \
            and global_topk <= 256:
        stats["topk_sample"] += 1
        B = logits.shape[0]
        if rand is None:
            rand = torch.full((B,), 0.5, device=logits.device)
        return _C().topk_sample(logits.contiguous(), top_k.to(torch.int32), top_p.float(), temperature.float(),
                                rand.float(), int(global_topk))
    return ref.sample(logits, top_k, top_p, temperature, rand, global_topk)


def moe_route(router_logits, top_k, act="softmax", normalize=True, act_over_topk=False, renorm_eps=None, correction=None, groups=None,
              scale=1.0):
    return ref.moe_route(router_logits, top_k, act, normalize, act_over_topk, renorm_eps, correction, groups, scale)


def router_topk(x, weight, top_k, act="softmax", normalize=True, act_over_topk=False, renorm_eps=None, correction=None, groups=None,
                scale=1.0):
    """fp32 router: ``logits = x W^T`` (W fp32), then :func:`moe_route`.  Sigmoid routers, and softmax routers that are not
    renormalised or that choose by corrected scores among kept groups, run as two kernels on CUDA (fp32 products with the rows in
    shared memory; scores, group limit, selection and scaling, one warp per token) instead of a cast, a library GEMM and a chain of
    elementwise / sort launches.  -> (logits, weights [N, k] fp32, expert ids [N, k])."""
    E = weight.shape[0]
    plain_softmax = act == "softmax" and (not normalize or correction is not None or groups is not None)
    if (_mix_cuda(x) and (act == "sigmoid" or plain_softmax) and not act_over_topk and weight.dtype == torch.float32 and x.dim() == 2
            and top_k <= E and E <= 512 and (groups is None or (E % int(groups[0]) == 0 and int(groups[1]) <= int(groups[0])))):
        stats["router_topk"] += 1
        count, keep = (int(groups[0]), int(groups[1])) if groups is not None else (1, 1)
        return _C().router_topk(x.contiguous(), weight.contiguous(), int(top_k), -1.0 if renorm_eps is None else float(renorm_eps),
                                act == "softmax", None if correction is None else correction.float().contiguous(), count, keep, float(scale))
    logits = torch.nn.functional.linear(x.float(), weight.float())
    w, idx = moe_route(logits, top_k, act, normalize, act_over_topk, renorm_eps, correction, groups, scale)
    return logits, w, idx


def identity_expert_add(y, x, topk_w, topk_i, num_experts: int):
    """``y + x * (sum of the weights of the slots routed to identity experts, ids >= num_experts)`` (definition: ops/reference.py)."""
    if _mix_cuda(y) and x.dtype == y.dtype and y.is_contiguous() and x.is_contiguous() and topk_i.shape[1] <= 64:
        stats["identity_expert_add"] += 1
        _C().identity_expert_add(y, x, topk_w.float().contiguous(), topk_i.to(torch.int32).contiguous(), int(num_experts))
        return y
    return ref.identity_expert_add(y, x, topk_w, topk_i, num_experts)


def moe_experts(x, w_gate_up, w_down, topk_w, topk_i, act="silu_mul", expert_offset=0,
                gate_up_bias=None, down_bias=None, act_fn=None, scale_input=False, gate_up_scale=None, down_scale=None):
    N = x.shape[0]
    if (act in _MOE_PLAIN_ACTS and _mix_cuda(x) and act_fn is None and gate_up_scale is None and down_scale is None and gate_up_bias is None
            and down_bias is None and not scale_input and w_gate_up.dtype == x.dtype and w_down.dtype == x.dtype and topk_i.dim() == 2
            and topk_i.shape[1] <= 64 and w_gate_up.shape[0] <= 512 and w_gate_up.is_contiguous() and w_down.is_contiguous()):
        # two-matrix experts ``down(act(up x))``: device-side permutation, grouped GEMMs with the activation in the first epilogue
        # (tcgen05 for bf16 shapes in multiples of 64, a tiled CUDA-core kernel for fp32 and every other shape), weighted combine
        stats["moe_plain"] += 1
        tc = _MOE_GROUPED and x.dtype == torch.bfloat16 and x.shape[1] % 64 == 0 and w_down.shape[2] % 64 == 0 and N > GEMV_MAX_TOKENS
        return _C().moe_plain(x.contiguous(), w_gate_up, w_down, topk_w.float().contiguous(), topk_i.to(torch.int32).contiguous(),
                              int(expert_offset), _MOE_PLAIN_ACTS[act], bool(tc), False)
    bf16_shapes = x.dtype == torch.bfloat16 and x.shape[1] % 64 == 0 and w_down.shape[2] % 64 == 0
    if (act == "silu_mul" and _mix_cuda(x) and not bf16_shapes and act_fn is None and gate_up_scale is None and down_scale is None
            and gate_up_bias is None and down_bias is None and not scale_input and w_gate_up.dtype == x.dtype and w_down.dtype == x.dtype
            and topk_i.dim() == 2 and topk_i.shape[1] <= 64 and w_gate_up.shape[0] <= 512 and w_gate_up.is_contiguous() and w_down.is_contiguous()):
        # gated experts in fp32 or with sizes the tensor-core kernels do not take: the same permutation around the CUDA-core grouped
        # GEMMs, the gate product as an elementwise pass between them
        stats["moe_plain_gated"] += 1
        return _C().moe_plain(x.contiguous(), w_gate_up, w_down, topk_w.float().contiguous(), topk_i.to(torch.int32).contiguous(),
                              int(expert_offset), _UNARY_ACTS["silu"], False, True)
    if gate_up_scale is not None or down_scale is not None:
        # fp8 experts with dynamic activation quantisation asked for: W8A8 grouped GEMMs on the kind::f8f6f4 tensor-core path
        if (_use_cuda(x) and _MOE_GROUPED and _ACT_QUANT and N > GEMV_MAX_TOKENS and x.dtype == torch.bfloat16 and act in _MOE_ACTS
                and w_gate_up.dtype == torch.float8_e4m3fn and w_down.dtype == torch.float8_e4m3fn and act_fn is None
                and gate_up_scale is not None and down_scale is not None and gate_up_scale.dim() == 2 and down_scale.dim() == 2
                and x.shape[1] % 128 == 0 and w_down.shape[2] % 128 == 0 and max(x.shape[1], w_down.shape[2]) <= 16384
                and topk_i.dim() == 2 and topk_i.shape[1] <= 64 and w_gate_up.shape[0] <= 512
                and (gate_up_bias is None or gate_up_bias.dtype == x.dtype) and (down_bias is None or down_bias.dtype == x.dtype)):
            stats["moe_grouped_fp8"] += 1
            return _C().moe_grouped(x.contiguous(), w_gate_up.contiguous(), w_down.contiguous(), topk_w.float().contiguous(),
                                    topk_i.to(torch.int32).contiguous(), int(expert_offset), _MOE_ACTS[act], bool(scale_input),
                                    None if gate_up_bias is None else gate_up_bias.contiguous(),
                                    None if down_bias is None else down_bias.contiguous(),
                                    gate_up_scale.float().contiguous(), down_scale.float().contiguous())
        # weight-only 8-bit experts: dequantise the selected experts on the fly
        return ref.moe_experts(x, w_gate_up, w_down, topk_w, topk_i, act, expert_offset, gate_up_bias, down_bias, act_fn, scale_input,
                               gate_up_scale, down_scale)
    # activations with a kernel implementation: the named GLU ones, or a callable that names its kernel twin (``kernel_act``)
    kact = act if act_fn is None else getattr(act_fn, "kernel_act", None)
    if (_use_cuda(x) and x.dtype in _FAST_DTYPES and w_gate_up.dtype == x.dtype and act == "silu_mul"
            and act_fn is None and gate_up_bias is None and down_bias is None and N <= GEMV_MAX_TOKENS and not scale_input
            and w_gate_up.is_contiguous() and w_down.is_contiguous() and topk_i.dim() == 2
            and x.shape[1] % 8 == 0 and w_down.shape[2] % 8 == 0 and max(x.shape[1], w_down.shape[2]) * 2 <= 65536):
        stats["moe_decode"] += 1
        return _C().moe_decode(x.contiguous(), w_gate_up, w_down, topk_w.float().contiguous(),
                               topk_i.to(torch.int32).contiguous(), int(expert_offset))
    # prefill-sized batches: device-side permutation + grouped tcgen05 GEMMs (static shapes: replays under CUDA graphs)
    if (_use_cuda(x) and _MOE_GROUPED and x.dtype == torch.bfloat16 and w_gate_up.dtype == x.dtype and w_down.dtype == x.dtype
            and kact in _MOE_ACTS and topk_i.dim() == 2 and topk_i.shape[1] <= 64
            and w_gate_up.is_contiguous() and w_down.is_contiguous() and x.shape[1] % 64 == 0 and w_down.shape[2] % 64 == 0
            and w_gate_up.shape[0] <= 512
            and (gate_up_bias is None or gate_up_bias.dtype == x.dtype) and (down_bias is None or down_bias.dtype == x.dtype)):
        stats["moe_grouped"] += 1
        return _C().moe_grouped(x.contiguous(), w_gate_up, w_down, topk_w.float().contiguous(), topk_i.to(torch.int32).contiguous(),
                                int(expert_offset), _MOE_ACTS[kact], bool(scale_input),
                                None if gate_up_bias is None else gate_up_bias.contiguous(),
                                None if down_bias is None else down_bias.contiguous(), None, None)
    return ref.moe_experts(x, w_gate_up, w_down, topk_w, topk_i, act, expert_offset, gate_up_bias, down_bias,
                           act_fn, scale_input)


_MOE_GROUPED = os.environ.get("NXDI_B200_MOE_GROUPED", "1") == "1"
_MOE_ACTS = {"silu_mul": 1, "gelu_tanh_mul": 2, "gelu_mul": 3, "gpt_oss_glu": 4}
_UNARY_ACTS = {"relu": 1, "relu2": 2, "silu": 3, "gelu_tanh": 4, "sigmoid": 5, "gelu": 6}         # codes of csrc/seqmix.cu (unary_act, moe_plain, gated_act_mul)
_MOE_PLAIN_ACTS = _UNARY_ACTS


def rmsnorm_quant(x, weight, eps, clamp=float("inf"), offset: float = 0.0):
    """(fp8-e4m3 activations, per-row fp32 scale): RMSNorm (``weight`` may be None) fused with dynamic per-token quantisation.
    ONE kernel on CUDA (csrc/quant.cu); reference kernel K6 (modeling_llama.py:553-575)."""
    if _use_cuda(x) and x.dtype in _FAST_DTYPES and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        stats["rmsnorm_quant"] += 1
        q, s = _C().rmsnorm_quant(x.reshape(-1, x.shape[-1]).contiguous(), weight, float(eps), float(offset), float(clamp))
        return q.view(x.shape), s.view(*x.shape[:-1], 1)
    return ref.rmsnorm_quant(x, weight, eps, clamp)


_ACT_QUANT = os.environ.get("NXDI_B200_FP8_ACT", "0") == "1"


def set_activation_quant(flag: bool):
    """W8A8: fp8 weights meet dynamically quantised fp8 activations on the tensor cores (tcgen05 kind::f8f6f4) for T > 8 tokens.
    Set from ``NeuronConfig.activation_quantization_type == "dynamic"`` / ``quantized_mlp_kernel_enabled``; off = weight-only."""
    global _ACT_QUANT
    _ACT_QUANT = bool(flag)


activation = ref.activation
build_mask = ref.build_mask
attention_with_mask = ref.attention_with_mask
quantize_per_channel = ref.quantize_per_channel
quantize_per_tensor = ref.quantize_per_tensor
quantize_blockwise = ref.quantize_blockwise


# ---- sequence mixers on ragged rows (csrc/seqmix.cu; definitions and conventions in ops/reference.py) ---------------------------
_MIX_DTYPES = (torch.bfloat16, torch.float32)
# launch limits of csrc/seqmix.cu (seqmix.h); shapes beyond them run the PyTorch definitions on the same device
_MIX_MAX_TAPS, _MIX_MAX_VDIM, _MIX_MAX_STATE = 8, 256, 256


def _mix_cuda(x) -> bool:
    return _use_cuda(x) and x.dtype in _MIX_DTYPES


def _i32(t):
    return t.to(torch.int32).contiguous()


def scaled_add_rmsnorm(x, y, weight, alpha: float, eps: float, offset: float = 0.0, lp_dtype=None):
    if _use_cuda(x) and x.dtype == torch.float32 and (y is None or y.dtype in _MIX_DTYPES):
        stats["scaled_add_rmsnorm"] += 1
        W = x.shape[-1]
        lp = lp_dtype if lp_dtype not in (None, torch.float32) else None
        out, out_lp = _C().scaled_add_rmsnorm(x.reshape(-1, W).contiguous(), None if y is None else y.reshape(-1, W).contiguous(),
                                              weight, float(alpha), float(eps), float(offset), lp == torch.bfloat16)
        return out.view(x.shape), (out_lp.view(x.shape) if lp is not None else None)
    return ref.scaled_add_rmsnorm(x, y, weight, alpha, eps, offset, lp_dtype)


def short_conv(u, weight, bias, state, slots, ctx_len, q_len, silu: bool = False):
    if _mix_cuda(u) and u.stride(-1) == 1 and weight.shape[1] <= _MIX_MAX_TAPS:
        stats["short_conv"] += 1
        return _C().short_conv(u, weight, bias, state, _i32(slots), _i32(ctx_len), _i32(q_len), bool(silu))
    return ref.short_conv(u, weight, bias, state, slots, ctx_len, q_len, silu)


def short_conv_update(u, state, slots, ctx_len, q_len):
    if _mix_cuda(u) and u.stride(-1) == 1 and state.shape[1] < _MIX_MAX_TAPS:
        stats["short_conv_update"] += 1
        return _C().short_conv_update(u, state, _i32(slots), _i32(ctx_len), _i32(q_len))
    return ref.short_conv_update(u, state, slots, ctx_len, q_len)


def conv_qknorm_rope_append(qkv, conv_w, state, slots, ctx_len, q_len, q_norm_w, k_norm_w, eps, n_q, n_kv, D, Dv, cos, sin,
                            k_cache, v_cache, block_table, out_dtype=None):
    if _mix_cuda(qkv) and qkv.stride(-1) == 1 and conv_w.shape[1] <= _MIX_MAX_TAPS and D % 2 == 0:
        stats["conv_qknorm_rope_append"] += 1
        return _C().conv_qknorm_rope_append(qkv, conv_w, state, _i32(slots), _i32(ctx_len), _i32(q_len), q_norm_w, k_norm_w, float(eps),
                                            int(n_q), int(n_kv), int(D), int(Dv), None if cos is None else cos.float().contiguous(),
                                            None if sin is None else sin.float().contiguous(),
                                            k_cache, v_cache, None if block_table is None else _i32(block_table))
    return ref.conv_qknorm_rope_append(qkv, conv_w, state, slots, ctx_len, q_len, q_norm_w, k_norm_w, eps, n_q, n_kv, D, Dv, cos, sin,
                                       k_cache, v_cache, block_table, out_dtype)


def paged_window_attention(q, k_cache, v_cache, block_table, ctx_len, q_len, scale, softcap, window, keep_first, gate=None, sinks=None,
                           gate_per_head: bool = False, chunk=None, slopes=None, value_dim=None, head_scale=None):
    Dv = v_cache.shape[-1] if value_dim is None else int(value_dim)
    if _mix_cuda(q) and k_cache.dtype == q.dtype and (gate is None or gate.stride(-1) == 1) and Dv <= _MIX_MAX_VDIM and not (chunk and window):
        stats["paged_window_attention"] += 1
        return _C().paged_window_attention(q.contiguous(), k_cache, v_cache, _i32(block_table), _i32(ctx_len), _i32(q_len), float(scale),
                                           float(softcap or 0.0), int(window or 0), int(keep_first or 0), gate,
                                           None if sinks is None else sinks.float().contiguous(), bool(gate_per_head), int(chunk or 0),
                                           None if slopes is None else slopes.float().contiguous(), Dv,
                                           None if head_scale is None else head_scale.float().contiguous())
    return ref.paged_window_attention(q, k_cache, v_cache, block_table, ctx_len, q_len, scale, softcap, window, keep_first, gate, sinks,
                                      gate_per_head, chunk, slopes, value_dim, head_scale)


def ssd_scan(xBC, dt_raw, z, A_log, dt_bias, D_skip, state, slots, ctx_len, q_len, n_heads, head_dim, n_state, n_groups):
    if (_use_cuda(xBC) and xBC.dtype == torch.float32 and dt_raw.dtype in _MIX_DTYPES and state.dtype == torch.float32
            and n_state <= _MIX_MAX_STATE):
        stats["ssd_scan"] += 1
        return _C().ssd_scan(xBC.contiguous(), dt_raw, z, A_log, dt_bias, D_skip, state, _i32(slots), _i32(ctx_len), _i32(q_len),
                             int(n_heads), int(head_dim), int(n_state), int(n_groups))
    return ref.ssd_scan(xBC, dt_raw, z, A_log, dt_bias, D_skip, state, slots, ctx_len, q_len, n_heads, head_dim, n_state, n_groups)


def group_rmsnorm(y, weight, groups: int, eps: float, out_dtype=None):
    od = out_dtype or y.dtype
    if _use_cuda(y) and y.dtype == torch.float32 and od in _MIX_DTYPES:
        stats["group_rmsnorm"] += 1
        W = y.shape[-1]
        return _C().group_rmsnorm(y.reshape(-1, W).contiguous(), weight, int(groups), float(eps), od == torch.bfloat16).view(y.shape)
    return ref.group_rmsnorm(y, weight, groups, eps, out_dtype)


def clamped_glu(gu, limit: float, alpha: float = 1.702):
    if _mix_cuda(gu):
        stats["clamped_glu"] += 1
        W = gu.shape[-1]
        return _C().clamped_glu(gu.reshape(-1, W).contiguous(), float(limit), float(alpha)).view(*gu.shape[:-1], W // 2)
    return ref.clamped_glu(gu, limit, alpha)


def stream_add_rmsnorm(x, adds=(), normed=None, normed_weight=None, vec=None, weight=None, eps: float = 1e-6, lp_dtype=None,
                       emit_stream_lp: bool = False):
    """fp32 residual stream update + the norm that reads it, ONE kernel (definition: ops/reference.py)."""
    adds = tuple(a for a in adds if a is not None)
    first = x if x is not None else (adds[0] if adds else normed)
    if (_use_cuda(first) and (x is None or x.dtype == torch.float32) and len(adds) <= 2 and all(a.dtype in _MIX_DTYPES for a in adds)
            and (normed is None or normed.dtype in _MIX_DTYPES) and len({a.dtype for a in adds + ((normed,) if normed is not None else ())}) <= 1):
        stats["stream_add_rmsnorm"] += 1
        W = first.shape[-1]
        lp = lp_dtype if lp_dtype not in (None, torch.float32) else None
        flat = lambda t: None if t is None else t.reshape(-1, W).contiguous()          # noqa: E731
        f32 = lambda t: None if t is None else t.float().contiguous()                  # noqa: E731
        s, s_lp, h = _C().stream_add_rmsnorm(flat(x), flat(adds[0]) if adds else None, flat(adds[1]) if len(adds) > 1 else None, flat(normed),
                                             f32(normed_weight), f32(vec), f32(weight), float(eps), lp == torch.bfloat16,
                                             bool(emit_stream_lp and lp is not None))
        shape = first.shape
        return s.view(shape), (None if s_lp is None else s_lp.view(shape)), (None if h is None else h.view(shape))
    return ref.stream_add_rmsnorm(x, adds, normed, normed_weight, vec, weight, eps, lp_dtype, emit_stream_lp)


def latent_norm_append(p, offset: int, rank: int, weight, eps: float, cache, block_table, ctx_len, q_len, emit_rows: bool = False,
                       rot_dim: int = 0, cos=None, sin=None, q_rank: int = 0, q_weight=None):
    """``emit_rows``: also return the cache rows in token order ``[B, T, 1, rank + rot_dim]`` (zeros past ``q_len``).  With ``q_rank``
    the result is ``(rows, normalised query latent [B, T, q_rank])``."""
    if _mix_cuda(p) and p.stride(-1) == 1 and cache.dtype == p.dtype and cache.is_contiguous() and rot_dim % 2 == 0:
        stats["latent_norm_append"] += 1
        f32 = lambda t: None if t is None else t.float().contiguous()          # noqa: E731
        rows, cq = _C().latent_norm_append(p, int(offset), int(rank), f32(weight), float(eps), cache, _i32(block_table),
                                           _i32(ctx_len), _i32(q_len), bool(emit_rows), int(rot_dim), f32(cos), f32(sin), int(q_rank), f32(q_weight))
        return (rows, cq) if q_rank else rows
    return ref.latent_norm_append(p, offset, rank, weight, eps, cache, block_table, ctx_len, q_len, emit_rows, rot_dim, cos, sin, q_rank,
                                  q_weight)


def rope_half_tail(src, dst, rot_dim: int, cos, sin):
    """Rotate-half rotation of the last ``rot_dim`` channels of every head of ``src`` into the last ``rot_dim`` channels of ``dst``."""
    if _mix_cuda(src) and dst.dtype == src.dtype and src.is_contiguous() and dst.is_contiguous() and rot_dim % 2 == 0:
        stats["rope_half_tail"] += 1
        _C().rope_half_tail(src, dst, int(rot_dim), cos.float().contiguous(), sin.float().contiguous())
        return dst
    return ref.rope_half_tail(src, dst, rot_dim, cos, sin)


def stream_norm_conv(x, adds, weight, conv_w, state, slots, ctx_len, q_len, eps: float, lp_dtype=None):
    """fp32 residual stream update + norm + short causal convolution of the normalised rows, ONE kernel (definition: ops/reference.py)."""
    adds = tuple(a for a in adds if a is not None)
    taps = 1 if conv_w is None else conv_w.shape[1]
    if (_use_cuda(x) and x.dtype == torch.float32 and len(adds) <= 2 and all(a.dtype in _MIX_DTYPES for a in adds) and taps <= _MIX_MAX_TAPS
            and x.dim() == 3 and (state is None or state.dtype == torch.float32)):
        stats["stream_norm_conv"] += 1
        lp = lp_dtype == torch.bfloat16
        a0, a1 = (adds + (None, None))[:2]
        c = lambda t: None if t is None else t.contiguous()          # noqa: E731
        return tuple(_C().stream_norm_conv(x.contiguous(), c(a0), c(a1), weight.float().contiguous(), None if conv_w is None else conv_w.float().contiguous(),
                                           state, None if slots is None else _i32(slots), _i32(ctx_len), _i32(q_len), float(eps), lp))
    return ref.stream_norm_conv(x, adds, weight, conv_w, state, slots, ctx_len, q_len, eps, lp_dtype)


def head_gate_mul(x, gate):
    """``x [B, T, H, D] * sigmoid(gate [B, T, H])`` per head, in fp32, result in the type of ``x`` (in place on CUDA)."""
    if _mix_cuda(x) and x.is_contiguous() and gate.dtype == x.dtype and gate.stride(-1) == 1 and (x.shape[-1] * x.element_size()) % 16 == 0 \
            and gate.stride(0) == gate.shape[1] * gate.stride(1):
        stats["head_gate_mul"] += 1
        _C().head_gate_mul(x, gate)
        return x
    return (x.float() * torch.sigmoid(gate.float()).unsqueeze(-1)).to(x.dtype)


def latent_prefill_on_tensor_cores(x, rank: int) -> bool:
    """Whole prompts (no row has earlier context) with 128-wide bf16 latent rows can use the contiguous-key tcgen05 flash kernel."""
    return _use_cuda(x) and x.dtype == torch.bfloat16 and rank == 128 and _ATTN_TC


def gated_act_mul(gate, other, act: str = "gelu_tanh", act_on_other: bool = False):
    if _mix_cuda(gate) and other.dtype == gate.dtype and other.stride(-1) == 1 and gate.is_contiguous() and act in _UNARY_ACTS \
            and other.dim() == gate.dim() and other.shape == gate.shape:
        stats["gated_act_mul"] += 1
        C = gate.shape[-1]
        o2 = other if other.dim() == 2 else other.reshape(-1, C) if other.is_contiguous() else _rows_view(other)
        return _C().gated_act_mul(gate.reshape(-1, C), o2, _UNARY_ACTS[act], bool(act_on_other)).view(gate.shape)
    return ref.gated_act_mul(gate, other, act, act_on_other)


def _rows_view(t):
    """[B, T, C] slice of a wider contiguous row -> [B * T, C] with the wide row stride (no copy)."""
    B, T, C = t.shape
    if t.stride(0) == T * t.stride(1):
        return t.as_strided((B * T, C), (t.stride(1), 1), t.storage_offset())
    return t.reshape(-1, C)


def unary_act(x, act: str):
    if _mix_cuda(x) and act in _UNARY_ACTS and x.is_contiguous():
        stats["unary_act"] += 1
        return _C().unary_act(x.reshape(-1, x.shape[-1]), _UNARY_ACTS[act]).view(x.shape)
    return ref.unary_act(x, act)


def stream_sandwich_norm(x, a=None, b=None, a_weight=None, b_weight=None, a_scale: float = 1.0, b_scale: float = 1.0, post_weight=None,
                         layer_scale=None, mult: float = 1.0, next_weight=None, eps: float = 1e-6, center: bool = True, lp_dtype=None):
    """Stream update of a block normalised on both sides of its sublayers + the norm the next sublayer reads, ONE kernel (definition:
    ops/reference.py)."""
    ys = tuple(t for t in (a, b) if t is not None)
    if (_use_cuda(x) and x.dtype == torch.float32 and all(t.dtype in _MIX_DTYPES for t in ys) and len({t.dtype for t in ys}) <= 1
            and x.shape[-1] <= 51200 and not (a is None and b is not None)):
        stats["stream_sandwich_norm"] += 1
        W = x.shape[-1]
        flat = lambda t: None if t is None else t.reshape(-1, W).contiguous()          # noqa: E731
        f32 = lambda t: None if t is None else t.float().contiguous()                  # noqa: E731
        s, h = _C().stream_sandwich_norm(flat(x), flat(a), flat(b), f32(a_weight), f32(b_weight), float(a_scale), float(b_scale),
                                         f32(post_weight), f32(layer_scale), float(mult), f32(next_weight), float(eps), bool(center),
                                         lp_dtype == torch.bfloat16)
        return s.view(x.shape), (None if h is None else h.view(x.shape))
    return ref.stream_sandwich_norm(x, a, b, a_weight, b_weight, a_scale, b_scale, post_weight, layer_scale, mult, next_weight, eps, center,
                                    lp_dtype)


def head_norm_rope_append(p, n_q, n_kv, D, Dv, cos, sin, q_norm_w, k_norm_w, norm_at: int, eps: float, value_from_key: bool, k_cache, v_cache,
                          block_table, ctx_len, q_len, out_dtype=None):
    """Per-head q / k RMS norm (before or after the rotation) + rotate-half rotation + paged cache write, ONE kernel (definition:
    ops/reference.py)."""
    if _mix_cuda(p) and p.stride(-1) == 1 and D <= 256 and k_cache.dtype == p.dtype and v_cache.dtype == p.dtype and (cos is None or cos.shape[-1] * 2 <= D):
        stats["head_norm_rope_append"] += 1
        f32 = lambda t: None if t is None else t.float().contiguous()          # noqa: E731
        return _C().head_norm_rope_append(p, int(n_q), int(n_kv), int(D), int(Dv), f32(cos), f32(sin), f32(q_norm_w), f32(k_norm_w), int(norm_at),
                                          float(eps), bool(value_from_key), k_cache, v_cache, _i32(block_table), _i32(ctx_len), _i32(q_len))
    return ref.head_norm_rope_append(p, n_q, n_kv, D, Dv, cos, sin, q_norm_w, k_norm_w, norm_at, eps, value_from_key, k_cache, v_cache,
                                     block_table, ctx_len, q_len, out_dtype)


def gated_delta_scan(qkv, beta_raw, a_raw, A_log, dt_bias, state, slots, ctx_len, q_len, n_heads, n_qk, D, Dv, unit_eps: float = 1e-6):
    if (_use_cuda(qkv) and qkv.dtype == torch.float32 and beta_raw.dtype in _MIX_DTYPES and a_raw.dtype == beta_raw.dtype
            and state.dtype == torch.float32 and D <= 256 and beta_raw.stride(-1) == 1 and a_raw.stride(-1) == 1):
        stats["gated_delta_scan"] += 1
        return _C().gated_delta_scan(qkv.contiguous(), beta_raw, a_raw, A_log, dt_bias, state, _i32(slots), _i32(ctx_len), _i32(q_len),
                                     int(n_heads), int(n_qk), int(D), int(Dv), float(unit_eps))
    return ref.gated_delta_scan(qkv, beta_raw, a_raw, A_log, dt_bias, state, slots, ctx_len, q_len, n_heads, n_qk, D, Dv, unit_eps)


def head_rmsnorm_gate(y, weight, heads: int, eps: float, gate, act: str = "silu", out_dtype=None):
    od = out_dtype or y.dtype
    C = y.shape[-1]
    if (_use_cuda(y) and y.dtype == torch.float32 and od in _MIX_DTYPES and gate.dtype in _MIX_DTYPES and gate.stride(-1) == 1 and act in _UNARY_ACTS
            and C // heads <= _MIX_MAX_VDIM and gate.shape == y.shape):
        stats["head_rmsnorm_gate"] += 1
        g2 = gate if gate.dim() == 2 else (gate.reshape(-1, C) if gate.is_contiguous() else _rows_view(gate))
        return _C().head_rmsnorm_gate(y.reshape(-1, C).contiguous(), weight.float().contiguous(), int(heads), float(eps), g2, _UNARY_ACTS[act],
                                      od == torch.bfloat16).view(y.shape)
    return ref.head_rmsnorm_gate(y, weight, heads, eps, gate, act, out_dtype)
