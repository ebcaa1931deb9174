"""Prefill / decode throughput of the Tusipel stack (pre-norm blocks over a convolved normalised stream; latent attention with a rotated
shared key part and a window; chunked grouped-query attention over convolved projections with a distance term; dense and
group-routed feed-forwards with identity experts) beside the closest stack on the same engine — Sodudra: latent attention and routed
experts on the same paged cache and scheduler — at equal layer sizes, random weights, plus a per-kernel table: every kernel the stack
added or extended, timed alone (CUDA events, L2 flushed between iterations) with its algorithmic bytes or FLOPs as a fraction of the
measured copy bandwidth / bf16 GEMM rate, next to the like kernel of the engine's other stacks.  Run through ``bench.py --config tusipel``."""
from __future__ import annotations

import json
import os
import tempfile

import torch

from .benchmark_latent_moe import SIZES as LATENT_SIZES
from .benchmark_latent_moe import _time, build_sodudra

SIZES = {
    # the latent / expert sizes of the Sodudra benchmark plus what only this stack has
    "small": dict(LATENT_SIZES["small"], rot=64, q_rank=512, window=256, kv_heads=4, conv=4, chunk=512, taps=4, dense_ff=4096, identity=4, groups=(4, 2)),
    "large": dict(LATENT_SIZES["large"], rot=64, q_rank=1024, window=256, kv_heads=8, conv=4, chunk=512, taps=4, dense_ff=8192, identity=8, groups=(8, 4)),
}
LAYERS = 4
VOCAB = 32000


def tusipel_config(s):
    lat = dict(heads=s["heads"], dim=s["dim"], rot_dim=s["rot"], vdim=s["vdim"], kv_rank=s["rank"], q_rank=s["q_rank"], scale=(s["dim"] + s["rot"]) ** -0.5,
               mask=dict(size=s["window"]), rot=dict(base=10000.0, dims=s["rot"], scaling=dict(factor=4.0, original=4096, fast=32.0, slow=1.0)))
    att = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["vdim"], conv=s["conv"], scale=s["dim"] ** -0.5, mask=dict(size=s["chunk"]))
    dense = dict(kind="dense", ff=s["dense_ff"], limit=7.0)
    moe = dict(kind="moe", expert=dict(ff=s["ff"]), router=dict(experts=s["experts"], identity=s["identity"], top=s["top"], scale=2.0,
                                                                 groups=dict(count=s["groups"][0], keep=s["groups"][1])))
    layers = [dict(type="latent_attention", mixer=lat, mlp=dense), dict(type="attention", mixer=att, mlp=moe),
              dict(type="attention", mixer=att, mlp=dense), dict(type="latent_attention", mixer=lat, mlp=moe)]
    return dict(architecture="Tusipel", layers=layers, norm=dict(eps=1e-5), vocab=VOCAB, width=s["width"], canon=dict(taps=s["taps"]),
                embedding=dict(scale=1.0), loop=dict(start=1, stop=3, times=1))


def build_tusipel(s, batch, max_tokens):
    from ..config import NeuronConfig, OnDeviceSamplingConfig
    from ..models.tusipel.modeling_tusipel import NeuronTusipelForCausalLM, TusipelInferenceConfig
    from ..runtime.scheduler import PagedBatchEngine
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(tusipel_config(s), f)
    page = 64
    ladder = [b for b in (64, 256, 1024, 4096) if b < max_tokens] + [max_tokens]
    nc = NeuronConfig(batch_size=batch, ctx_batch_size=batch, tkg_batch_size=batch, max_batch_size=batch, kv_cache_batch_size=batch,
                      seq_len=max_tokens, max_context_length=max_tokens, torch_dtype="bfloat16", is_block_kv_layout=True, pa_block_size=page,
                      pa_num_blocks=batch * (-(-max_tokens // page)), enable_bucketing=True, context_encoding_buckets=ladder,
                      is_continuous_batching=True, on_device_sampling_config=OnDeviceSamplingConfig(top_k=1), skip_warmup=True)
    app = NeuronTusipelForCausalLM(d, TusipelInferenceConfig.from_pretrained(d, nc))
    app.load(None, skip_warmup=True, random_weights=True)
    return PagedBatchEngine(app)


def model_numbers(size, batch, prompt, decode_steps, warmup):
    """tokens/s of one prefill step (batch rows x prompt tokens, host-resident ids in, tokens out) and of decode steps at that context,
    through the engine's step call, for both stacks."""
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, VOCAB, (batch, prompt), generator=g)
    out = {}
    for name, build, s in (("tusipel", build_tusipel, SIZES[size]), ("sodudra", build_sodudra, LATENT_SIZES[size])):
        eng = build(s, batch, prompt + decode_steps + warmup + 64)

        def f_prefill():
            for b in range(batch):
                eng.release(b)
            return eng.step([(b, ids[b].tolist(), ()) for b in range(batch)], sample=True)
        ms = _time(f_prefill, n=3, warm=max(1, min(warmup, 2)))
        out[f"{name}_prefill_tok_s"] = batch * prompt * 1e3 / ms
        tok = f_prefill()

        def f_decode(n):
            nonlocal tok
            for _ in range(n):
                tok = eng.step([(b, [tok[b]], ()) for b in range(batch)], sample=True)
        f_decode(warmup)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        f_decode(decode_steps)
        e1.record()
        torch.cuda.synchronize()
        out[f"{name}_decode_tok_s"] = batch * decode_steps * 1e3 / e0.elapsed_time(e1)
        out[f"{name}_decode_ms_per_step"] = e0.elapsed_time(e1) / decode_steps
        del eng
        torch.cuda.empty_cache()
    return out


def kernel_table(size, batch, prompt, hbm_gbs, tflops):
    """Each kernel alone at the layer's shapes: name, ms, algorithmic GB and GFLOP, the fraction of the measured copy bandwidth and of
    the measured bf16 GEMM rate; prefill (batch x prompt tokens) and decode (batch x 1 token at context ``prompt``); after every new
    or extended kernel the like kernel of another stack on the same shapes."""
    from .. import ops
    from ..ops import reference as ref
    s = SIZES[size]
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def run(name, fn, nbytes, flops=0.0, n=5):
        best = float("inf")
        for i in range(n + 2):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                best = min(best, e0.elapsed_time(e1))
        rows.append(dict(kernel=name, ms=round(best, 4), gb=round(nbytes / 1e9, 4), frac_of_measured_hbm=round(nbytes / 1e6 / best / hbm_gbs, 3),
                         tflops=round(flops / 1e9 / best, 1), frac_of_measured_bf16=round(flops / 1e9 / best / tflops, 3)))

    W, H, G, D, Dv, R, rot, Q = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["rank"], s["rot"], s["q_rank"]
    E, ident, k, F, page, K = s["experts"], s["identity"], s["top"], s["ff"], 64, s["taps"]
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=dev, dtype=dt)          # noqa: E731
    for phase, T, ctx0 in (("prefill", prompt, 0), ("decode", 1, prompt)):
        B = batch
        N = B * T
        ctx = torch.full((B,), ctx0, dtype=torch.int32, device=dev)
        ql = torch.full((B,), T, dtype=torch.int32, device=dev)
        lines = torch.arange(B, dtype=torch.int32, device=dev)
        nblk = -(-(ctx0 + T) // page)
        table = torch.arange(B * nblk, dtype=torch.int32, device=dev).view(B, nblk)
        keys = ctx0 + T
        # ---- stream: sum + norm + convolution -----------------------------------------------------------------------------------
        x32, y1 = rnd(B, T, W, dt=torch.float32), rnd(B, T, W)
        wn, cw, st = rnd(W, dt=torch.float32), rnd(W, K, dt=torch.float32), rnd(B + 1, K - 1, W, dt=torch.float32)
        run(f"{phase}: stream_norm_conv (x + y -> stream, norm, {K}-tap convolution, bf16 rows)",
            lambda: ops.stream_norm_conv(x32, (y1,), wn, cw, st, lines, ctx, ql, 1e-5, bf), N * W * (4 + 2 + 4 + 2))
        run(f"{phase}: short_conv_update (carried stream rows)", lambda: ops.short_conv_update(x32, st, lines, ctx, ql), B * (K - 1) * W * 4 * 2)
        x2, y2 = x32.view(N, W), y1.view(N, W)
        run(f"{phase}: like: stream_add_rmsnorm (x + y -> stream, norm, no convolution)",
            lambda: ops.stream_add_rmsnorm(x2, (y2,), weight=wn, eps=1e-5, lp_dtype=bf), N * W * (4 + 2 + 4 + 2))
        # ---- latent mixer ------------------------------------------------------------------------------------------------------
        C = Q + R + rot + H * Dv
        p = rnd(B, T, C)
        cache = rnd(B * nblk, page, 1, R + rot)
        lw, qw = torch.ones(R, device=dev), torch.ones(Q, device=dev)
        cos, sin = rnd(B, T, rot // 2, dt=torch.float32), rnd(B, T, rot // 2, dt=torch.float32)
        run(f"{phase}: latent_norm_append (latent norm, rotated key part, query latent norm)",
            lambda: ops.latent_norm_append(p, Q, R, lw, 1e-5, cache, table, ctx, ql, False, rot, cos, sin, Q, qw), N * (2 * (R + rot) + 2 * Q) * 2)
        c0 = rnd(B * nblk, page, 1, R)
        run(f"{phase}: like: latent_norm_append (latent norm only)", lambda: ops.latent_norm_append(p, Q, R, lw, 1e-5, c0, table, ctx, ql), N * R * 2 * 2)
        qf, a = rnd(B, T, H, D + rot), rnd(B, T, H, R + rot) * 0.2
        run(f"{phase}: rope_half_tail (rotated query channels behind the absorbed ones)", lambda: ops.rope_half_tail(qf, a, rot, cos, sin), N * H * rot * 2 * 2)
        win = min(s["window"], keys)
        lat_flops = 2.0 * B * H * (2 * R + rot) * sum(min(t + 1 + ctx0, s["window"]) for t in range(T))
        run(f"{phase}: paged_window_attention (latent rows + rotated tail as keys, prefix as values, window {s['window']})",
            lambda: ops.paged_window_attention(a, cache, cache, table, ctx, ql, 0.1, None, s["window"], 0, value_dim=R),
            B * min(keys, T + win) * (R + rot) * 2 + N * H * (2 * R + rot) * 2, lat_flops)
        a0 = rnd(B, T, H, R) * 0.2
        run(f"{phase}: like: paged_window_attention (latent rows as keys and values, same window)",
            lambda: ops.paged_window_attention(a0, c0, c0, table, ctx, ql, 0.1, None, s["window"], 0),
            B * min(keys, T + win) * R * 2 + N * H * R * 2 * 2, lat_flops * 2 * R / (2 * R + rot))
        o, gate = rnd(B, T, H * Dv), p[..., Q + R + rot:]
        run(f"{phase}: gated_act_mul (sigmoid of the strided gate slice, per channel)", lambda: ops.gated_act_mul(o, gate, "sigmoid", act_on_other=True),
            N * H * Dv * 2 * 3)
        o4, hg = rnd(B, T, H, Dv), rnd(B, T, H)
        run(f"{phase}: like: head_gate_mul (one gate per head)", lambda: ops.head_gate_mul(o4, hg), N * H * Dv * 2 * 2)
        # ---- attention mixer ---------------------------------------------------------------------------------------------------
        Cq = H * D + G * (D + Dv)
        pr = rnd(B, T, Cq)
        kc, vc = rnd(B * nblk, page, G, D), rnd(B * nblk, page, G, Dv)
        cwq, stq = rnd(Cq, s["conv"], dt=torch.float32), rnd(B + 1, s["conv"] - 1, Cq)
        run(f"{phase}: conv_qknorm_rope_append (convolution + cache write, no norms, no rotation)",
            lambda: ops.conv_qknorm_rope_append(pr, cwq, stq, lines, ctx, ql, None, None, 1e-5, H, G, D, Dv, None, None, kc, vc, table), N * Cq * 2 * 2)
        qn, kn = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
        cs2, sn2 = rnd(B, T, D // 4, dt=torch.float32), rnd(B, T, D // 4, dt=torch.float32)
        run(f"{phase}: like: conv_qknorm_rope_append (with row norms and rotation)",
            lambda: ops.conv_qknorm_rope_append(pr, cwq, stq, lines, ctx, ql, qn, kn, 1e-5, H, G, D, Dv, cs2, sn2, kc, vc, table), N * Cq * 2 * 2)
        qa = rnd(B, T, H, D) * 0.2
        sl = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
        ch = s["chunk"]
        seen = sum((t + ctx0) % ch + 1 for t in range(T))
        att_flops = 2.0 * B * H * (D + Dv) * seen
        att_bytes = B * min(keys, T + ch) * G * (D + Dv) * 2 + N * H * (D + Dv) * 2
        run(f"{phase}: paged_window_attention (grouped kv heads, chunks of {ch}, distance slopes)",
            lambda: ops.paged_window_attention(qa, kc, vc, table, ctx, ql, 0.1, None, None, 0, chunk=ch, slopes=sl), att_bytes, att_flops)
        run(f"{phase}: like: paged_window_attention (grouped kv heads, window {ch}, no slopes)",
            lambda: ops.paged_window_attention(qa, kc, vc, table, ctx, ql, 0.1, None, ch, 0), att_bytes,
            2.0 * B * H * (D + Dv) * sum(min(t + 1 + ctx0, ch) for t in range(T)))
        # ---- feed-forwards -----------------------------------------------------------------------------------------------------
        x = rnd(N, W)
        wr, corr = rnd(E + ident, W, dt=torch.float32) * W ** -0.5, rnd(E + ident, dt=torch.float32) * 0.05
        run(f"{phase}: router_topk (softmax, corrected choice among {s['groups'][1]} of {s['groups'][0]} groups, scaled)",
            lambda: ops.router_topk(x, wr, k, "softmax", False, False, None, corr, s["groups"], 2.0), N * W * 2 + (E + ident) * W * 4, 2.0 * N * (E + ident) * W)
        run(f"{phase}: like: router_topk (sigmoid, renormalised)", lambda: ops.router_topk(x, wr, k, "sigmoid", True, False, 1e-20),
            N * W * 2 + (E + ident) * W * 4, 2.0 * N * (E + ident) * W)
        tw, ti = ref.moe_route(rnd(N, E + ident, dt=torch.float32), k, "softmax", False, False, None, corr, s["groups"], 2.0)
        ti = ti.to(torch.int32)
        w_gu, w_dn = rnd(E, 2 * F, W) * W ** -0.5, rnd(E, W, F) * F ** -0.5
        w_up = rnd(E, F, W) * W ** -0.5
        used = min(E, N * k)
        real = float((ti < E).sum()) / max(1, N)
        run(f"{phase}: moe experts, gated SiLU (ids past the experts skipped)", lambda: ops.moe_experts(x, w_gu, w_dn, tw, ti, "silu_mul"),
            used * 3 * F * W * 2 + N * W * 2 * 2, 6.0 * N * real * F * W)
        y = rnd(N, W)
        run(f"{phase}: identity_expert_add", lambda: ops.identity_expert_add(y, x, tw, ti, E), N * W * 2 * 3)
        run(f"{phase}: like: moe experts, two matrices, squared ReLU", lambda: ops.moe_experts(x, w_up, w_dn, tw, ti, "relu2"),
            used * 2 * F * W * 2 + N * W * 2 * 2, 4.0 * N * real * F * W)
        gu = rnd(N, 2 * s["dense_ff"])
        run(f"{phase}: clamped_glu (dense feed-forward; the post-norm stack's kernel)", lambda: ops.clamped_glu(gu, 7.0), N * s["dense_ff"] * 2 * 3)
    return rows


def run(size="small", batch=4, prompt=1024, decode_steps=32, warmup=3):
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            peaks = json.load(f)
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    tf = float(peaks.get("bf16_tflops", 1590.0))
    res = dict(size=size, shapes={k: (list(v) if isinstance(v, tuple) else v) for k, v in SIZES[size].items()}, layers=LAYERS, batch=batch, prompt=prompt,
               decode_steps=decode_steps, hbm_gbs=hbm, bf16_tflops=tf, peaks_source="measured" if peaks else "fallback")
    res.update(model_numbers(size, batch, prompt, decode_steps, warmup))
    res["kernels"] = kernel_table(size, batch, prompt, hbm, tf)
    return res
