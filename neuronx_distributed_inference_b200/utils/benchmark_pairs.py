"""Prefill / decode throughput of the Zanivik stack beside the closest stack on the same engine (Fetodra: attention and Mamba-2 layers
one after the other, each sublayer between a sum and a norm) at equal layer sizes, random weights, plus a per-kernel table: every
kernel the new stack adds or extends timed alone (CUDA events, L2 flushed between iterations) with its algorithmic bytes as a fraction of
the measured copy bandwidth, next to the like kernel of the closest stack.  Run through ``bench.py --config zanivik``.

Equal sizes: a Zanivik block holds an attention layer AND a recurrent layer, so two Zanivik blocks (one of each pair type) stand beside
four Fetodra layers (attention, Mamba-2, attention, Mamba-2; feed-forwards after the attention layers only); the two-matrix feed-forward
is 1.5 x as wide as the three-matrix one, which gives both stacks the same number of weights per feed-forward."""
from __future__ import annotations

import json
import os
import tempfile

import torch

SIZES = {
    # width, q / kv heads x head size, window, three-matrix ff, Mamba-2 heads x head size, state, groups, delta heads / qk heads x sizes
    "small": dict(width=2048, heads=16, kv_heads=4, dim=128, window=512, ff=8192, m_heads=64, m_dim=64, state=128, groups=1,
                  d_heads=16, d_qk=8, d_dim=128, d_vdim=128),
    "large": dict(width=4096, heads=32, kv_heads=8, dim=128, window=512, ff=14336, m_heads=128, m_dim=64, state=128, groups=8,
                  d_heads=32, d_qk=16, d_dim=128, d_vdim=128),
}
VOCAB = 32000


def zanivik_config(s):
    rot = dict(base=1e6, dims=s["dim"])
    left = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["dim"], scale=s["dim"] ** -0.5, mask=dict(size=s["window"]))
    mlp = dict(kind="dense", ff=s["ff"] * 3 // 2)
    a = dict(type="parallel", mlp=mlp, mixer=dict(
        left=dict(left, rot=dict(rot, scaling=dict(factor=16.0, low=2.0, high=8.0, original=4096))), left_scale=0.8, right_scale=0.6,
        right=dict(heads=s["d_heads"], kv_heads=s["d_qk"], dim=s["d_dim"], vdim=s["d_vdim"], conv=4)))
    b = dict(type="parallel_2", mlp=mlp, mixer=dict(
        left=dict(left, rot=rot), right=dict(heads=s["m_heads"], vdim=s["m_dim"], state=s["state"], groups=s["groups"], norm_groups=1, conv=4)))
    return dict(architecture="Zanivik", layers=[a, b], norm=dict(eps=1e-6), residual_mult=0.7, vocab=VOCAB, width=s["width"])


def fetodra_config(s):
    att = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["dim"], conv=4, rot=dict(dims=s["dim"] // 2, base=1e6),
               scale=s["dim"] ** -0.5, softcap=30.0, mask=dict(size=s["window"], keep_first=4))
    mam = dict(heads=s["m_heads"], vdim=s["m_dim"], state=s["state"], groups=s["groups"], norm_groups=1, conv=4)
    mlp = dict(kind="dense", ff=s["ff"], limit=7.0)
    layers = [dict(type="attention", mixer=att, mlp=mlp), dict(type="mamba2", mixer=mam, mlp=None)] * 2
    return dict(architecture="Fetodra", layers=layers, norm=dict(eps=1e-5), postln_alpha=1.0, vocab=VOCAB, width=s["width"])


def build(cfg, batch, max_tokens):
    from ..config import NeuronConfig, OnDeviceSamplingConfig
    from ..runtime.scheduler import PagedBatchEngine
    from .constants import ARCHITECTURES, get_model_cls
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    page = 64
    ladder = [b for b in (64, 256, 1024, 4096) if b < max_tokens] + [max_tokens]
    nc = NeuronConfig(batch_size=batch, ctx_batch_size=batch, tkg_batch_size=batch, max_batch_size=batch, kv_cache_batch_size=batch,
                      seq_len=max_tokens, max_context_length=max_tokens, torch_dtype="bfloat16", is_block_kv_layout=True, pa_block_size=page,
                      pa_num_blocks=batch * (-(-max_tokens // page)), enable_bucketing=True, context_encoding_buckets=ladder,
                      is_continuous_batching=True, on_device_sampling_config=OnDeviceSamplingConfig(top_k=1), skip_warmup=True)
    cls = get_model_cls(ARCHITECTURES[cfg["architecture"]])
    app = cls.from_pretrained(d, nc)
    app.load(None, skip_warmup=True, random_weights=True)
    return PagedBatchEngine(app)


def _time(fn, n=3, warm=1):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def model_numbers(size, batch, prompt, decode_steps, warmup):
    """tokens/s of one prefill step (batch rows x prompt tokens, host-resident ids in, tokens out) and of decode steps at that context,
    both stacks through ``PagedBatchEngine.step``."""
    s = SIZES[size]
    ids = torch.randint(0, VOCAB, (batch, prompt), generator=torch.Generator().manual_seed(0))
    out = {}
    for name, cfg in (("zanivik", zanivik_config(s)), ("fetodra", fetodra_config(s))):
        eng = build(cfg, batch, prompt + decode_steps + warmup + 64)

        def prefill():
            for b in range(batch):
                eng.release(b)
            return eng.step([(b, ids[b].tolist(), ()) for b in range(batch)], sample=True)
        ms = _time(prefill, n=3, warm=max(1, min(warmup, 2)))
        out[f"{name}_prefill_tok_s"] = batch * prompt * 1e3 / ms
        tok = prefill()

        def decode(n):
            nonlocal tok
            for _ in range(n):
                tok = eng.step([(b, [tok[b]], ()) for b in range(batch)], sample=True)
        decode(warmup)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        decode(decode_steps)
        e1.record()
        torch.cuda.synchronize()
        out[f"{name}_decode_tok_s"] = batch * decode_steps * 1e3 / e0.elapsed_time(e1)
        out[f"{name}_decode_ms_per_step"] = e0.elapsed_time(e1) / decode_steps
        out[f"{name}_weights_gb"] = sum(p.numel() * p.element_size() for p in eng.app.parameters()) / 1e9 if hasattr(eng.app, "parameters") else None
        del eng
        torch.cuda.empty_cache()
    return out


def kernel_table(size, batch, prompt, hbm_gbs):
    """[name, ms, GB moved (algorithmic), fraction of the measured copy bandwidth] of every kernel the stack adds or extends, followed by
    the like kernel of the Fetodra stack on the same shapes; prefill (batch x prompt tokens) and decode (batch x 1 token at context ``prompt``)."""
    from .. import ops
    s = SIZES[size]
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def run(name, fn, nbytes, n=5, flops=None):
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
        row = dict(kernel=name, ms=round(best, 4), gb=round(nbytes / 1e9, 4), frac_of_measured_hbm=round(nbytes / 1e6 / best / hbm_gbs, 3))
        if flops:
            row["tflops"] = round(flops / best / 1e9, 1)
        rows.append(row)

    W, H, G, D, win = s["width"], s["heads"], s["kv_heads"], s["dim"], s["window"]
    nh, P, N, Gm = s["m_heads"], s["m_dim"], s["state"], s["groups"]
    dh, dq, dD, dV = s["d_heads"], s["d_qk"], s["d_dim"], s["d_vdim"]
    K, page = 4, 64
    for phase, T, ctx0 in (("prefill", prompt, 0), ("decode", 1, prompt)):
        B = batch
        R = B * T
        ctx = torch.full((B,), ctx0, dtype=torch.int32, device=dev)
        ql = torch.full((B,), T, dtype=torch.int32, device=dev)
        lines = torch.arange(B, dtype=torch.int32, device=dev)
        nblk = -(-(ctx0 + T) // page)
        table = torch.arange(B * nblk, dtype=torch.int32, device=dev).view(B, nblk)
        # residual stream
        x32, ya, yb = torch.randn(R, W, device=dev), torch.randn(R, W, device=dev, dtype=bf), torch.randn(R, W, device=dev, dtype=bf)
        w1, w2, w3, w4, w5 = (torch.randn(W, device=dev) for _ in range(5))
        run(f"{phase}: stream_sandwich_norm (two normalised results + post-norm + layer scale + sum + next norm)",
            lambda: ops.stream_sandwich_norm(x32, ya, yb, w1, w2, 0.5, 0.5, w3, w4, 0.5, w5, 1e-5, True, bf), R * W * (4 + 2 + 2 + 4 + 2))
        run(f"{phase}: stream_sandwich_norm (one result)", lambda: ops.stream_sandwich_norm(x32, ya, None, None, None, 1.0, 1.0, w3, w4, 0.5, w5, 1e-5, True, bf),
            R * W * (4 + 2 + 4 + 2))
        run(f"{phase}: scaled_add_rmsnorm (Fetodra: sum + norm)", lambda: ops.scaled_add_rmsnorm(x32, ya, w1, 1.0, 1e-5, 1.0, bf), R * W * (4 + 2 + 4 + 2))
        # attention front half
        Cq, Ck = H * D, G * D
        p = torch.randn(B, T, Cq + 2 * Ck + Cq, device=dev, dtype=bf)
        cos, sin = torch.randn(B, T, D // 2, device=dev), torch.randn(B, T, D // 2, device=dev)
        kc, vc = (torch.randn(B * nblk, page, G, D, device=dev, dtype=bf) for _ in range(2))
        qw, kw = torch.ones(D, device=dev), torch.ones(D, device=dev)
        run(f"{phase}: head_norm_rope_append (norm after rotation, own values)",
            lambda: ops.head_norm_rope_append(p, H, G, D, D, cos, sin, None, None, 2, 1e-5, False, kc, vc, table, ctx, ql), R * (Cq + 2 * Ck) * 2 * 2)
        run(f"{phase}: head_norm_rope_append (weighted norm before rotation, values from keys)",
            lambda: ops.head_norm_rope_append(p, H, G, D, D, cos, sin, qw, kw, 1, 1e-5, True, kc, vc, table, ctx, ql), R * (Cq + Ck) * 2 * 2 + R * Ck * 2)
        C = Cq + 2 * Ck
        cw, st = torch.randn(C, K, device=dev), torch.zeros(B + 1, K - 1, C, device=dev, dtype=bf)
        c4, s4 = torch.randn(B, T, D // 4, device=dev), torch.randn(B, T, D // 4, device=dev)
        qn, kn = torch.ones(Cq, device=dev), torch.ones(Ck, device=dev)
        run(f"{phase}: conv_qknorm_rope_append (Fetodra)", lambda: ops.conv_qknorm_rope_append(p, cw, st, lines, ctx, ql, qn, kn, 1e-5, H, G, D, D, c4, s4, kc, vc, table),
            R * C * 2 * 2)
        # attention
        q = torch.randn(B, T, H, D, device=dev, dtype=bf)
        keys = min(ctx0 + T, win) if T == 1 else ctx0 + T
        attn_bytes = (B * keys * G * D * 2 * 2) + R * H * D * 2 * 3
        pairs = sum(min(t + 1 + ctx0, win) for t in range(T)) * B * H
        fl = 4.0 * pairs * D
        sinks, temp, gate = torch.zeros(H, device=dev), torch.ones(H, device=dev), p[..., C:]
        run(f"{phase}: paged_window_attention (window {win}, sink, output gate)",
            lambda: ops.paged_window_attention(q, kc, vc, table, ctx, ql, D ** -0.5, None, win, 0, gate, sinks), attn_bytes, flops=fl)
        run(f"{phase}: paged_window_attention (window {win}, per-head temperature)",
            lambda: ops.paged_window_attention(q, kc, vc, table, ctx, ql, D ** -0.5, None, win, 0, None, None, head_scale=temp), attn_bytes, flops=fl)
        run(f"{phase}: paged_window_attention (Fetodra: window {win} + 4 kept, soft cap, output gate)",
            lambda: ops.paged_window_attention(q, kc, vc, table, ctx, ql, D ** -0.5, 30.0, win, 4, gate), attn_bytes, flops=fl)
        # gated delta rule beside Mamba-2
        Cd = 2 * dq * dD + dh * dV
        pd = torch.randn(B, T, Cd + 2 * dh + dh * dV, device=dev, dtype=bf)
        dw, dst = torch.randn(Cd, K, device=dev) * 0.3, torch.zeros(B + 1, K - 1, Cd, device=dev, dtype=bf)
        run(f"{phase}: short_conv+silu (q|k|v of the delta rule)", lambda: ops.short_conv(pd[..., :Cd], dw, None, dst, lines, ctx, ql, True), R * Cd * (2 + 4))
        qkv = torch.randn(B, T, Cd, device=dev) * 0.3
        Al, db = torch.zeros(dh, device=dev), torch.full((dh,), -2.0, device=dev)
        S0 = torch.zeros(B + 1, dh, dD, dV, device=dev)
        run(f"{phase}: gated_delta_scan ({dh} heads x {dD} x {dV})",
            lambda: ops.gated_delta_scan(qkv, pd[..., Cd:Cd + dh], pd[..., Cd + dh:Cd + 2 * dh], Al, db, S0, lines, ctx, ql, dh, dq, dD, dV),
            R * (Cd * 4 + dh * dV * 4) + B * dh * dD * dV * 4 * 2, n=3, flops=6.0 * R * dh * dD * dV)
        od, nw = torch.randn(B, T, dh * dV, device=dev), torch.ones(dV, device=dev)
        run(f"{phase}: head_rmsnorm_gate", lambda: ops.head_rmsnorm_gate(od, nw, dh, 1e-5, pd[..., Cd + 2 * dh:], "silu", bf), R * dh * dV * (4 + 2 + 2))
        inner = nh * P
        Cm = inner + 2 * Gm * N
        pm = torch.randn(B, T, inner + Cm + nh, device=dev, dtype=bf)
        xBC = torch.randn(B, T, Cm, device=dev) * 0.3
        Am, dm, Dk = torch.zeros(nh, device=dev), torch.full((nh,), -2.0, device=dev), torch.ones(nh, device=dev)
        Sm = torch.zeros(B + 1, nh, N, P, device=dev)
        run(f"{phase}: ssd_scan (Mamba-2 of both stacks, {nh} heads x {N} x {P})",
            lambda: ops.ssd_scan(xBC, pm[..., inner + Cm:], pm[..., :inner], Am, dm, Dk, Sm, lines, ctx, ql, nh, P, N, Gm),
            R * (Cm * 4 + inner * (2 + 4)) + B * nh * N * P * 4 * 2, n=3, flops=6.0 * R * nh * N * P)
        yv, wg = torch.randn(R, inner, device=dev), torch.ones(inner, device=dev)
        run(f"{phase}: group_rmsnorm (Mamba-2 of both stacks)", lambda: ops.group_rmsnorm(yv, wg, 1, 1e-5, bf), R * inner * (4 + 2))
        # feed-forward activations
        F = s["ff"]
        up = torch.randn(R, F * 3 // 2, device=dev, dtype=bf)
        run(f"{phase}: unary_act (erf GELU)", lambda: ops.unary_act(up, "gelu"), R * (F * 3 // 2) * 2 * 2)
        gu = torch.randn(R, 2 * F, device=dev, dtype=bf)
        run(f"{phase}: clamped_glu (Fetodra)", lambda: ops.clamped_glu(gu, 7.0), R * F * 2 * 3)
    return rows


def run(size="small", batch=4, prompt=1024, decode_steps=32, warmup=3):
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            peaks = json.load(f)
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    res = dict(size=size, shapes=SIZES[size], batch=batch, prompt=prompt, decode_steps=decode_steps, hbm_gbs=hbm,
               hbm_source="measured" if peaks else "fallback", bf16_tflops=peaks.get("bf16_tflops"))
    res.update(model_numbers(size, batch, prompt, decode_steps, warmup))
    res["kernels"] = kernel_table(size, batch, prompt, hbm)
    return res
