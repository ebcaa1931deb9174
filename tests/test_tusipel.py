"""Tusipel through the engine (loader, caches and carried rows per layer run, ragged batches, scheduler) against the plain definition
in ``tusipel_oracle.py``.  Every test makes its own small configuration and random checkpoint; the CPU tests run the PyTorch
definitions of the ops in float32, the ``gpu`` tests the sm_100a kernels in float32 and bfloat16."""
import json
import os

import pytest
import torch

import tusipel_oracle as oracle

PAGE = 8
YARN = dict(factor=3.0, original=40, fast=4.0, slow=0.5)


def latent(heads=3, dim=8, rot=8, vdim=12, kv_rank=20, q_rank=10, window=7, scale=0.3, base=100.0, scaling=YARN):
    rot_cfg = dict(base=base, dims=rot)
    if scaling:
        rot_cfg["scaling"] = dict(scaling)
    m = dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale, rot=rot_cfg)
    if window:
        m["mask"] = dict(size=window)
    return m


def attn(heads=4, kv_heads=2, dim=8, vdim=6, conv=2, chunk=9, scale=0.35):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, scale=scale)
    if chunk:
        m["mask"] = dict(size=chunk)
    return m


def dense(ff=24, limit=1.5):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(experts=5, identity=3, top=3, ff=16, groups=(4, 2), scale=1.7):
    r = dict(experts=experts, identity=identity, top=top, scale=scale)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(kind="moe", expert=dict(ff=ff), router=r)


def layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def make_config(layers, width=48, vocab=97, eps=1e-4, loop=(1, 3, 2), taps=4, emb_scale=2.5):
    cfg = dict(architecture="Tusipel", layers=layers, norm=dict(eps=eps), vocab=vocab, width=width, embedding=dict(scale=emb_scale))
    if taps:
        cfg["canon"] = dict(taps=taps)
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


STACK = [layer("attention", attn(), dense()), layer("latent_attention", latent(), moe()),
         layer("attention", attn(heads=6, kv_heads=3, dim=4, vdim=8, conv=3, chunk=5, scale=0.5), moe(experts=4, identity=2, top=2, ff=8, groups=(3, 2), scale=0.8)),
         layer("latent_attention", latent(heads=2, dim=16, rot=4, vdim=8, kv_rank=12, q_rank=24, window=11, scale=0.2, scaling=None), dense(ff=40, limit=0.7))]


def make_weights(cfg, seed=0):
    """Random checkpoint in the design's tensor names (bf16-representable values), every part large enough to matter."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=1.0, mean=0.0: (torch.randn(*s, generator=g) * std + mean).bfloat16().float()       # noqa: E731
    W, V, w = cfg["width"], cfg["vocab"], {}
    taps = (cfg.get("canon") or {}).get("taps")
    w["embed"], w["head"], w["final.norm"] = r(V, W, std=0.4), r(V, W, std=W ** -0.5 * 3), r(W, std=0.2)
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}.mix."
        w[f"l{i}.norm1"] = r(W, std=0.2)
        if taps:
            w[f"l{i}.canon1"] = r(W, taps, std=0.4)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "latent_attention":
            R, rot, Q = m["kv_rank"], m["rot_dim"], m["q_rank"]
            w[p + "dq"], w[p + "dq.norm"], w[p + "uq"] = r(Q, W, std=W ** -0.5), r(Q, std=0.3, mean=1.0), r(H * (d + rot), Q, std=Q ** -0.5 * 2)
            w[p + "dkv"], w[p + "dkv.norm"] = r(R + rot, W, std=W ** -0.5 * 1.5), r(R, std=0.3, mean=1.0)
            w[p + "uk"], w[p + "uv"] = r(H * d, R, std=R ** -0.5 * 2), r(H * dv, R, std=R ** -0.5)
            w[p + "g"] = r(H * dv, W, std=W ** -0.5 * 2)
        else:
            G = m["kv_heads"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[p + n] = r(rows, W, std=W ** -0.5 * 1.5)
                if m.get("conv"):
                    w[p + n + ".conv"] = r(rows, m["conv"], std=0.6)
        w[p + "o"] = r(W, H * dv, std=(H * dv) ** -0.5)
        f = L["mlp"]
        if f is None:
            continue
        q = f"l{i}.mlp."
        w[f"l{i}.norm2"] = r(W, std=0.2)
        if taps:
            w[f"l{i}.canon2"] = r(W, taps, std=0.4)
        if f["kind"] == "dense":
            w[q + "gate"], w[q + "up"], w[q + "down"] = r(f["ff"], W, std=W ** -0.5 * 2), r(f["ff"], W, std=W ** -0.5 * 2), r(W, f["ff"], std=f["ff"] ** -0.5)
        else:
            n = f["router"]["experts"] + f["router"].get("identity", 0)
            w[q + "router"], w[q + "correction"] = r(n, W, std=W ** -0.5 * 2), r(n, std=0.15)
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                w[f"{q}e{e}.gate"], w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = r(ff, W, std=W ** -0.5 * 2), r(ff, W, std=W ** -0.5), r(W, ff, std=ff ** -0.5)
    return w


def make_engine(tmp_path, cfg, w, dtype="float32", device="cpu", max_tokens=512, max_requests=4, name="ckpt", page=PAGE):
    from safetensors.torch import save_file
    from neuronx_distributed_inference_b200.runtime.scheduler import build_engine
    d = tmp_path / name
    os.makedirs(d, exist_ok=True)
    with open(d / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.bfloat16().contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
    return build_engine(str(d), dtype, max_tokens, max_requests, page, device=device)


def rel_err(got, want):
    got, want = got.double(), want.double()
    return float((got - want).norm() / want.norm().clamp_min(1e-9))


def feed(engine, rid, tokens, cuts, want=None):
    rows, a = [], 0
    for b in list(cuts) + [len(tokens)]:
        if b <= a:
            continue
        idx = [i - a for i in (range(a, b) if want is None else [p for p in want if a <= p < b])]
        rows.append(engine.step([(rid, tokens[a:b], idx)])[0])
        a = b
    return torch.cat(rows, 0)


TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def close(got, want, dtype):
    """float32: the whole block within a tight relative error.  bfloat16: rounding may flip a router's choice between two experts whose
    scores nearly tie, which moves single positions by more than rounding does, so positions are assessed one by one: the typical
    one within the tolerance, few beyond three times that."""
    if dtype == "float32":
        return rel_err(got, want) < TOL[dtype]
    got, want = got.double(), want.double()
    e = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-9)
    return float(e.median()) < TOL[dtype] and float((e > 3 * TOL[dtype]).double().mean()) <= 0.1


def check_schedules(tmp_path, device, dtype, layers=STACK, T=61, seed=0, **cfg_kw):
    cfg = make_config(layers, **cfg_kw)
    w = make_weights(cfg, seed)
    eng = make_engine(tmp_path, cfg, w, dtype, device)
    toks = torch.randint(0, cfg["vocab"], (T,), generator=torch.Generator().manual_seed(seed + 1)).tolist()
    want = oracle.forward(cfg, w, toks)
    whole = feed(eng, "whole", toks, [])
    assert close(whole, want, dtype)
    eng.release("whole")
    # most of the prompt at once, the rest token by token (slot and pages of the released request are used again): windows and chunks
    # pass over decoded tokens, their edges fall on decoded positions
    dec = feed(eng, "dec", toks, [T - 25] + list(range(T - 24, T)))
    assert close(dec, want, dtype) and close(dec[-25:], want[-25:], dtype)
    eng.release("dec")
    # token by token from the first token on
    one = feed(eng, "one", toks[:24], range(1, 24))
    assert close(one, want[:24], dtype) and close(one[:3], want[:3], dtype)
    eng.release("one")
    # portions of changing size, down to two tokens and across page, window and chunk borders
    cuts, a, sizes = [], 0, [2, 7, 2, 3, PAGE, 1, 2, 13, 5, 2]
    while a < T:
        a += sizes[len(cuts) % len(sizes)]
        cuts.append(min(a, T))
    ch = feed(eng, "ch", toks, cuts)
    assert close(ch, want, dtype)
    eng.release("ch")
    assert eng.pages.available == eng.pages.num_pages and eng.slots.available == eng.slots.num_pages
    return eng, cfg, w


def check_mixed_batches(eng, cfg, w, dtype, n_req=6, seed=3):
    """Unequal requests side by side (portions of some beside single tokens of others) against each alone; more requests than slots,
    so slots and pages are freed and taken again."""
    g = torch.Generator().manual_seed(seed)
    lens = [int(torch.randint(5, 60, (1,), generator=g)) for _ in range(n_req)]
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    want = [oracle.forward(cfg, w, r) for r in reqs]
    got, at = [[] for _ in reqs], [0] * n_req
    waiting, live, step = list(range(n_req)), [], 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries = []
        for k, i in enumerate(live):
            left = len(reqs[i]) - at[i]
            n = 1 if (at[i] > 0 and (step + k) % 3 == 0) else min(left, [2, 9, 4, 17][(step + i) % 4])
            entries.append((("r", i), reqs[i][at[i]:at[i] + n], list(range(n))))
        rows = eng.step(entries)
        for (rid, toks, _), row in zip(entries, rows):
            i = rid[1]
            got[i].append(row)
            at[i] += len(toks)
            if at[i] == len(reqs[i]):
                eng.release(rid)
                live.remove(i)
        step += 1
    if dtype == "float32":
        for i in range(n_req):
            assert close(torch.cat(got[i], 0), want[i], dtype), i
        return
    # bfloat16: a short request can sit next to a router tie from its first tokens on, so the positions of all requests are assessed
    # together; that a request's rows do not depend on its neighbours is checked against the same request fed alone
    assert close(torch.cat([torch.cat(x, 0) for x in got], 0), torch.cat(want, 0), dtype)
    for i in range(n_req):
        alone = feed(eng, ("alone", i), reqs[i], [])
        eng.release(("alone", i))
        e = (torch.cat(got[i], 0).double() - alone.double()).norm(dim=-1) / want[i].norm(dim=-1)
        assert float(e.median()) < TOL[dtype] / 2 and float((e > 3 * TOL[dtype]).double().mean()) <= 0.1, i      # a flipped tie moves single positions


def check_generate(eng, cfg, w, dtype):
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (5, 23, 1, 40, 12, 9)]
    outs = eng.generate(prompts, max_new_tokens=6, max_step_tokens=16)
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        seq = list(p)
        for tok in o:       # every emitted token is the arg-max of the plain model (ties aside: compare its logit with the best)
            lg = oracle.forward(cfg, w, seq)[-1]
            assert float(lg.max() - lg[tok]) <= (1e-3 if dtype == "float32" else 0.15) * float(lg.abs().max())
            seq.append(tok)


# ---- CPU: PyTorch definitions of the ops, float32 --------------------------------------------------------------------------
def test_stack_schedules_mixed_batches_and_generation(tmp_path):
    eng, cfg, w = check_schedules(tmp_path, "cpu", "float32")
    check_mixed_batches(eng, cfg, w, "float32")
    check_generate(eng, cfg, w, "float32")


OTHER = [
    # one latent layer: one head, plain frequencies, no window, a feed-forward without groups, identity experts or scale
    ([layer("latent_attention", latent(heads=1, dim=4, rot=2, vdim=4, kv_rank=4, q_rank=4, window=None, scaling=None),
            moe(experts=3, identity=0, top=1, ff=8, groups=None, scale=1.0))], dict(loop=None, taps=0, emb_scale=1.0)),
    # attention alone: as many kv heads as heads, one tap (no convolution), no chunk, no feed-forward; the only layer repeats
    ([layer("attention", attn(heads=2, kv_heads=2, dim=6, vdim=6, conv=1, chunk=None), None)], dict(loop=(0, 1, 3), taps=1)),
    # one kv head for all heads, a span of one layer that runs once, every expert chosen, two taps everywhere
    ([layer("attention", attn(heads=3, kv_heads=1, dim=4, vdim=10, conv=5, chunk=3), moe(experts=2, identity=2, top=4, ff=12, groups=(2, 2))),
      layer("latent_attention", latent(window=1), dense()), layer("latent_attention", latent(heads=5, dim=6, rot=6, vdim=10, kv_rank=14, q_rank=7, window=64), None)],
     dict(loop=(2, 3, 1), taps=2, width=40, vocab=31)),
    # the whole stack repeats; head, value and latent sizes that coincide; a window and a chunk of one page
    ([layer("latent_attention", latent(heads=2, dim=8, rot=8, vdim=8, kv_rank=8, q_rank=8, window=PAGE), dense(ff=48)),
      layer("attention", attn(heads=2, kv_heads=1, dim=8, vdim=8, conv=4, chunk=PAGE), moe(experts=6, identity=2, top=2, ff=8, groups=(4, 1)))],
     dict(loop=(0, 2, 2), taps=4, width=56)),
]


@pytest.mark.parametrize("layers,kw", OTHER)
def test_other_sizes_and_layouts(tmp_path, layers, kw):
    check_schedules(tmp_path, "cpu", "float32", layers=layers, T=45, seed=5, **kw)


def test_streams_after_every_run_and_run_order(tmp_path):
    assert oracle.layer_order(5, dict(start=1, stop=3, times=2)) == [(0, False), (1, False), (2, False), (1, True), (2, False), (3, False), (4, False)]
    cfg = make_config(STACK)
    w = make_weights(cfg, 2)
    eng = make_engine(tmp_path, cfg, w)
    toks = list(range(3, 20))
    streams = []
    oracle.forward(cfg, w, toks, streams)
    model = eng.app.context_encoding_model.model if hasattr(eng.app, "context_encoding_model") else eng.app.model
    assert [i for i, _ in model.runs] == [i for i, _ in oracle.layer_order(len(STACK), cfg["loop"])]
    T = len(toks)
    out = model(torch.tensor([toks]), attention_mask=torch.ones(1, T, dtype=torch.int32), position_ids=torch.arange(T).view(1, T),
                seq_ids=torch.tensor([0]), slot_mapping=torch.arange(T).view(1, T).int(), block_table=torch.arange(4).view(1, 4).int(),
                computed_context_lens=torch.tensor([0]), capture=True)
    assert len(streams) == 6
    for r, s in enumerate(streams):
        assert torch.allclose(out.captured[f"runs.{r}.out"][0].double(), s, atol=2e-4), r


def test_long_decoding_over_many_pages(tmp_path):
    cfg = make_config(STACK[:2], loop=(0, 2, 2))
    w = make_weights(cfg, 9)
    eng = make_engine(tmp_path, cfg, w)
    toks = torch.randint(0, cfg["vocab"], (90,), generator=torch.Generator().manual_seed(2)).tolist()
    got = feed(eng, "x", toks, range(3, 90))         # 3-token prompt, then 87 single tokens over twelve pages
    assert rel_err(got, oracle.forward(cfg, w, toks)) < TOL["float32"]


def test_cache_pool_smaller_than_all_requests(tmp_path):
    """The pool holds two requests' worth of pages: the third request runs on the pages and the slot the first gave back, and must not
    see what the first left in them (keys, carried rows)."""
    cfg = make_config(STACK[:3], loop=None)
    w = make_weights(cfg, 4)
    eng = make_engine(tmp_path, cfg, w, max_tokens=64, max_requests=2)
    g = torch.Generator().manual_seed(6)
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (30, 27, 31)]
    a = feed(eng, 0, reqs[0], [11])
    b = feed(eng, 1, reqs[1], [5, 6])
    with pytest.raises(MemoryError):
        eng.step([(2, reqs[2], [])])
    eng.release(2)
    eng.release(0)
    c = feed(eng, 2, reqs[2], [2, 17])
    for got, r in ((a, reqs[0]), (b, reqs[1]), (c, reqs[2])):
        assert rel_err(got, oracle.forward(cfg, w, r)) < TOL["float32"]


# ---- mechanisms alone: op definitions (CPU) or kernels (GPU) against the plain functions ---------------------------------------
def paged(rows, page, g, spare=3):
    """rows [n, C] -> (cache [blocks, page, 1, C] on scattered pages, block table [1, blocks])."""
    n, C = rows.shape
    nblk = -(-n // page)
    perm = torch.randperm(nblk + spare, generator=g)[:nblk]
    cache = torch.zeros(nblk + spare, page, 1, C)
    for j in range(n):
        cache[perm[j // page], j % page, 0] = rows[j]
    return cache, perm.view(1, -1).int()


def loud_key_case(dev, dtype, target, pos, *, window=None, chunk=None, slopes=False, tail=0, page=4, as_prompt=False, extra=0):
    """Two heads over a cache of one kv head whose row ``target`` is made to dominate the query at ``pos`` (scale one query and one key so
    that one score stands out); ``tail`` > 0: the key row is ``tail`` numbers wider than the value, which is its prefix; ``extra`` later
    rows sit in the same portion.  Returns (op output, plain output, the loud row's value) for the query at ``pos``."""
    from neuronx_distributed_inference_b200 import ops
    H, R = 2, 8
    D = R + tail
    g = torch.Generator().manual_seed(target * 131 + pos)
    n = pos + 1 + extra
    c = torch.randn(n, D, generator=g) * 0.1
    q = torch.randn(n, H, D, generator=g) * 0.1
    if 0 <= target < n:
        c[target] = 3.0
    q[pos] = 3.0
    sl = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]) if slopes else None
    j = torch.arange(pos + 1)
    see = torch.ones(pos + 1, dtype=torch.bool)
    if window:
        see &= (pos - j) < window
    if chunk:
        see &= (j // chunk) == (pos // chunk)
    s = torch.einsum("hr,jr->hj", q[pos].double(), c[:pos + 1].double()) * 0.25
    if slopes:
        s = s - sl.double().view(H, 1) * (pos - j).double()
    want = (oracle.softmax_rows(s, see.view(1, -1)) @ c[:pos + 1, :R].double()).reshape(-1)
    cache, table = paged(c, page, g)
    to = lambda t: t.to(dev, dtype)                                      # noqa: E731
    i32 = lambda *v: torch.tensor(v).int().to(dev)                       # noqa: E731
    kw = dict(chunk=chunk, slopes=None if sl is None else sl.to(dev), value_dim=R if tail else None)
    if as_prompt:
        got = ops.paged_window_attention(to(q.view(1, n, H, D)), to(cache), to(cache), table.to(dev), i32(0), i32(n), 0.25, None, window, 0, **kw)[0, pos]
    else:
        got = ops.paged_window_attention(to(q[pos].view(1, 1, H, D)), to(cache), to(cache), table.to(dev), i32(pos), i32(1), 0.25, None, window, 0, **kw)
    return got.float().cpu().view(-1), want.float(), (c[target, :R] if 0 <= target < n else None)


# (mask, position, loud key, is it visible): far keys, page borders (pages of 4), the first tokens, both sides of every edge
EDGES = [(dict(window=40), 300, 261, True), (dict(window=40), 300, 260, False), (dict(window=40), 39, 0, True), (dict(window=40), 40, 0, False),
         (dict(window=40), 40, 1, True), (dict(window=1), 9, 9, True), (dict(window=1), 9, 8, False), (dict(window=4), 8, 5, True), (dict(window=4), 8, 4, False),
         (dict(chunk=96), 300, 288, True), (dict(chunk=96), 300, 287, False), (dict(chunk=96), 95, 0, True), (dict(chunk=96), 96, 95, False),
         (dict(chunk=96), 96, 96, True), (dict(chunk=4), 7, 4, True), (dict(chunk=4), 7, 3, False), (dict(chunk=4), 8, 7, False), (dict(chunk=1), 5, 4, False),
         (dict(), 300, 0, True), (dict(), 301, 150, True), (dict(), 0, 0, True), (dict(), 4, 4, True), (dict(), 8, 7, True)]


@pytest.mark.parametrize("mask,pos,target,visible", EDGES)
@pytest.mark.parametrize("as_prompt", [False, True])
@pytest.mark.parametrize("tail", [0, 4])
def test_loud_keys_at_window_chunk_and_page_edges(mask, pos, target, visible, as_prompt, tail):
    got, want, row = loud_key_case("cpu", torch.float32, target, pos, as_prompt=as_prompt, tail=tail, **mask)
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.allclose(got[:8], row, atol=1e-3) == visible          # the loud row is what the head returns exactly when it is visible


def test_a_prompt_does_not_see_later_rows_of_its_portion():
    got, want, row = loud_key_case("cpu", torch.float32, 21, 20, as_prompt=True, extra=3, chunk=16)       # the loud row is one step ahead
    assert torch.allclose(got, want, atol=1e-5) and not torch.allclose(got[:8], row, atol=0.5)


def test_distance_term_grows_with_distance_and_differs_by_head():
    near, want, row = loud_key_case("cpu", torch.float32, 398, 400, slopes=True, chunk=512)
    assert torch.allclose(near, want, atol=1e-5) and torch.allclose(near[:8], row, atol=1e-2)
    far, want, row = loud_key_case("cpu", torch.float32, 2, 400, slopes=True, chunk=512)
    assert torch.allclose(far, want, atol=1e-5)
    # score 18 against a distance term of 398 * (1/16 | 1/256): head 0 has lost the loud key, head 1 still returns it
    assert not torch.allclose(far[:8], row, atol=0.5) and torch.allclose(far[8:], row, atol=1e-2)


def test_stream_norm_and_convolution_carry_rows_across_cuts():
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(5)
    T, W, K, eps = 19, 24, 4, 1e-3
    x, y, z = (torch.randn(1, T, W, generator=g) for _ in range(3))
    wn, cw = torch.randn(W, generator=g) * 0.2, torch.randn(W, K, generator=g)
    want_s = (x + y + z)[0].double()
    want = oracle.canon(oracle.block_norm(want_s, wn.double(), eps), cw.double())
    state = torch.full((3, K - 1, W), 7.0)                                     # a dirty line: it counts as zero for a fresh sequence
    line, got, at = torch.tensor([1]).int(), [], 0
    for n in (1, 2, 5, 1, 1, 3, 6):
        sl = slice(at, at + n)
        ctx, ql = torch.tensor([at]).int(), torch.tensor([n]).int()
        s, h = ops.stream_norm_conv(x[:, sl], (y[:, sl], z[:, sl]), 1.0 + wn, cw, state, line, ctx, ql, eps)
        ops.short_conv_update(s, state, line, ctx, ql)
        assert torch.allclose(s[0].double(), want_s[sl], atol=1e-6)
        got.append(h[0])
        at += n
    assert torch.allclose(torch.cat(got).double(), want, atol=1e-5)
    assert torch.all(state[0] == 7.0) and torch.all(state[2] == 7.0)          # other sequences' lines are untouched
    s, h = ops.stream_norm_conv(x, (), 1.0 + wn, None, None, None, torch.tensor([0]).int(), torch.tensor([T]).int(), eps)
    assert torch.allclose(h[0].double(), oracle.block_norm(x[0].double(), wn.double(), eps), atol=1e-5)


def test_scaled_rotation_tables_and_rotate_half_layout():
    from neuronx_distributed_inference_b200 import ops
    from neuronx_distributed_inference_b200.models.tusipel.modeling_tusipel import rope_of
    from neuronx_distributed_inference_b200.modules.attention.conv_window_attention import ragged_rope_tables

    class Meta:
        extras = dict(ctx_len=torch.tensor([0, 1000]).int())
    for rot in (dict(base=100.0, dims=8, scaling=YARN), dict(base=50000.0, dims=6), dict(base=10.0, dims=4, scaling=dict(factor=1.0, original=8, fast=2.0, slow=1.0))):
        inv, mag, tag = rope_of(rot)
        Meta.extras = dict(ctx_len=torch.tensor([0, 1000]).int())
        cos, sin = ragged_rope_tables(Meta, 5, rot["dims"], 0.0, inv, mag, tag)
        c, s = oracle.yarn_tables(1005, rot)
        assert torch.allclose(cos[0].double(), c[:5], atol=1e-6) and torch.allclose(sin[1].double(), s[1000:], atol=1e-6)
    rot = dict(base=100.0, dims=8, scaling=YARN)
    Meta.extras = dict(ctx_len=torch.tensor([0, 1000]).int())
    cos, sin = ragged_rope_tables(Meta, 5, 8, 0.0, *rope_of(rot))
    c, s = oracle.yarn_tables(1005, rot)
    g = torch.Generator().manual_seed(2)
    src, dst = torch.randn(2, 5, 3, 12, generator=g), torch.zeros(2, 5, 3, 20)
    ops.rope_half_tail(src, dst, 8, cos, sin)
    want = oracle.rotate_half(src[1, :, :, 4:].double(), c[1000:], s[1000:])
    assert torch.allclose(dst[1, :, :, 12:].double(), want, atol=1e-5) and torch.all(dst[..., :12] == 0)


def test_latent_rows_rotated_part_and_query_latent_land_where_they_belong():
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(1)
    B, T, Q, R, rot, page = 2, 6, 5, 10, 4, 4
    p, wn, wq = torch.randn(B, T, Q + R + rot + 7, generator=g), torch.randn(R, generator=g), torch.randn(Q, generator=g)
    cos, sin = torch.randn(B, T, rot // 2, generator=g), torch.randn(B, T, rot // 2, generator=g)
    cache = torch.full((7, page, 1, R + rot), 9.0)
    table, ctx, ql = torch.tensor([[5, 2, 0], [1, 6, 3]]).int(), torch.tensor([3, 0]).int(), torch.tensor([2, 6]).int()
    _, cq = ops.latent_norm_append(p, Q, R, wn, 1e-3, cache, table, ctx, ql, rot_dim=rot, cos=cos, sin=sin, q_rank=Q, q_weight=wq)
    for b in range(B):
        for t in range(int(ql[b])):
            pos = int(ctx[b]) + t
            row = cache[int(table[b, pos // page]), pos % page, 0].double()
            assert torch.allclose(row[:R], oracle.rms(p[b, t, Q:Q + R].double(), 1e-3) * wn.double(), atol=1e-5)
            assert torch.allclose(row[R:], oracle.rotate_half(p[b, t, Q + R:Q + R + rot].double(), cos[b, t].double(), sin[b, t].double()), atol=1e-5)
            assert torch.allclose(cq[b, t].double(), oracle.rms(p[b, t, :Q].double(), 1e-3) * wq.double(), atol=1e-5)
    assert int((cache != 9.0).any(-1).sum()) == 8                       # nothing but the live rows was written


def test_router_groups_correction_and_identity_experts():
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(8)
    z, corr = torch.randn(40, 12, generator=g) * 2, torch.randn(12, generator=g) * 0.2
    r = dict(experts=9, identity=3, top=3, scale=2.5, groups=dict(count=4, keep=2))
    wt, idx = ops.moe_route(z, 3, "softmax", False, False, None, corr, (4, 2), 2.5)
    wo, io = oracle.route(z.double(), corr.double(), r)
    assert torch.equal(idx.sort(-1).values, io.sort(-1).values) and torch.allclose(wt.double().sum(-1), wo.sum(-1), atol=1e-6)
    assert float(wt.sum(-1).max()) <= 2.5 + 1e-5 and not torch.allclose(wt.sum(-1), torch.full((40,), 2.5))      # scaled, not renormalised
    # corrections that make every choice score negative: an expert outside the kept groups is never chosen although "0" would beat them
    neg = -1.0 - torch.rand(12, generator=g)
    _, idx = ops.moe_route(z, 3, "softmax", False, False, None, neg, (4, 1), 1.0)
    assert torch.equal(idx.sort(-1).values, oracle.route(z.double(), neg.double(), dict(r, groups=dict(count=4, keep=1)))[1].sort(-1).values)
    assert torch.all((idx // 3) == (idx // 3)[:, :1])                    # all three from the one kept group
    # a correction moves the choice, not the weight
    push = torch.zeros(12)
    push[7] = 5.0
    wt, idx = ops.moe_route(z, 1, "softmax", False, False, None, push, None, 1.0)
    assert torch.all(idx == 7) and torch.allclose(wt[:, 0], torch.softmax(z, -1)[:, 7], atol=1e-6)
    # identity experts: ids past the real experts return the input times the weight
    x, y = torch.randn(40, 16, generator=g), torch.randn(40, 16, generator=g)
    wt, idx = ops.moe_route(z, 3, "softmax", False, False, None, corr, None, 2.5)
    got = ops.identity_expert_add(y.clone(), x, wt, idx, 9)
    coef = (wt * (idx >= 9)).sum(-1, keepdim=True)
    assert torch.allclose(got, y + x * coef, atol=1e-6) and float(coef.max()) > 0


def test_feed_forwards_and_mixers_match_the_plain_functions(tmp_path):
    """One layer of each kind through the model's own modules (loader included) against the plain function of the same mechanism."""
    for spec in (layer("attention", attn(), moe()), layer("latent_attention", latent(), dense())):
        cfg = make_config([spec], loop=None)
        w = make_weights(cfg, 7)
        eng = make_engine(tmp_path, cfg, w, name=spec["type"])
        model = eng.app.context_encoding_model.model if hasattr(eng.app, "context_encoding_model") else eng.app.model
        T = 21
        toks = torch.randint(0, cfg["vocab"], (T,), generator=torch.Generator().manual_seed(1))
        wd = {k: v.double() for k, v in w.items()}
        x = wd["embed"][toks] * cfg["embedding"]["scale"]
        h = oracle.canon(oracle.block_norm(x, wd["l0.norm1"], cfg["norm"]["eps"]), wd["l0.canon1"])
        mix = oracle.conv_attention(h, wd, "l0.mix.", spec["mixer"]) if spec["type"] == "attention" else \
            oracle.latent_attention(h, wd, "l0.mix.", spec["mixer"], cfg["norm"]["eps"])
        x1 = x + mix
        h2 = oracle.canon(oracle.block_norm(x1, wd["l0.norm2"], cfg["norm"]["eps"]), wd["l0.canon2"])
        ff = oracle.moe_ff(h2, wd, "l0.mlp.", spec["mlp"]) if spec["mlp"]["kind"] == "moe" else oracle.dense_ff(h2, wd, "l0.mlp.", spec["mlp"])
        meta = model.build_meta(toks.view(1, T), torch.ones(1, T, dtype=torch.int32), torch.arange(T).view(1, T), torch.tensor([0]), True,
                                slot_mapping=torch.arange(T).view(1, T).int(), block_table=torch.arange(4).view(1, 4).int(),
                                computed_context_lens=torch.tensor([0]))
        xs, pending = model.layers[0](model.embed(toks.view(1, T)), None, meta, model.kv_mgr, 0)
        assert torch.allclose(xs[0].double(), x1, atol=1e-4)
        assert torch.allclose(pending[0].double(), ff, atol=1e-4)


def test_registry_picks_the_model_from_config_json(tmp_path):
    from neuronx_distributed_inference_b200.utils.constants import get_model_cls, model_type_of
    with open(tmp_path / "config.json", "w") as f:
        json.dump(make_config(STACK), f)
    assert get_model_cls(model_type_of(str(tmp_path))).__name__ == "NeuronTusipelForCausalLM"


def test_command_line_generates_from_token_ids(tmp_path, capsys):
    from neuronx_distributed_inference_b200 import inference_demo
    cfg = make_config(STACK)
    w = make_weights(cfg)
    eng = make_engine(tmp_path, cfg, w)
    want = eng.generate([[1, 2, 3, 4], [7, 8]], 5)
    inference_demo.main(["--model-type", "tusipel", "--task-type", "causal-lm", "run", "--model-path", str(tmp_path / "ckpt"),
                         "--compiled-model-path", str(tmp_path / "c"), "--on-cpu", "--torch-dtype", "float32", "--prompt-token-ids", "1,2,3,4",
                         "--prompt-token-ids", "7,8", "--max-new-tokens", "5", "--pa-block-size", str(PAGE)])
    out = capsys.readouterr().out
    assert "Output 0: " + ",".join(map(str, want[0])) in out and "Output 1: " + ",".join(map(str, want[1])) in out


# ---- GPU: the sm_100a kernels --------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpu_stack_schedules_mixed_batches_and_generation(tmp_path, dtype):
    from neuronx_distributed_inference_b200 import ops
    ops.stats.clear()
    eng, cfg, w = check_schedules(tmp_path, "cuda", dtype)
    check_mixed_batches(eng, cfg, w, dtype)
    check_generate(eng, cfg, w, dtype)
    for k in ("stream_norm_conv", "short_conv_update", "latent_norm_append", "rope_half_tail", "conv_qknorm_rope_append", "paged_window_attention",
              "gated_act_mul", "clamped_glu", "router_topk", "identity_expert_add", "stream_add_rmsnorm"):
        assert ops.stats[k] > 0, k
    assert ops.stats["moe_plain_gated"] > 0                                # experts of sizes no tensor-core tile fits
    tkg = eng.app.token_generation_model          # single-token steps replayed from CUDA graphs (capture did not fall back to eager)
    assert tkg.use_graphs and len(tkg._graphs) > 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank,rot", [(128, 64), (64, 16), (96, 32)])
def test_gpu_wider_stack(tmp_path, dtype, rank, rot):
    """Head sizes of 64 / 128 and latent rows of 128 + 64 and 64 + 16 numbers (tensor-core attention on bf16 portions) beside a row size
    that takes the CUDA-core kernel; experts in multiples of 64 (grouped tensor-core products) beside a size that is not."""
    layers = [layer("latent_attention", latent(heads=6, dim=32, rot=rot, vdim=48, kv_rank=rank, q_rank=72, window=33, scale=0.15), moe(experts=6, identity=2, top=3, ff=128, groups=(4, 3))),
              layer("attention", attn(heads=6, kv_heads=2, dim=64, vdim=64, conv=3, chunk=40, scale=0.12), dense(ff=256, limit=2.0)),
              layer("attention", attn(heads=4, kv_heads=4, dim=128, vdim=64, conv=2, chunk=24, scale=0.1), moe(experts=5, identity=1, top=2, ff=40, groups=None))]
    eng, cfg, w = check_schedules(tmp_path, "cuda", dtype, layers=layers, T=77, width=384, vocab=301, eps=1e-6, seed=7, loop=(0, 2, 2), taps=3)
    check_mixed_batches(eng, cfg, w, dtype, n_req=5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layers,kw", OTHER)
def test_gpu_other_sizes_and_layouts(tmp_path, dtype, layers, kw):
    """Sizes that no vector access or tensor-core tile fits (odd widths, one head, one expert) take the scalar kernels and library products."""
    check_schedules(tmp_path, "cuda", dtype, layers=layers, T=45, seed=5, **kw)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mask,pos,target,visible", EDGES)
@pytest.mark.parametrize("as_prompt", [False, True])
def test_gpu_loud_keys_at_window_chunk_and_page_edges(mask, pos, target, visible, dtype, as_prompt):
    for tail, slopes in ((0, False), (4, False), (0, True)):
        got, want, row = loud_key_case("cuda", dtype, target, pos, as_prompt=as_prompt, tail=tail, slopes=slopes, **mask)
        assert torch.allclose(got, want, atol=1e-4 if dtype == torch.float32 else 3e-2)
        if not slopes:
            assert torch.allclose(got[:8], row, atol=3e-2) == visible


@pytest.mark.gpu
def test_gpu_kernels_match_definitions():
    """Each new or extended kernel against the PyTorch definition of the same op, both activation types, ragged rows, strided inputs."""
    from neuronx_distributed_inference_b200 import ops
    from neuronx_distributed_inference_b200.ops import reference as ref
    dev = "cuda"
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)        # noqa: E731
    on = lambda *ts: [None if t is None else t.to(dev) for t in ts]      # noqa: E731
    for dt in (torch.float32, torch.bfloat16):
        tol = 1e-5 if dt == torch.float32 else 3e-2
        # stream sum + norm + convolution over ragged rows with carried rows
        for W, K in ((200, 3), (1024, 4), (72, 1), (2048, 2)):
            B, T = 3, 11
            ctx, ql, lines = torch.tensor([0, 5, 40]).int(), torch.tensor([11, 4, 1]).int(), torch.tensor([2, 0, 3]).int()
            x, y1, y2, wn, cw, st = rn(B, T, W), rn(B, T, W).to(dt), rn(B, T, W), rn(W), rn(W, K), rn(5, K - 1, W)
            a = ref.stream_norm_conv(x, (y1, y2), wn, cw, st, lines, ctx, ql, 1e-5, dt)
            b = ops.stream_norm_conv(*on(x), tuple(on(y1, y2)), *on(wn, cw, st, lines, ctx, ql), 1e-5, dt)
            live = (torch.arange(T).view(1, T) < ql.view(B, 1)).unsqueeze(-1)
            assert torch.allclose(a[0] * live, b[0].cpu() * live, atol=1e-5) and torch.allclose(a[1].float() * live, b[1].float().cpu() * live, atol=tol * 4)
        # latent rows with a rotated part and a query latent
        B, T, Q, R, rot, page, H = 3, 40, 24, 48, 16, 8, 5
        ctx, ql = torch.tensor([0, 13, 30]).int(), torch.tensor([40, 9, 1]).int()
        nblk = 9
        table = torch.randperm(B * nblk, generator=g).view(B, nblk).int()          # every row its own pages
        p, lw, qw = rn(B, T, Q + R + rot + H * 8).to(dt), rn(R), rn(Q)
        cos, sin = rn(B, T, rot // 2), rn(B, T, rot // 2)
        c1 = rn(B * nblk, page, 1, R + rot).to(dt)
        c2 = c1.clone().to(dev)
        _, q1 = ref.latent_norm_append(p, Q, R, lw, 1e-5, c1, table, ctx, ql, False, rot, cos, sin, Q, qw)
        _, q2 = ops.latent_norm_append(*on(p), Q, R, *on(lw), 1e-5, c2, *on(table, ctx, ql), False, rot, *on(cos, sin), Q, *on(qw))
        live = (torch.arange(T).view(1, T) < ql.view(B, 1)).unsqueeze(-1)
        assert torch.allclose(c1.float(), c2.float().cpu(), atol=tol, rtol=1e-4) and torch.allclose(q1.float() * live, q2.float().cpu() * live, atol=tol * 2)
        src = rn(B, T, H, 12 + rot).to(dt)
        d1, d2 = torch.zeros(B, T, H, R + rot, dtype=dt), torch.zeros(B, T, H, R + rot, dtype=dt, device=dev)
        ref.rope_half_tail(src, d1, rot, cos, sin)
        ops.rope_half_tail(src.to(dev), d2, rot, *on(cos, sin))
        assert torch.allclose(d1.float(), d2.float().cpu(), atol=tol)
        # attention over those rows: window, values as the prefix of the key rows
        q = rn(B, T, H, R + rot).to(dt) * 0.3
        a = ref.paged_window_attention(q, c1, c1, table, ctx, ql, 0.2, None, 7, 0, value_dim=R)
        b = ops.paged_window_attention(q.to(dev), c2, c2, *on(table, ctx, ql), 0.2, None, 7, 0, value_dim=R)
        assert torch.allclose(a.float() * live, b.float().cpu() * live, atol=tol)
        # grouped-query attention with chunks and distance slopes; convolved projections without norms or rotation
        Hq, G, D, Dv, K = 6, 2, 16, 24, 3
        C = Hq * D + G * (D + Dv)
        pr, cw, st, lines = rn(B, T, C + 5).to(dt), rn(C, K), rn(4, K - 1, C).to(dt), torch.tensor([1, 0, 2]).int()
        k1, v1 = rn(B * nblk, page, G, D).to(dt), rn(B * nblk, page, G, Dv).to(dt)
        k2, v2 = k1.clone().to(dev), v1.clone().to(dev)
        qa = ref.conv_qknorm_rope_append(pr, cw, st, lines, ctx, ql, None, None, 1e-5, Hq, G, D, Dv, None, None, k1, v1, table)
        qb = ops.conv_qknorm_rope_append(*on(pr, cw, st, lines, ctx, ql), None, None, 1e-5, Hq, G, D, Dv, None, None, k2, v2, table.to(dev))
        assert torch.allclose(qa.float() * live.unsqueeze(-1), qb.float().cpu() * live.unsqueeze(-1), atol=tol * 4)
        assert torch.allclose(k1.float(), k2.float().cpu(), atol=tol * 4) and torch.allclose(v1.float(), v2.float().cpu(), atol=tol * 4)
        sl = torch.tensor([2.0 ** (-8.0 * (h + 1) / Hq) for h in range(Hq)])
        a = ref.paged_window_attention(qa, k1, v1, table, ctx, ql, 0.2, None, None, 0, chunk=12, slopes=sl)
        b = ops.paged_window_attention(qa.to(dev), k1.to(dev), v1.to(dev), *on(table, ctx, ql), 0.2, None, None, 0, chunk=12, slopes=sl.to(dev))
        assert torch.allclose(a.float() * live, b.float().cpu() * live, atol=tol)
        # gate on the strided operand; identity experts; gated experts of sizes the tensor-core path does not take; the router
        gt, ot = rn(50, 24).to(dt), rn(50, 100).to(dt)
        assert torch.allclose(ref.gated_act_mul(gt, ot[:, 24:48], "sigmoid", True).float(),
                              ops.gated_act_mul(gt.to(dev), ot.to(dev)[:, 24:48], "sigmoid", True).float().cpu(), atol=tol)
        for (N, Hh, I, E, k, ident) in ((200, 72, 40, 6, 3, 2), (5, 72, 40, 6, 2, 1), (300, 128, 64, 8, 3, 0), (1, 64, 48, 4, 4, 3)):
            xx, wu, wd = rn(N, Hh).to(dt), (rn(E, 2 * I, Hh) * Hh ** -0.5).to(dt), (rn(E, Hh, I) * I ** -0.5).to(dt)
            corr = rn(E + ident) * 0.1
            tw, ti = ref.moe_route(rn(N, E + ident), k, "softmax", False, False, None, corr, None, 1.5)
            a = ref.identity_expert_add(ref.moe_experts(xx, wu, wd, tw, ti, "silu_mul"), xx, tw, ti, E)
            b = ops.identity_expert_add(ops.moe_experts(*on(xx, wu, wd, tw, ti), "silu_mul"), *on(xx, tw, ti), E)
            assert torch.allclose(a.float(), b.float().cpu(), atol=1e-4 if dt == torch.float32 else 6e-2), (N, Hh, I, E, k)
        for (N, Wd, E, k, groups) in ((37, 72, 12, 3, (4, 2)), (1, 200, 33, 33, None), (300, 256, 64, 4, (8, 3)), (9, 64, 6, 2, (6, 2))):
            xx, wr, corr = rn(N, Wd).to(dt), rn(E, Wd) * Wd ** -0.5 * 3, rn(E) * 0.1
            lg, tw, ti = ops.router_topk(*on(xx, wr), k, "softmax", False, False, None, corr.to(dev), groups, 2.5)
            want_lg = xx.double() @ wr.double().T
            r = dict(experts=E, top=k, scale=2.5)
            if groups:
                r["groups"] = dict(count=groups[0], keep=groups[1])
            wo, io = oracle.route(want_lg, corr.double(), r)
            assert torch.allclose(lg.double().cpu(), want_lg, atol=1e-4) and torch.equal(ti.cpu().long().sort(-1).values, io.sort(-1).values)
            assert torch.allclose(tw.double().cpu().sum(-1), wo.sum(-1), atol=1e-5)
    assert ops.stats["moe_plain_gated"] > 0 and ops.stats["router_topk"] > 0 and ops.stats["stream_norm_conv"] > 0
    # bf16 portions of 16+ tokens on the tensor-core kernel: latent rows with a tail (one tile serves keys and values), chunks and slopes
    for (D, Dv, prefix) in ((192, 128, True), (80, 64, True), (64, 64, False), (128, 64, False)):
        B, T, H, page = 2, 150, 6, 16
        G = 1 if prefix else 2
        ctx, ql = torch.tensor([0, 70]).int(), torch.tensor([150, 93]).int()
        nblk = 11
        table = torch.randperm(B * nblk, generator=g).view(B, nblk).int()
        kc, q = (rn(B * nblk, page, G, D) * 0.5).bfloat16(), (rn(B, T, H, D) * 0.3).bfloat16()
        vc = kc if prefix else (rn(B * nblk, page, G, Dv) * 0.5).bfloat16()
        sl = None if prefix else torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])
        kw = dict(value_dim=Dv) if prefix else dict(chunk=48, slopes=sl)
        a = ref.paged_window_attention(q.float(), kc.float(), vc.float(), table, ctx, ql, 0.2, None, 37 if prefix else None, 0, **kw)
        kd = kc.to(dev)
        kw = dict(value_dim=Dv) if prefix else dict(chunk=48, slopes=sl.to(dev))
        b = ops.paged_window_attention(q.to(dev), kd, kd if prefix else vc.to(dev), *on(table, ctx, ql), 0.2, None, 37 if prefix else None, 0, **kw)
        live = (torch.arange(T).view(1, T) < ql.view(B, 1)).unsqueeze(-1)
        assert torch.allclose(a * live, b.float().cpu() * live, atol=3e-2), (D, Dv)
