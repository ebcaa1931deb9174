"""Zanivik through the engine (loader, paged cache, state lines, ragged batches, scheduler) against the plain definition in
``zanivik_oracle.py``.  Every test makes its own small configuration and random checkpoint; the CPU tests run the PyTorch
definitions of the ops in float32, the ``gpu`` tests the sm_100a kernels in float32 and bfloat16."""
import json
import os

import pytest
import torch

import zanivik_oracle as oracle

PAGE = 8
SCALING = dict(factor=3.0, low=1.0, high=5.0, original=60)


def left_a(heads=4, kv_heads=2, dim=12, vdim=6, rot=8, window=9, scale=0.3, base=50.0, scaling=SCALING):
    rot_cfg = dict(base=base, dims=rot)
    if scaling:
        rot_cfg["scaling"] = dict(scaling)
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=rot_cfg)
    if window:
        m["mask"] = dict(size=window)
    return m


def right_a(heads=6, kv_heads=3, dim=8, vdim=10, conv=3):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


def left_b(heads=6, kv_heads=2, dim=10, rot=10, window=7, scale=0.25, base=200.0, scaling=None):
    m = left_a(heads, kv_heads, dim, dim, rot, window, scale, base, scaling)
    return m


def right_b(heads=4, vdim=6, state=10, groups=2, norm_groups=3, conv=4):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)


def pair_a(left=None, right=None, ls=0.7, rs=1.3, ff=40):
    return dict(type="parallel", mixer=dict(left=left or left_a(), right=right or right_a(), left_scale=ls, right_scale=rs),
                mlp=dict(kind="dense", ff=ff) if ff else None)


def pair_b(left=None, right=None, ff=24):
    return dict(type="parallel_2", mixer=dict(left=left or left_b(), right=right or right_b()), mlp=dict(kind="dense", ff=ff) if ff else None)


def make_config(layers, width=36, vocab=83, eps=1e-4, mult=0.6):
    return dict(architecture="Zanivik", layers=layers, norm=dict(eps=eps), residual_mult=mult, vocab=vocab, width=width)


STACK = [pair_a(), pair_b(), pair_b(left_b(heads=2, kv_heads=1, dim=16, rot=6, window=12, scaling=SCALING), right_b(heads=6, vdim=4, state=6, groups=3, norm_groups=1, conv=2), ff=0),
         pair_a(left_a(heads=3, kv_heads=3, dim=8, vdim=14, rot=8, window=5, scaling=None), right_a(heads=2, kv_heads=1, dim=12, vdim=6, conv=4), ls=1.0, rs=0.4)]


def make_weights(cfg, seed=0):
    """Random checkpoint in the design's tensor names (bf16-representable values), every part large enough to matter."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=1.0, mean=0.0: (torch.randn(*s, generator=g) * std + mean).bfloat16().float()       # noqa: E731
    W, V, w = cfg["width"], cfg["vocab"], {}
    w["embed"], w["head"], w["final.norm"] = r(V, W, std=0.5), r(V, W, std=W ** -0.5 * 3), r(W, std=0.2, mean=1.0)
    for i, L in enumerate(cfg["layers"]):
        a = f"l{i}."
        for n in ("norm1", "norm1b"):
            w[a + n] = r(W, std=0.2, mean=1.0)
        w[a + "ls1"] = r(W, std=0.3, mean=0.8)
        l, rt = L["mixer"]["left"], L["mixer"]["right"]
        p, q = a + "mix.left.", a + "mix.right."
        H, G, d = l["heads"], l["kv_heads"], l["dim"]
        w[p + "q"], w[p + "k"] = r(H * d, W, std=W ** -0.5 * 2), r(G * d, W, std=W ** -0.5 * 2)
        if L["type"] == "parallel":
            dv = l["vdim"]
            w[p + "v"], w[p + "g"], w[p + "sink"] = r(G * dv, W, std=W ** -0.5 * 2), r(H * dv, W, std=W ** -0.5 * 2), r(H, std=1.5)
            w[p + "o"] = r(W, H * dv, std=(H * dv) ** -0.5)
            Hr, Gr, D, Dv, K = rt["heads"], rt["kv_heads"], rt["dim"], rt["vdim"], rt["conv"]
            for n, rows in (("q", Gr * D), ("k", Gr * D), ("v", Hr * Dv)):
                w[q + n], w[q + n + ".conv"] = r(rows, W, std=W ** -0.5 * 2), r(rows, K, std=0.6)
            w[q + "b"], w[q + "a"], w[q + "g"] = r(Hr, W, std=W ** -0.5 * 2), r(Hr, W, std=W ** -0.5 * 2), r(Hr * Dv, W, std=W ** -0.5 * 2)
            w[q + "A_log"], w[q + "dt_bias"], w[q + "norm"] = r(Hr, std=0.5, mean=-1.0), r(Hr, std=0.5), r(Dv, std=0.3, mean=1.0)
            w[q + "o"] = r(W, Hr * Dv, std=(Hr * Dv) ** -0.5)
        else:
            w[p + "q.norm"], w[p + "k.norm"], w[p + "temp"] = r(d, std=0.3, mean=1.0), r(d, std=0.3, mean=1.0), r(H, std=0.4, mean=1.2)
            w[p + "o"], w[p + "out"] = r(W, H * d, std=(H * d) ** -0.5), r(W, std=0.3, mean=1.0)
            Hr, P, N, Gr, K = rt["heads"], rt["vdim"], rt["state"], rt["groups"], rt["conv"]
            I, cd = Hr * P, Hr * P + 2 * Gr * N
            w[q + "in"], w[q + "conv"], w[q + "conv.b"] = r(2 * I + 2 * Gr * N + Hr, W, std=W ** -0.5 * 2), r(cd, K, std=0.6), r(cd, std=0.2)
            w[q + "dt_bias"], w[q + "A_log"], w[q + "D"] = r(Hr, std=0.5), r(Hr, std=0.5, mean=-0.5), r(Hr, std=0.5, mean=1.0)
            w[q + "norm"], w[q + "o"], w[q + "out"] = r(I, std=0.3, mean=1.0), r(W, I, std=I ** -0.5), r(W, std=0.3, mean=1.0)
        f = L["mlp"]
        if f is not None:
            for n in ("norm2", "norm2b"):
                w[a + n] = r(W, std=0.2, mean=1.0)
            w[a + "ls2"] = r(W, std=0.3, mean=0.8)
            w[a + "mlp.up"], w[a + "mlp.down"] = r(f["ff"], W, std=W ** -0.5 * 2), r(W, f["ff"], std=f["ff"] ** -0.5)
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
    """float32: the whole block within a tight relative error.  bfloat16: in stacks this narrow a norm over a handful of channels or a
    peaked softmax can magnify the rounding of single positions, so positions are assessed one by one: the typical one within the
    tolerance, few beyond three times that."""
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
    # most of the prompt at once, the rest token by token (slot and pages of the released request are used again): windows pass over
    # decoded tokens, their edges fall on decoded positions, the recurrent states go on from where the prompt left them
    dec = feed(eng, "dec", toks, [T - 25] + list(range(T - 24, T)))
    assert close(dec, want, dtype) and close(dec[-25:], want[-25:], dtype)
    eng.release("dec")
    # token by token from the first token on
    one = feed(eng, "one", toks[:24], range(1, 24))
    assert close(one, want[:24], dtype) and close(one[:3], want[:3], dtype)
    eng.release("one")
    # portions of changing size, down to two tokens and across page and window borders
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
    else:
        assert close(torch.cat([torch.cat(x, 0) for x in got], 0), torch.cat(want, 0), dtype)
    for i in range(n_req):          # a request's rows do not depend on its neighbours: the same request fed alone
        alone = feed(eng, ("alone", i), reqs[i], [])
        eng.release(("alone", i))
        e = (torch.cat(got[i], 0).double() - alone.double()).norm(dim=-1) / want[i].norm(dim=-1)
        assert float(e.median()) < TOL[dtype] / 2 and float((e > 3 * TOL[dtype]).double().mean()) <= 0.1, i


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
    # one pair of the first kind alone: one head everywhere, every channel rotated, no window, no feed-forward, multiplier and scales of one
    ([pair_a(left_a(heads=1, kv_heads=1, dim=4, vdim=4, rot=4, window=None, scaling=None), right_a(heads=1, kv_heads=1, dim=4, vdim=4, conv=1), ls=1.0, rs=1.0, ff=0)],
     dict(mult=1.0, width=20, vocab=31)),
    # one pair of the second kind alone: one kv head and one group for all heads, one norm group, a window of one token, nothing rotated
    ([pair_b(left_b(heads=4, kv_heads=1, dim=6, rot=0, window=1), right_b(heads=2, vdim=8, state=4, groups=1, norm_groups=1, conv=2), ff=12)], dict(width=28)),
    # sizes that coincide: head, value and state sizes equal, as many kv heads as heads, window of one page, two taps
    ([pair_b(left_b(heads=2, kv_heads=2, dim=8, rot=8, window=PAGE, scaling=SCALING), right_b(heads=2, vdim=8, state=8, groups=2, norm_groups=2, conv=2), ff=32),
      pair_a(left_a(heads=2, kv_heads=2, dim=8, vdim=8, rot=2, window=PAGE), right_a(heads=2, kv_heads=2, dim=8, vdim=8, conv=2), ls=0.5, rs=0.5, ff=32)], dict(width=32, mult=0.25)),
    # the second kind twice in a row before the first, a window longer than the prompts, wide heads next to narrow ones
    ([pair_b(), pair_b(left_b(heads=3, kv_heads=3, dim=20, rot=4, window=200), right_b(heads=8, vdim=2, state=12, groups=4, norm_groups=4, conv=5)),
      pair_a(left_a(heads=8, kv_heads=1, dim=6, vdim=4, rot=6, window=3), right_a(heads=4, kv_heads=2, dim=16, vdim=4, conv=6), ff=0)], dict(width=48, vocab=59, eps=1e-6)),
]


@pytest.mark.parametrize("layers,kw", OTHER)
def test_other_sizes_and_layouts(tmp_path, layers, kw):
    check_schedules(tmp_path, "cpu", "float32", layers=layers, T=45, seed=5, **kw)


def _model(eng):
    return eng.app.context_encoding_model.model if hasattr(eng.app, "context_encoding_model") else eng.app.model


def test_streams_after_every_layer(tmp_path):
    cfg = make_config(STACK)
    w = make_weights(cfg, 2)
    eng = make_engine(tmp_path, cfg, w)
    toks = list(range(3, 20))
    streams = []
    oracle.forward(cfg, w, toks, streams)
    T = len(toks)
    out = _model(eng)(torch.tensor([toks]), attention_mask=torch.ones(1, T, dtype=torch.int32), position_ids=torch.arange(T).view(1, T),
                      seq_ids=torch.tensor([0]), slot_mapping=torch.arange(T).view(1, T).int(), block_table=torch.arange(4).view(1, 4).int(),
                      computed_context_lens=torch.tensor([0]), capture=True)
    for i, s in enumerate(streams):
        assert torch.allclose(out.captured[f"layers.{i}.out"][0].double(), s, atol=2e-4), i


def test_long_decoding_over_many_pages(tmp_path):
    cfg = make_config(STACK[:2])
    w = make_weights(cfg, 9)
    eng = make_engine(tmp_path, cfg, w)
    toks = torch.randint(0, cfg["vocab"], (90,), generator=torch.Generator().manual_seed(2)).tolist()
    got = feed(eng, "x", toks, range(3, 90))         # 3-token prompt, then 87 single tokens over twelve pages
    assert rel_err(got, oracle.forward(cfg, w, toks)) < TOL["float32"]


def test_cache_pool_smaller_than_all_requests(tmp_path):
    """The pool holds two requests' worth of pages: the third request runs on the pages and the slot the first gave back, and must not
    see what the first left in them (keys, convolution tails, recurrent states)."""
    cfg = make_config(STACK[:3])
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


def test_a_long_lived_state_carries_the_first_tokens_far(tmp_path):
    """Decays close to one: what the first tokens wrote into the recurrent states still shapes the logits hundreds of tokens on, far
    outside every attention window, whether the prompt arrives whole, in portions or token by token."""
    cfg = make_config([pair_a(ff=0), pair_b(ff=0)])
    w = make_weights(cfg, 1)
    w["l0.mix.right.A_log"].fill_(-9.0)
    w["l1.mix.right.A_log"].fill_(-7.0)
    eng = make_engine(tmp_path, cfg, w, max_tokens=1024)
    g = torch.Generator().manual_seed(8)
    toks = torch.randint(0, cfg["vocab"], (260,), generator=g).tolist()
    other = [(toks[0] + 1) % cfg["vocab"], (toks[1] + 7) % cfg["vocab"]] + toks[2:]
    want, moved = oracle.forward(cfg, w, toks), oracle.forward(cfg, w, other)
    assert rel_err(moved[-5:], want[-5:]) > 5e-3                  # the first two tokens matter at the end
    last = list(range(255, 260))
    for cuts in ([], [100, 200], [3] + list(range(230, 260))):
        got = feed(eng, "s", toks, cuts, want=last)
        eng.release("s")
        assert rel_err(got, want[-5:]) < TOL["float32"]


# ---- mechanisms alone: op definitions (CPU) or kernels (GPU) against the plain functions ---------------------------------------
def paged(rows, page, g, spare=3):
    """rows [n, G, C] -> (cache [blocks, page, G, C] on scattered pages, block table [1, blocks])."""
    n, G, C = rows.shape
    nblk = -(-n // page)
    perm = torch.randperm(nblk + spare, generator=g)[:nblk]
    cache = torch.zeros(nblk + spare, page, G, C)
    for j in range(n):
        cache[perm[j // page], j % page] = rows[j]
    return cache, perm.view(1, -1).int()


def loud_key_case(dev, dtype, target, pos, *, window=None, page=4, as_prompt=False, extra=0, sink=None, temp=False):
    """Four heads over two kv heads whose key row ``target`` is made to dominate the query at ``pos`` (one query and one key are scaled
    so that one score stands out).  ``sink``: the same number for every head; ``temp``: a temperature per head.  Returns (op output,
    plain output, the loud row's values per head) for the query at ``pos``."""
    from neuronx_distributed_inference_b200 import ops
    H, G, D, Dv = 4, 2, 8, 6
    g = torch.Generator().manual_seed(target * 131 + pos)
    n = pos + 1 + extra
    k, v, q = torch.randn(n, G, D, generator=g) * 0.1, torch.randn(n, G, Dv, generator=g), torch.randn(n, H, D, generator=g) * 0.1
    if 0 <= target < n:
        k[target] = 3.0
    q[pos] = 3.0
    tm = torch.tensor([0.8, 1.0, 1.3, 0.9]) if temp else None
    sk = torch.full((H,), float(sink)) if sink is not None else None
    want = oracle.window_attention(q[:pos + 1].double(), k[:pos + 1].double(), v[:pos + 1].double(), 0.25, window,
                                   None if sk is None else sk.double(), None if tm is None else tm.double())[pos].reshape(-1)
    kc, table = paged(k, page, torch.Generator().manual_seed(5))
    vc, _ = paged(v, page, torch.Generator().manual_seed(5))
    to = lambda t: t.to(dev, dtype)                                      # noqa: E731
    i32 = lambda *x: torch.tensor(x).int().to(dev)                       # noqa: E731
    kw = dict(sinks=None if sk is None else sk.to(dev), head_scale=None if tm is None else tm.to(dev))
    if as_prompt:
        got = ops.paged_window_attention(to(q.view(1, n, H, D)), to(kc), to(vc), table.to(dev), i32(0), i32(n), 0.25, None, window, 0, **kw)[0, pos]
    else:
        got = ops.paged_window_attention(to(q[pos].view(1, 1, H, D)), to(kc), to(vc), table.to(dev), i32(pos), i32(1), 0.25, None, window, 0, **kw)
    row = v[target].repeat_interleave(H // G, 0).reshape(-1) if 0 <= target < n else None
    return got.float().cpu().view(-1), want.float(), row


# (window, position, loud key, is it visible): far keys, page borders (pages of 4), the first tokens, both sides of every edge
EDGES = [(40, 300, 261, True), (40, 300, 260, False), (40, 39, 0, True), (40, 40, 0, False), (40, 40, 1, True), (1, 9, 9, True), (1, 9, 8, False),
         (4, 8, 5, True), (4, 8, 4, False), (5, 8, 4, True), (5, 8, 3, False), (None, 300, 0, True), (None, 301, 150, True), (None, 0, 0, True),
         (None, 4, 4, True), (None, 8, 7, True), (64, 64, 0, False), (64, 63, 0, True), (64, 64, 1, True)]


@pytest.mark.parametrize("window,pos,target,visible", EDGES)
@pytest.mark.parametrize("as_prompt", [False, True])
def test_loud_keys_at_window_and_page_edges(window, pos, target, visible, as_prompt):
    for temp in (False, True):
        got, want, row = loud_key_case("cpu", torch.float32, target, pos, window=window, as_prompt=as_prompt, temp=temp)
        assert torch.allclose(got, want, atol=1e-5)
        assert torch.allclose(got, row, atol=1e-3) == visible          # the loud row's value is what every head returns exactly when it is visible


def test_a_prompt_does_not_see_later_rows_of_its_portion():
    got, want, row = loud_key_case("cpu", torch.float32, 21, 20, as_prompt=True, extra=3, window=16)       # the loud row is one step ahead
    assert torch.allclose(got, want, atol=1e-5) and not torch.allclose(got, row, atol=0.5)


def test_the_sink_takes_weight_without_a_value():
    """A sink far above every score leaves almost nothing for the keys; one far below changes nothing; it is not multiplied by the scale."""
    none, want0, _ = loud_key_case("cpu", torch.float32, -1, 30, window=12)
    low, want1, _ = loud_key_case("cpu", torch.float32, -1, 30, window=12, sink=-30.0)
    mid, want2, _ = loud_key_case("cpu", torch.float32, -1, 30, window=12, sink=1.0)
    high, want3, _ = loud_key_case("cpu", torch.float32, -1, 30, window=12, sink=30.0)
    for got, want in ((none, want0), (low, want1), (mid, want2), (high, want3)):
        assert torch.allclose(got, want, atol=1e-5)
    assert torch.allclose(low, none, atol=1e-5) and float(high.abs().max()) < 1e-6 and 0.05 < float(mid.norm() / none.norm()) < 0.95


def ragged_case(B=3, T=11):
    return torch.tensor([0, 5, 40]).int(), torch.tensor([T, 4, 1]).int(), torch.tensor([2, 0, 3]).int()


def check_stream_sandwich_norm(dev, dt, tol):
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)        # noqa: E731
    for W in (36, 200, 1024):
        x, a, b = rn(7, W), rn(7, W).to(dt), (rn(7, W) * 3).to(dt)
        aw, bw, pw, ls, nw = rn(W), rn(W), rn(W), rn(W), rn(W)
        eps = 1e-3
        for center in (True, False):
            norm = (lambda v, w_: oracle.layer_norm(v, w_, eps)) if center else (lambda v, w_: oracle.rms_norm(v, eps, w_))
            for pair, scales in ((True, (0.5, 0.5)), (False, (0.7, 1.3)), (None, (1.0, 1.0))):
                ad, bd = a.double(), b.double()
                if pair is True:
                    y = scales[0] * oracle.rms_norm(ad, eps, aw.double()) + scales[1] * oracle.rms_norm(bd, eps, bw.double())
                elif pair is False:
                    y = scales[0] * ad + scales[1] * bd
                else:
                    y = ad
                s_want = x.double() + 0.6 * norm(y, pw.double()) * ls.double()
                h_want = norm(s_want, nw.double())
                on = lambda t: None if t is None else t.to(dev)      # noqa: E731
                s, h = ops.stream_sandwich_norm(on(x), on(a), on(b) if pair is not None else None, on(aw) if pair else None, on(bw) if pair else None,
                                                scales[0], scales[1], on(pw), on(ls), 0.6, on(nw), eps, center, dt)
                assert torch.allclose(s.double().cpu(), s_want, atol=1e-5, rtol=1e-5)
                assert torch.allclose(h.double().cpu(), h_want, atol=tol * 4, rtol=tol)
        s, h = ops.stream_sandwich_norm(x.to(dev), next_weight=nw.to(dev), eps=eps, lp_dtype=dt)          # nothing to add: the norm alone
        assert torch.equal(s.cpu(), x) and torch.allclose(h.double().cpu(), oracle.layer_norm(x.double(), nw.double(), eps), atol=tol * 4, rtol=tol)


def check_head_norm_rope_append(dev, dt, tol):
    """Norm before or after the rotation, weights or none, values from their own slice or from the keys, a rotation of part of a head,
    positions from the context length, rows scattered over pages, strided input rows."""
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(1)
    rn = lambda *s: torch.randn(*s, generator=g)        # noqa: E731
    B, T, page, nblk = 3, 11, 4, 14
    ctx, ql, _ = ragged_case(B, T)
    for (H, G, D, Dv, R, norm_at, with_w, vfk) in ((4, 2, 12, 6, 8, 2, False, False), (6, 2, 10, 10, 10, 1, True, True), (2, 1, 16, 16, 6, 1, True, True),
                                                   (3, 3, 8, 14, 0, 0, False, False), (2, 2, 64, 64, 64, 1, True, True), (1, 1, 40, 20, 24, 2, False, False),
                                                   # head sizes of 64 / 128 / 256 in rows aligned for one vector access per lane
                                                   (2, 1, 128, 64, 64, 2, False, False), (1, 1, 256, 256, 256, 1, True, True), (2, 2, 64, 32, 0, 1, True, False),
                                                   (4, 2, 128, 128, 128, 1, True, True), (2, 2, 64, 24, 32, 2, True, False)):
        C = H * D + G * D + (0 if vfk else G * Dv)
        wide = rn(B, T, C + 16).to(dt)
        p = wide[..., 8:8 + C + 2]
        rot = dict(base=77.0, dims=R, scaling=SCALING)
        qw, kw_ = (rn(D), rn(D)) if with_w else (None, None)
        table = torch.randperm(B * nblk, generator=g).view(B, nblk).int()
        kc, vc = torch.zeros(B * nblk, page, G, D, dtype=dt), torch.zeros(B * nblk, page, G, Dv, dtype=dt)
        cos = sin = None
        if R:
            f = oracle.rotary_frequencies(rot)
            ang = (ctx.double().view(B, 1) + torch.arange(T).double().view(1, T)).unsqueeze(-1) * f
            cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
        on = lambda t: None if t is None else t.to(dev)      # noqa: E731
        kd, vd = kc.to(dev), vc.to(dev)
        q = ops.head_norm_rope_append(on(p), H, G, D, Dv, on(cos), on(sin), on(qw), on(kw_), norm_at, 1e-3, vfk, kd, vd, on(table), on(ctx), on(ql))
        for b in range(B):
            n, c0 = int(ql[b]), int(ctx[b])
            rows = p[b, :n].double()
            qr, kr = rows[:, :H * D].view(n, H, D), rows[:, H * D:H * D + G * D].view(n, G, D)
            vr = kr if vfk else rows[:, H * D + G * D:C].view(n, G, Dv)

            def prep(x, w_):
                if norm_at == 1:
                    x = oracle.rms_norm(x, 1e-3, None if w_ is None else w_.double())
                x = oracle.rotate(x, rot, c0)
                if norm_at == 2:
                    x = oracle.rms_norm(x, 1e-3, None if w_ is None else w_.double())
                return x
            assert torch.allclose(q[b, :n].double().cpu(), prep(qr, qw), atol=tol * 3, rtol=tol)
            for t in range(n):
                pos = c0 + t
                blk = int(table[b, pos // page])
                assert torch.allclose(kd[blk, pos % page].double().cpu(), prep(kr, kw_)[t], atol=tol * 3, rtol=tol)
                assert torch.allclose(vd[blk, pos % page].double().cpu(), vr[t], atol=tol, rtol=tol)


def check_gated_delta(dev, dt, tol):
    """The recurrence against the plain loop: whole rows, and the same rows cut into two calls with the state carried in its line; heads
    that share q / k heads; lines used in another order; decays near one and near zero."""
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(2)
    rn = lambda *s: torch.randn(*s, generator=g)        # noqa: E731
    for (H, G, D, Dv, T) in ((4, 2, 8, 10, 37), (2, 2, 16, 4, 20), (3, 1, 4, 20, 18), (2, 1, 128, 16, 40), (1, 1, 136, 8, 19)):
        B = 2
        C = 2 * G * D + H * Dv
        qkv, beta, a = rn(B, T, C), rn(B, T, H + 3).to(dt)[..., 1:1 + H], (rn(B, T, H) * 2).to(dt)
        A_log, dtb = rn(H) - 1.0, rn(H)
        q = qkv[..., :G * D].double().view(B, T, G, D)
        k = qkv[..., G * D:2 * G * D].double().view(B, T, G, D)
        v = qkv[..., 2 * G * D:].double().view(B, T, H, Dv)
        unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)       # noqa: E731
        qn, kn = (unit(q) * D ** -0.5).repeat_interleave(H // G, 2), unit(k).repeat_interleave(H // G, 2)
        decay = torch.exp(-torch.exp(A_log.double()) * torch.nn.functional.softplus(a.double() + dtb.double(), threshold=1e9))
        want = torch.stack([oracle.gated_delta_rule(qn[b], kn[b], v[b], torch.sigmoid(beta[b].double()), decay[b]) for b in range(B)]).reshape(B, T, H * Dv)
        on = lambda t: t.to(dev)      # noqa: E731
        i32 = lambda *x: torch.tensor(x).int().to(dev)                       # noqa: E731
        state = (rn(5, H, D, Dv) * 9).to(dev)                               # what an earlier request left in the lines
        got = ops.gated_delta_scan(on(qkv), on(beta), on(a), on(A_log), on(dtb), state, i32(3, 1), i32(0, 0), i32(T, T), H, G, D, Dv)
        assert torch.allclose(got.double().cpu(), want, atol=tol, rtol=tol)
        cut = 7
        state2 = (rn(5, H, D, Dv) * 9).to(dev)
        first = ops.gated_delta_scan(on(qkv[:, :cut]), on(beta[:, :cut]), on(a[:, :cut]), on(A_log), on(dtb), state2, i32(0, 4), i32(0, 0), i32(cut, cut - 2), H, G, D, Dv)
        rest0 = ops.gated_delta_scan(on(qkv[:1, cut:]), on(beta[:1, cut:]), on(a[:1, cut:]), on(A_log), on(dtb), state2, i32(0), i32(cut), i32(T - cut), H, G, D, Dv)
        rest1 = ops.gated_delta_scan(on(qkv[1:, cut - 2:]), on(beta[1:, cut - 2:]), on(a[1:, cut - 2:]), on(A_log), on(dtb), state2, i32(4), i32(cut - 2), i32(T - cut + 2), H, G, D, Dv)
        assert torch.allclose(torch.cat([first[0, :cut], rest0[0]], 0).double().cpu(), want[0], atol=tol, rtol=tol)
        assert torch.allclose(torch.cat([first[1, :cut - 2], rest1[0]], 0).double().cpu(), want[1], atol=tol, rtol=tol)
        assert torch.allclose(state2[0].cpu(), state[3].cpu(), atol=tol, rtol=tol) and torch.allclose(state2[4].cpu(), state[1].cpu(), atol=tol, rtol=tol)
        # the per-head norm with a shared weight and the activated gate that follow the recurrence
        wn, gate = rn(Dv), rn(B, T, H * Dv + 5).to(dt)[..., 2:2 + H * Dv]
        o = ops.head_rmsnorm_gate(got, on(wn), H, 1e-3, on(gate), "silu", out_dtype=dt)
        o_want = oracle.rms_norm(got.double().cpu().view(B, T, H, Dv), 1e-3, wn.double()).reshape(B, T, -1) * oracle.silu(gate.double())
        otol = 1e-2 if dt == torch.bfloat16 else 4 * tol          # the result is rounded to the activation type
        assert torch.allclose(o.double().cpu(), o_want, atol=otol, rtol=otol)


def test_stream_norms_sum_and_layer_scale():
    check_stream_sandwich_norm("cpu", torch.float32, 1e-5)


def test_head_norms_rotation_and_cache_rows():
    check_head_norm_rope_append("cpu", torch.float32, 1e-5)


def test_gated_delta_rule_and_its_carried_state():
    check_gated_delta("cpu", torch.float32, 1e-5)


def test_scaled_frequencies_follow_the_three_bands():
    from neuronx_distributed_inference_b200.modules.attention.head_norm_window_attention import HeadNormWindowAttention
    rot = dict(base=50.0, dims=16, scaling=SCALING)
    f = oracle.rotary_frequencies(rot)
    plain = oracle.rotary_frequencies(dict(base=50.0, dims=16))
    ratio = (f / plain).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 3) < 1e-12 and any(1 / 3 + 1e-6 < r < 1 - 1e-6 for r in ratio)      # kept, divided, blended
    m = HeadNormWindowAttention(32, 2, 1, 16, 16, rot_dims=16, rot_base=50.0, rot_scaling=SCALING, scale=1.0, window=None, eps=1e-5, layer_idx=0,
                                dtype=torch.float32)
    assert torch.allclose(m.rope_inv_freq, f, rtol=1e-12, atol=0)


def test_activation_is_the_erf_gelu():
    from neuronx_distributed_inference_b200 import ops
    x = torch.linspace(-6, 6, 101)
    assert torch.allclose(ops.unary_act(x, "gelu").double(), oracle.gelu_erf(x.double()), atol=1e-6)
    assert not torch.allclose(ops.unary_act(x, "gelu_tanh").double(), oracle.gelu_erf(x.double()), atol=1e-4)


def test_registry_picks_the_model_from_config_json(tmp_path):
    from neuronx_distributed_inference_b200.utils.constants import get_model_cls, model_type_of
    with open(tmp_path / "config.json", "w") as f:
        json.dump(make_config(STACK), f)
    assert get_model_cls(model_type_of(str(tmp_path))).__name__ == "NeuronZanivikForCausalLM"


def test_command_line_generates_from_token_ids(tmp_path, capsys):
    from neuronx_distributed_inference_b200 import inference_demo
    cfg = make_config(STACK)
    w = make_weights(cfg)
    eng = make_engine(tmp_path, cfg, w)
    want = eng.generate([[1, 2, 3, 4], [7, 8]], 5)
    inference_demo.main(["--model-type", "zanivik", "--task-type", "causal-lm", "run", "--model-path", str(tmp_path / "ckpt"),
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
    for k in ("stream_sandwich_norm", "head_norm_rope_append", "paged_window_attention", "short_conv", "short_conv_update", "gated_delta_scan",
              "head_rmsnorm_gate", "ssd_scan", "group_rmsnorm", "unary_act"):
        assert ops.stats[k] > 0, k
    tkg = eng.app.token_generation_model          # single-token steps replayed from CUDA graphs (capture did not fall back to eager)
    assert tkg.use_graphs and len(tkg._graphs) > 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpu_wider_stack(tmp_path, dtype):
    """Head sizes of 64 and 128 (tensor-core attention on bf16 portions) beside sizes that take the CUDA-core kernel; recurrent heads
    with 128 and 136 key channels (one and two register blocks per lane)."""
    layers = [pair_a(left_a(heads=4, kv_heads=2, dim=64, vdim=64, rot=32, window=33, scale=0.12), right_a(heads=4, kv_heads=2, dim=128, vdim=32, conv=4), ff=256),
              pair_b(left_b(heads=2, kv_heads=1, dim=128, rot=128, window=40, scale=0.09), right_b(heads=8, vdim=16, state=64, groups=2, norm_groups=2, conv=4), ff=192),
              pair_a(left_a(heads=6, kv_heads=3, dim=48, vdim=24, rot=48, window=20, scale=0.15, scaling=None), right_a(heads=2, kv_heads=1, dim=136, vdim=20, conv=3), ff=0)]
    eng, cfg, w = check_schedules(tmp_path, "cuda", dtype, layers=layers, T=77, width=384, vocab=301, eps=1e-6, seed=7)
    check_mixed_batches(eng, cfg, w, dtype, n_req=5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layers,kw", OTHER)
def test_gpu_other_sizes_and_layouts(tmp_path, dtype, layers, kw):
    check_schedules(tmp_path, "cuda", dtype, layers=layers, T=45, seed=5, **kw)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,pos,target,visible", EDGES)
@pytest.mark.parametrize("as_prompt", [False, True])
def test_gpu_loud_keys_at_window_and_page_edges(window, pos, target, visible, dtype, as_prompt):
    for temp, sink in ((False, None), (True, None), (True, 0.5)):
        got, want, row = loud_key_case("cuda", dtype, target, pos, window=window, as_prompt=as_prompt, temp=temp, sink=sink)
        assert torch.allclose(got, want, atol=1e-4 if dtype == torch.float32 else 3e-2)
        if sink is None:
            assert torch.allclose(got, row, atol=3e-2) == visible


@pytest.mark.gpu
@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1e-2)])
def test_gpu_kernels_match_the_plain_functions(dt, tol):
    check_stream_sandwich_norm("cuda", dt, tol)
    check_head_norm_rope_append("cuda", dt, tol)
    check_gated_delta("cuda", dt, 2e-5 if dt == torch.float32 else 2e-4)          # q / k / v and the state are fp32 in both; beta and a are rounded


@pytest.mark.gpu
def test_gpu_long_lived_state_and_long_decoding(tmp_path):
    cfg = make_config(STACK[:2])
    w = make_weights(cfg, 9)
    w["l0.mix.right.A_log"].fill_(-8.0)
    eng = make_engine(tmp_path, cfg, w, "float32", "cuda")
    toks = torch.randint(0, cfg["vocab"], (150,), generator=torch.Generator().manual_seed(2)).tolist()
    got = feed(eng, "x", toks, range(3, 150))
    assert rel_err(got, oracle.forward(cfg, w, toks)) < TOL["float32"]
