"""Mukenex through the engine against the plain implementation (``plain_mukenex.py``), in float32 and bfloat16.

Mechanisms alone (kernels against the plain functions, and one-mixer models), whole prompts against token-by-token
decoding, portions down to two tokens, batches of unequal requests against each alone, pages and state slots that
are freed and used again, keys that stand out just inside and just outside a window's and a block's edge, far keys,
long decoding, greedy generation through the scheduler, and trace replay through ``bin/trace_run``.
"""
import math

import numpy as np
import pytest
import torch

import mukenex_kit as M
import plain_mukenex as P

pytestmark = pytest.mark.gpu

PORTIONS = [2, 37, 3, 16, 64, 5, 1, 22]


def cut(total, sizes):
    out, k = [], 0
    while total > 0:
        n = min(total, sizes[k % len(sizes)])
        out.append(n)
        total -= n
        k += 1
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, weights, folder stored in bfloat16)."""
    out = {}
    named = dict(M.CONFIGS, latent=M.ONLY_LATENT, blocks=M.ONLY_BLOCKS, lightning=M.ONLY_LIGHTNING)
    for i, (name, raw) in enumerate(named.items()):
        w = M.random_weights(raw, 200 + i)
        out[name] = (raw, w, M.write_model(str(tmp_path_factory.mktemp("mukenex_" + name)), raw, w))
    return out


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("S", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("width", [44, 264])
def test_streams_write_back_read_and_norm_in_one_kernel(S, width):
    """Three sublayers in a row on S streams against the equations, then the last read (the sum of the streams, chosen
    rows, nothing stored); the outputs arrive in float32 and in bfloat16."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(S * 1000 + width)
    T, eps = 9, 1e-5
    e = torch.randn(T, width, generator=g, dtype=torch.float64) * 2
    coefs = [(torch.randn(S, generator=g, dtype=torch.float64), torch.randn(S, generator=g, dtype=torch.float64),
              torch.randn(S, S, generator=g, dtype=torch.float64)) for _ in range(3)]
    ws = [0.3 * torch.randn(width, generator=g, dtype=torch.float64) for _ in range(4)]
    ys = [torch.randn(T, width, generator=g, dtype=torch.float64) for _ in range(3)]
    ys[1] = ys[1].to(torch.bfloat16).double()
    X = [e.clone() for _ in range(S)]
    streams = torch.full((T, S, width), 9.0, device=dev)                     # stale values
    packed = [torch.cat([c.reshape(-1) for c in cf]).float().to(dev) for cf in coefs]
    before = None
    for q in range(3):
        cin, cout, cmix = coefs[q]
        want = P.rms_norm(sum(cin[s] * X[s] for s in range(S)), ws[q], eps, one_plus=True)
        y_prev = None if q == 0 else (ys[q - 1].to(torch.bfloat16 if q == 2 else torch.float32).to(dev))
        got = ops.stream_step(streams, ws[q].float().to(dev), 1.0, eps, torch.float32,
                              start=e.float().to(dev) if q == 0 else None, y=y_prev, before=before,
                              read_in=packed[q][:S])
        torch.testing.assert_close(got.cpu().double(), want, rtol=2e-5, atol=2e-5)
        X = [sum(cmix[s, t] * X[s] for s in range(S)) + cout[t] * ys[q] for t in range(S)]
        before = packed[q]
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=dev)
    kept = streams.clone()
    want = P.rms_norm(sum(X), ws[3], eps, one_plus=True)[[7, 0, 3]]
    got = ops.stream_step(streams, ws[3].float().to(dev), 1.0, eps, torch.bfloat16, y=ys[2].float().to(dev),
                          before=before, rows=rows, store=False)
    assert torch.equal(streams, kept)
    torch.testing.assert_close(got.cpu().double(), want, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width,ff,experts,top", [(1, 40, 24, 5, 2), (70, 44, 20, 4, 1), (300, 64, 48, 3, 3),
                                                         (130, 248, 88, 12, 2), (700, 192, 136, 9, 2)])
def test_experts_chosen_by_a_table(tokens, width, ff, experts, top, dtype):
    """Few and many pairs (the second take the tcgen05 products in bfloat16), experts with many, few and no tokens."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(tokens + top)
    vocab = 37
    w = {}
    for e in range(experts):
        w[f"e{e}.gate"] = M.bf16_values(torch.randn(ff, width, generator=g) * width ** -0.5)
        w[f"e{e}.up"] = M.bf16_values(torch.randn(ff, width, generator=g) * width ** -0.5)
        w[f"e{e}.down"] = M.bf16_values(torch.randn(width, ff, generator=g) * ff ** -0.5)
    w["table"] = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(vocab)]).to(torch.int32)
    ids = torch.randint(0, vocab, (tokens,), generator=g)
    ids[: min(tokens, 40)] = ids[0]                               # many tokens on the same experts, others on few
    x = M.bf16_values(torch.randn(tokens, width, generator=g))
    want = P.table_experts(x.double(), ids.tolist(), {n: t.double() if t.is_floating_point() else t for n, t in w.items()},
                           "", top)
    gate_up = torch.cat([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]).view(experts, 2 * ff, width)
    down = torch.cat([w[f"e{e}.down"] for e in range(experts)]).view(experts, width, ff)
    got = ops.table_experts(x.to(dev, dtype), ids.to(dev, torch.int32), w["table"].to(dev),
                            gate_up.to(dev, dtype).contiguous(), down.to(dev, dtype).contiguous())
    assert got.dtype == torch.float32
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(got.cpu().double(), want, rtol=tol, atol=tol)
    if dtype == torch.bfloat16 and width % 8 == 0 and ff % 8 == 0 and tokens > 1:
        for tensor_memory in (True, False):                       # both kinds of product on the same step
            again = ops.table_experts(x.to(dev, dtype), ids.to(dev, torch.int32), w["table"].to(dev),
                                      gate_up.to(dev, dtype).contiguous(), down.to(dev, dtype).contiguous(),
                                      tensor_memory=tensor_memory)
            torch.testing.assert_close(again.cpu().double(), want, rtol=tol, atol=tol)
        ops.check_errors(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [70, 72])            # rows of odd size, and rows of whole 16-byte pieces (eight a thread)
def test_activations_joint_norm_with_gate_and_cap(dtype, width):
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(2)
    z = (torch.randn(5, width, generator=g) * 3).to(dtype)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    zd = z.double()
    tanh_form = 0.5 * zd * (1 + torch.tanh(math.sqrt(2 / math.pi) * (zd + 0.044715 * zd ** 3)))
    for act, want in (("silu", P.silu(zd)), ("gelu_erf", P.gelu_erf(zd)), ("gelu_tanh", tanh_form)):
        torch.testing.assert_close(ops.activate(z.to(dev), act).cpu().double(), want, **tol)
    for columns in (33, 40):                                                  # the first columns only, in place
        part = z.to(dev).clone()
        ops.activate(part, "silu", columns=columns, in_place=True)
        torch.testing.assert_close(part[:, :columns].cpu().double(), P.silu(zd[:, :columns]), **tol)
        assert torch.equal(part[:, columns:].cpu(), z[:, columns:])
    o = torch.randn(5, 30, generator=g) * 4
    wn = 1 + 0.2 * torch.randn(30, generator=g)
    want = P.rms_norm(o.double(), wn.double(), 1e-5, one_plus=False) * P.sigmoid(zd[:, 40:70])
    got = ops.row_norm_gate(o.to(dev), wn.to(dev), z.to(dev), 40, 1e-5)
    torch.testing.assert_close(got.cpu().double(), want, **tol)
    logits = torch.randn(3, 50, generator=g) * 40
    torch.testing.assert_close(ops.tanh_cap(logits.to(dev).clone(), 30.0).cpu().double(),
                               30.0 * torch.tanh(logits.double() / 30.0), rtol=1e-5, atol=1e-5)


def _attend_in_portions(q, k, v, portions, dtype, window, chunk, sinks, scale, page=8):
    """q [T, H, d], k [T, G, d], v [T, G, dv] through the prepare kernel (a plain copy here) and the attention kernels,
    portion by portion, over pages handed out in a scrambled order; the outputs [T, H, dv]."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    pages = -(-T // page)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(5)) + 1
    k_cache = torch.full((pages + 1, G, page, d), 77.0, device=dev, dtype=dtype)        # stale values everywhere
    v_cache = torch.full((pages + 1, G, page, dv), 77.0, device=dev, dtype=dtype)
    table = order.to(torch.int32).reshape(1, -1).to(dev)
    packed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).to(dev, dtype).contiguous()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    out, at = [], 0
    for n in portions:
        pos = list(range(at, at + n))
        slots = i32([int(order[p // page]) * page + p % page for p in pos])
        qo = torch.empty((n, H * d), device=dev, dtype=dtype)
        ops.heads_prepare(packed[at:at + n].contiguous(), qo, k_cache, v_cache, i32(pos), slots, H, G, d, dv)
        o = torch.empty((n, H * dv), device=dev, dtype=dtype)
        args = (table, i32([0, n]), i32([at + n]))
        if n > 1:
            ops.prefill_attention(qo, k_cache, v_cache, o, *args, i32([at]), i32([0]), 1, n, H, G, d, page, window,
                                  scale, v_head_dim=dv, precise_weights=True, chunk=chunk, sinks=sinks)
        else:
            splits = 1 if at <= 40 else (2 if at <= 80 else 3)      # one CTA, a cluster of two, parts merged by a kernel
            need = ops.decode_scratch_floats(1, H, max(d, dv), splits)
            scratch = torch.empty(max(need, 1), device=dev)
            ops.decode_attention(qo, k_cache, v_cache, o, scratch, *args, i32([0]), 1, H, G, d, page, window, scale,
                                 splits, v_head_dim=dv, precise_weights=True, chunk=chunk, sinks=sinks)
        out.append(o.cpu().float().reshape(n, H, dv))
        at += n
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mask,size", [("window", 21), ("window", 8), ("chunk", 24), ("chunk", 5), ("none", 0)])
@pytest.mark.parametrize("d,dv,H,G", [(12, 14, 4, 2), (32, 32, 2, 1)])
def test_keys_that_stand_out_just_inside_and_just_outside_an_edge(mask, size, d, dv, H, G, dtype):
    """For chosen queries, in prompt portions and decoded alone, the key just OUTSIDE the window or block is made to
    fit the query far better than any other (it would take all the weight if it were seen), and for others the
    key just inside, or the very first key of the sequence, or a large sink: against the plain attention."""
    g = torch.Generator().manual_seed(size + d)
    T = 100
    q = M.bf16_values(torch.randn(T, H, d, generator=g))
    k = M.bf16_values(torch.randn(T, G, d, generator=g))
    v = M.bf16_values(torch.randn(T, G, dv, generator=g))
    sinks = torch.tensor([3.0, -2.0, 0.5, 8.0][:H])
    portions = [30, 2, 9, 1, 1, 1, 20, 1, 1, 17] + [1] * 17
    assert sum(portions) == T
    for i in (25, 31, 41, 42, 43, 55, 63, 64, 70, 83, 90, 99):                # in portions and decoded alone
        if mask == "window":
            edge = i - size                                                 # the last key that is NOT seen
        elif mask == "chunk":
            edge = i - i % size - 1
        else:
            edge = 0
        for j, boost in ((edge, 6.0), (edge + 1, 4.0), (0, 3.0)):
            if 0 <= j <= i:
                k[j, :, :] = M.bf16_values(boost * q[i, 0:1, :] / q[i, 0].norm() * 2.0)
    window, chunk = (size if mask == "window" else None), (size if mask == "chunk" else None)
    visible = P.window_mask(T, size) if mask == "window" else (P.chunk_mask(T, size) if mask == "chunk" else P.window_mask(T, T))
    rep = H // G
    want = P.masked_softmax_attention(q.double(), k.double().repeat_interleave(rep, 1), v.double().repeat_interleave(rep, 1),
                                      0.7, visible, sink=sinks.double())
    got = _attend_in_portions(q, k, v, portions, dtype, window, chunk, sinks.cuda(), 0.7)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(got.double(), want, rtol=tol, atol=tol)
    no_sink = _attend_in_portions(q, k, v, [T], dtype, window, chunk, None, 0.7)
    want = P.masked_softmax_attention(q.double(), k.double().repeat_interleave(rep, 1), v.double().repeat_interleave(rep, 1),
                                      0.7, visible)
    torch.testing.assert_close(no_sink.double(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv", [(5, 96, 80), (3, 14, 10), (32, 320, 256), (40, 96, 48), (4, 448, 384)])
def test_values_that_are_columns_of_the_key_rows(H, dk, dv, dtype):
    """One row a token that is every head's key and whose first columns are its value (a latent): no value cache.
    Widths that take the all-sizes kernel and widths that take the tensor-core kernels (one and several column tiles
    of the values, more heads than one CTA serves), a window, sinks, prompt portions and decoded tokens."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(H + dk)
    T, page, window, scale = 150, 16, 37, 1.0 / math.sqrt(dk)
    q = M.bf16_values(torch.randn(T, H, dk, generator=g))
    k = M.bf16_values(torch.randn(T, 1, dk, generator=g))
    sinks = torch.randn(H, generator=g)
    for i in (60, 100, 149):                                                  # a key at the window's edges that fits the query
        k[i - window] = M.bf16_values(8.0 * q[i, 0:1] / q[i, 0].norm())
        k[i - window + 1] = M.bf16_values(5.0 * q[i, 0:1] / q[i, 0].norm())
    want = P.masked_softmax_attention(q.double(), k.double().expand(T, H, dk), k.double()[..., :dv].expand(T, H, dv),
                                      scale, P.window_mask(T, window), sink=sinks.double())
    pages = -(-T // page)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(3)) + 1
    k_cache = torch.full((pages + 1, 1, page, dk), 55.0, device=dev, dtype=dtype)
    table = order.to(torch.int32).reshape(1, -1).to(dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    got, at = [], 0
    for n in [70, 2, 33, 1, 1, 1, 20] + [1] * 22:
        for p_ in range(at, at + n):
            k_cache[int(order[p_ // page]), 0, p_ % page] = k[p_, 0].to(dev, dtype)
        qo = q[at:at + n].reshape(n, -1).to(dev, dtype).contiguous()
        o = torch.empty((n, H * dv), device=dev, dtype=dtype)
        args = (table, i32([0, n]), i32([at + n]))
        if n > 1:
            ops.prefill_attention(qo, k_cache, None, o, *args, i32([at]), i32([0]), 1, n, H, 1, dk, page, window, scale,
                                  v_head_dim=dv, precise_weights=True, sinks=sinks.to(dev), shared_values=True)
        else:
            splits = 1 if at <= 110 else (2 if at <= 130 else 3)
            scratch = torch.empty(max(ops.decode_scratch_floats(1, H, dk, splits), 1), device=dev)
            ops.decode_attention(qo, k_cache, None, o, scratch, *args, i32([0]), 1, H, 1, dk, page, window, scale,
                                 splits, v_head_dim=dv, precise_weights=True, sinks=sinks.to(dev), shared_values=True)
        got.append(o.cpu().float().reshape(n, H, dv))
        at += n
    assert at == T
    ops.check_errors(dev)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(torch.cat(got).double(), want, rtol=tol, atol=tol)


# ----------------------------------------------------------------------------- models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M1", "M2", "M3", "M4", "latent", "blocks", "lightning"])
def test_whole_decoded_and_in_portions(name, dtype, models):
    raw, w, folder = models[name]
    T = 150
    ids = M.tokens(raw["vocab"], T, 3)
    want = M.oracle(raw, w, ids)
    eng = M.make_engine(folder, dtype, page_size=8, pool_tokens=256)
    tol = M.tolerance(name, dtype)
    M.check(M.run_alone(eng, 1, ids, [T]), want, dtype, "whole", tol)
    M.check(M.run_alone(eng, 2, ids, [T - 40] + [1] * 40), want, dtype, "last 40 decoded", tol)
    M.check(M.run_alone(eng, 3, ids, cut(T, PORTIONS)), want, dtype, "in portions", tol)
    M.check(M.run_alone(eng, 4, ids[:24], [1] * 24), want[:24], dtype, "token by token from the first", tol)
    M.check(M.run_alone(eng, 5, ids[:61], [2] * 30 + [1]), want[:61], dtype, "two tokens at a time", tol)
    assert eng.cache.manager.check() == ""


def drawn_config(seed):
    """A configuration whose every size, option and layer order is drawn: any model of the design must run as it is."""
    import random
    rng = random.Random(seed)
    even = lambda lo, hi: 2 * rng.randint(lo // 2, hi // 2)

    def feed_forward():
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return M.dense(rng.randint(8, 64))
        experts = rng.randint(2, 6)
        return M.moe(rng.randint(8, 40), experts, rng.randint(1, experts))

    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["latent", "attention", "lightning"])
        if kind == "latent":
            tensor_cores = rng.random() < 0.4                 # widths that the tensor-core kernels take, and others
            rot_dim = rng.choice([16, 32]) if tensor_cores else even(2, 16)
            rank = rng.choice([16, 32, 48]) if tensor_cores else even(4, 40)
            layers.append(M.latent(rng.randint(1, 8), even(4, 24), rot_dim, rng.randint(2, 24), rank,
                                   rng.uniform(0.1, 0.6), rng.randint(3, 70), base=rng.choice([50.0, 1000.0, 20000.0]),
                                   dims=even(2, rot_dim), mlp=feed_forward()))
        elif kind == "attention":
            kv = rng.randint(1, 3)
            dim = rng.choice([16, 32]) if rng.random() < 0.4 else even(4, 40)
            vdim = dim if rng.random() < 0.5 else even(4, 40)
            layers.append(M.attention(kv * rng.randint(1, 4), kv, dim, vdim, rng.uniform(0.1, 0.6), rng.randint(3, 70),
                                      mlp=feed_forward()))
        else:
            heads = rng.randint(1, 3)
            layers.append(M.lightning(heads, even(4, 40), even(4, 40), [rng.uniform(0.5, 0.999) for _ in range(heads)],
                                      mlp=feed_forward()))
    loop = None
    if rng.random() < 0.6:
        start = rng.randint(0, len(layers) - 1)
        loop = (start, rng.randint(start, len(layers)), rng.randint(1, 3))
    return M.config(rng.randint(50, 300), even(24, 96), rng.choice([1e-5, 1e-6, 3e-4]), layers,
                    streams=rng.choice([None, 1, 2, 3, 4, 5]), loop=loop, softcap=rng.choice([None, 8.0, 40.0]))


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(seed, tmp_path):
    raw = drawn_config(seed)
    w = M.random_weights(raw, 300 + seed)
    folder = M.write_model(str(tmp_path / "m"), raw, w)
    T = 90
    ids = M.tokens(raw["vocab"], T, seed)
    want = M.oracle(raw, w, ids)
    for dtype in ("float32", "bfloat16"):
        eng = M.make_engine(folder, dtype, page_size=(4, 8, 16)[seed % 3], pool_tokens=256)
        M.check(M.run_alone(eng, 1, ids, [T]), want, dtype, f"{seed} whole")
        M.check(M.run_alone(eng, 2, ids, [T - 30] + [1] * 30), want, dtype, f"{seed} last 30 decoded")
        M.check(M.run_alone(eng, 3, ids, cut(T, [2, 17, 3, 40, 1, 5])), want, dtype, f"{seed} in portions")
        assert eng.cache.manager.check() == ""
        del eng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_with_sharp_scores_and_slow_decays(dtype, models):
    """Prompts of hundreds of tokens over many pages; scores so sharp that the best key inside the window or block,
    wherever it lies, takes nearly all of a position's weight, and decays so slow that the first tokens still count
    at the end."""
    for name in ("latent", "blocks", "lightning"):
        raw, w, folder = models[name]
        T = 500
        ids = M.tokens(raw["vocab"], T, 11)
        want = M.oracle(raw, w, ids)
        eng = M.make_engine(folder, dtype, page_size=16, pool_tokens=512)
        tol = M.tolerance(name, dtype)
        M.check(M.run_alone(eng, 1, ids, [T]), want, dtype, name + " whole", tol)
        M.check(M.run_alone(eng, 2, ids, [T - 70, 37, 2] + [1] * 31), want, dtype, name + " tail decoded", tol)
        M.check(M.run_alone(eng, 3, ids, cut(T, [127, 2, 16, 129, 15, 1 + 16 * 7])), want, dtype, name + " in portions", tol)
        del eng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M1", "M3"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype, models):
    """Up to three live requests of unequal length in a pool that holds far less than all of them, two state slots
    fewer than requests: portions of some beside decoded tokens of others, and every position's logits as alone."""
    from llm_infer_rust_b200.engine import StepEntry
    from replay_driver import mixed_schedule
    raw, w, folder = models[name]
    lengths = {"a": 90, "b": 37, "c": 120, "d": 5, "e": 64, "f": 101}
    reqs = {r: (M.tokens(raw["vocab"], n, 20 + i), max(2, n - 12 - i)) for i, (r, n) in enumerate(lengths.items())}
    want = {r: M.oracle(raw, w, ids) for r, (ids, _) in reqs.items()}
    eng = M.make_engine(folder, dtype, page_size=8, pool_tokens=320, max_requests=3)
    got = {r: [] for r in reqs}
    number = {r: i + 1 for i, r in enumerate(reqs)}
    opened = set()
    for entries, end in mixed_schedule(reqs, 320, seed=4, max_live=3):
        batch = []
        for r, toks, wanted in entries:
            if r not in opened:
                eng.open_request(number[r])
                opened.add(r)
            batch.append(StepEntry(number[r], list(toks), list(wanted)))
        logits = eng.step(batch).cpu().numpy()
        at = 0
        for r, toks, _ in entries:
            got[r].append(logits[at:at + len(toks)].copy())
            at += len(toks)
        for r in end:
            eng.close_request(number[r])
        assert eng.cache.manager.check() == ""
    eng.check_kernel_errors()
    for r in reqs:
        M.check(np.concatenate(got[r]), want[r], dtype, f"request {r} in mixed batches")


def test_a_slot_that_is_used_again_starts_from_nothing(models):
    """One state slot: the second request gets the slot (and the pages) that the first one left full."""
    raw, w, folder = models["M1"]
    eng = M.make_engine(folder, "float32", page_size=4, pool_tokens=64, max_requests=1)
    first, second = M.tokens(raw["vocab"], 50, 1), M.tokens(raw["vocab"], 33, 2)
    M.check(M.run_alone(eng, 1, first, [20, 30]), M.oracle(raw, w, first), "float32", "first user of the slot")
    M.check(M.run_alone(eng, 2, second, [1, 1, 31]), M.oracle(raw, w, second), "float32", "second user of the slot")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, models):
    raw, w, folder = models["M1"]
    ids = M.tokens(raw["vocab"], 260, 8)
    eng = M.make_engine(folder, dtype, page_size=16, pool_tokens=320)
    M.check(M.run_alone(eng, 1, ids, [6] + [1] * 254), M.oracle(raw, w, ids), dtype, "254 tokens decoded one by one")


@pytest.mark.parametrize("dtype,graphs,portion_graphs", [("float32", 0, 0), ("bfloat16", 0, 0), ("bfloat16", 4, 0),
                                                         ("bfloat16", 4, 64)])
def test_greedy_generation_through_the_scheduler(dtype, graphs, portion_graphs, models):
    """``Engine.generate``: prompts cut by the scheduler's token budget, more prompts than state slots, decode
    graphs in bfloat16, and graphs of prompt portions whose shape comes again.  float32: the tokens are the plain
    implementation's; bfloat16: every generated token is one whose plain logit is within a small margin of the best."""
    from llm_infer_rust_b200 import SamplingParams
    raw, w, folder = models["M3"]
    prompts = [M.tokens(raw["vocab"], n, 40 + n) for n in (5, 23, 1, 12, 30, 64, 50)]
    eng = M.make_engine(folder, dtype, page_size=8, pool_tokens=512, max_requests=3, cuda_graph_bs=graphs,
                        chunked_prefill_size=16, max_prefill_tokens_per_batch=16,
                        prefill_cuda_graph_max_tokens=portion_graphs)
    results = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    eng.check_kernel_errors()
    for prompt, res in zip(prompts, results):
        assert len(res.tokens) == 12
        logits = M.oracle(raw, w, prompt + res.tokens)
        for i, tok in enumerate(res.tokens):
            row = logits[len(prompt) - 1 + i]
            margin = 1e-4 if dtype == "float32" else 0.05 * max(1.0, np.abs(row).max())
            assert row[tok] >= row.max() - margin, f"token {i} of a prompt of {len(prompt)}: {tok} is not the best"


def test_trace_replay_as_a_user_runs_it(models, tmp_path):
    from replay_driver import Replay, run_alone
    raw, w, folder = models["M2"]
    ids = M.tokens(raw["vocab"], 70, 9)
    want = M.oracle(raw, w, ids)
    for dtype in ("bfloat16", "float32"):
        rp = Replay(folder, dtype, 128, str(tmp_path / dtype), raw["vocab"], ["--page-size", "8"])
        try:
            M.check(run_alone(rp, "x", ids, [33, 2, 3] + [1] * 32), want, dtype, "replay")
        finally:
            assert rp.close() == 0


def test_command_line_random_weights_mode(tmp_path):
    """The command line writes a random Mukenex model from a configuration and serves it; the same folder through
    ``Engine.generate`` gives the same tokens."""
    import json
    import os
    import subprocess
    import sys
    from llm_infer_rust_b200 import SamplingParams
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(M.CONFIGS["M1"]))
    made = tmp_path / "made"
    cmd = [sys.executable, "-m", "llm_infer_rust_b200", "--model-path", str(made), "--random-weights", "--config",
           str(cfg), "--seed", "5", "--dtype", "float32", "--page-size", "4", "--max-total-tokens", "256",
           "--max-running-req", "2", "--max-seq-len", "64", "--cuda-graph-bs", "0", "--prompt-ids", "1,2,3",
           "--prompt-ids", "9,8,7,6,5", "--max-tokens", "6", "--ignore-eos"]
    done = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    lines = [json.loads(x) for x in done.stdout.strip().splitlines()]
    assert sorted(os.listdir(made)) == ["config.json", "model.safetensors"]
    eng = M.make_engine(str(made), "float32", page_size=4, pool_tokens=256, max_requests=2)
    want = eng.generate([[1, 2, 3], [9, 8, 7, 6, 5]], SamplingParams(max_tokens=6, ignore_eos=True))
    assert [x["output_ids"] for x in lines] == [r.tokens for r in want]
    eng.check_kernel_errors()
