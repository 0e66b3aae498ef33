"""Kefetar through the engine against the plain implementation (``plain_kefetar.py``), in float32 and bfloat16.

Mechanisms alone (kernels against the plain functions, and one-mixer models), whole prompts against token-by-token
decoding, portions down to two tokens, batches of unequal requests against each alone, pages and state slots that
are freed and used again, long prompts with scores so sharp that one far key decides a position, long decoding,
greedy generation through the scheduler, and trace replay through ``bin/trace_run``.
"""
import types

import numpy as np
import pytest
import torch

import kefetar_kit as K
import plain_kefetar as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, weights, folder stored in bfloat16)."""
    out = {}
    named = dict(K.CONFIGS, attention=K.ONLY_ATTENTION, retention=K.ONLY_RETENTION)
    for i, (name, raw) in enumerate(named.items()):
        w = K.random_weights(raw, 100 + i)
        out[name] = (raw, w, K.write_model(str(tmp_path_factory.mktemp("kefetar_" + name)), raw, w))
    return out


def step_ctx(rows, device):
    """The index arrays that the kernels read, for rows of (state slot, prefix length, tokens in this step)."""
    cu, row_of, pos = [0], [], []
    for r, (_, prefix, n) in enumerate(rows):
        cu.append(cu[-1] + n)
        row_of += [r] * n
        pos += list(range(prefix, prefix + n))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return types.SimpleNamespace(num_rows=len(rows), row_of_token=i32(row_of), cu_q=i32(cu), positions=i32(pos),
                                 prefix_len=i32([p for _, p, _ in rows]), state_slots=i32([s for s, _, _ in rows]))


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("C", [70, 72])          # rows of odd size, and rows of whole 16-byte pieces (eight channels a thread)
@pytest.mark.parametrize("taps,identity", [(2, True), (3, True), (4, False), (8, True), (1, True)])
def test_scaled_norm_and_causal_taps_in_portions_with_state(taps, identity, C):
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(taps)
    lengths = [11, 1, 6]
    w = torch.randn(C, taps, generator=g)
    gain = torch.tensor([1.3])
    xs = [torch.randn(n, C, generator=g) * 3 for n in lengths]
    want = []
    for x in xs:
        h = P.scalar_rms_norm(x.double(), gain.double(), 1e-5)
        y = P.causal_taps(h, w.double())
        want.append((h + y) if identity else y)
    state = torch.full((5, taps - 1, C), 7.0, device=dev)                   # stale values in every slot
    fed = [0, 0, 0]
    slots = [3, 1, 4]
    got = [[] for _ in xs]
    # steps: unequal portions of the three sequences side by side, down to single tokens
    for portion in ([2, 1, 1], [1, 0, 2], [5, 0, 1], [3, 0, 2]):
        rows, parts, who = [], [], []
        for r, n in enumerate(portion):
            if n:
                rows.append((slots[r], fed[r], n))
                parts.append(xs[r][fed[r]:fed[r] + n])
                who.append(r)
        ctx = step_ctx(rows, dev)
        x = torch.cat(parts).to(dev).contiguous()
        scale = ops.residual_scale(x, None, gain.to(dev), 1e-5)
        y = ops.causal_taps(x, w.to(dev), state if taps > 1 else None, ctx, torch.float32, scale=scale,
                            identity=identity)
        at = 0
        for r, (_, _, n) in zip(who, rows):
            got[r].append(y[at:at + n].cpu())
            fed[r] += n
            at += n
    for r in range(3):
        assert fed[r] == lengths[r]
        torch.testing.assert_close(torch.cat(got[r]).double(), want[r], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("taps", [1, 3, 5])
def test_add_norm_and_taps_in_one_kernel_for_rows_of_one_token(taps):
    """Three sequences decoded side by side, token by token, through the fused kernel; a fourth step that has a longer
    row is refused by it (None) and the fused steps leave the states as the two kernels would."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(taps)
    C, T = 64, 7
    w, gain = torch.randn(C, taps, generator=g), torch.tensor([0.8])
    xs = torch.randn(3, T, C, generator=g) * 2
    ys = (torch.randn(3, T, C, generator=g)).to(torch.bfloat16)
    state = torch.full((5, max(taps - 1, 0), C), 3.0, device=dev)
    slots = [4, 1, 2]
    got = []
    for t in range(T):
        ctx = step_ctx([(slots[r], t, 1) for r in range(3)], dev)
        ctx.num_prefill = 0
        x = xs[:, t].to(dev).contiguous()
        out = ops.add_norm_taps_single(x, ys[:, t].to(dev).contiguous(), gain.to(dev), 1e-5, w.to(dev),
                                       state if taps > 1 else None, ctx, torch.float32, True)
        assert out is not None
        torch.testing.assert_close(x.cpu(), xs[:, t] + ys[:, t].float())
        got.append(out.cpu())
    got = torch.stack(got, 1)
    for r in range(3):
        h = P.scalar_rms_norm((xs[r] + ys[r].float()).double(), gain.double(), 1e-5)
        torch.testing.assert_close(got[r].double(), P.canon(h, w.double()), rtol=1e-5, atol=1e-5)
    ctx = step_ctx([(1, 0, 2)], dev)
    ctx.num_prefill = 1
    assert ops.add_norm_taps_single(xs[0, :2].to(dev).contiguous(), None, gain.to(dev), 1e-5, w.to(dev),
                                    state if taps > 1 else None, ctx, torch.float32, True) is None


def test_residual_sum_is_taken_in_float():
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    x = torch.full((3, 64), 256.0, device=dev)
    y = torch.full((3, 64), 0.5, dtype=torch.bfloat16, device=dev)        # lost if the sum were rounded to bfloat16
    s = ops.residual_scale(x, y, torch.tensor([2.0], device=dev), 0.0)
    assert torch.all(x == 256.5)
    torch.testing.assert_close(s, torch.full((3,), 2.0 / 256.5, device=dev))


@pytest.mark.parametrize("width", [150, 152, 9000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_poly_norm_and_gates(dtype, width):
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    z = (torch.randn(7, width, generator=g) * 2).to(dtype)
    coef = torch.tensor([0.7, -1.1, 0.4, 0.25])
    got = ops.poly_norm(z.to(dev), coef.to(dev), 1e-5).float().cpu()
    want = P.poly_norm(z.double(), coef.double(), 1e-5).float()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(got, want, rtol=tol, atol=tol)
    # unit norm per head times silu(gate), the gate read from the columns of a wider matrix
    heads, dv = 3, 20
    o = torch.randn(7, heads * dv, generator=g) * 5
    packed = torch.randn(7, 11 + heads * dv, generator=g).to(dtype)
    got = ops.head_unit_norm_gate(o.to(dev), packed.to(dev), 11, heads, dv, 1e-5).float().cpu()
    gate = packed[:, 11:].double()
    want = (P.unit_rms(o.double().view(7, heads, dv), 1e-5).reshape(7, -1) * gate * torch.sigmoid(gate)).float()
    torch.testing.assert_close(got, want, rtol=tol, atol=tol)
    a = torch.randn(7, 33, generator=g).to(dtype)
    packed = torch.randn(7, 40, generator=g).to(dtype)
    got = ops.sigmoid_gate_mul(a.to(dev).clone(), packed.to(dev), 7).float().cpu()
    want = (a.double() * torch.sigmoid(packed[:, 7:].double())).float()
    torch.testing.assert_close(got, want, rtol=tol, atol=tol)


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("heads,d,dv,rot", [(2, 8, 16, 4), (1, 24, 40, 24), (3, 100, 36, 0), (2, 128, 128, 64), (1, 320, 72, 32)])
def test_retention_kernel_against_the_recurrence_in_portions(heads, d, dv, rot, chunked):
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(d)
    T = 45 if not chunked else 215
    decay = torch.tensor([0.9, 0.999, 0.5][:heads])
    x = torch.randn(T, heads * (2 * d + dv) + 5, generator=g)               # five columns that are not its own
    q = x[:, :heads * d].view(T, heads, d).double()
    k = x[:, heads * d:2 * heads * d].view(T, heads, d).double()
    v = x[:, 2 * heads * d:2 * heads * d + heads * dv].view(T, heads, dv).double()
    inv_freq = None
    if rot:
        q, k = P.rotate_half_split(q, 50.0, rot, 2.0), P.rotate_half_split(k, 50.0, rot, 2.0)
        inv_freq = (torch.pow(torch.tensor(50.0, dtype=torch.float64), -torch.arange(0, rot, 2, dtype=torch.float64) / rot)
                    / 2.0).float().to(dev)
    want, S = P.retention_recurrence(q, k * 0.3, v, decay.double(), return_state=True)
    state = torch.full((4, heads, d, dv), 9.0, device=dev)                  # a slot that was used before
    got, at = [], 0
    for n in ((1, 2, 17, 8, 1, 16) if not chunked else (1, 70, 2, 64, 13, 65)):
        ctx = step_ctx([(2, at, n)], dev)
        got.append(ops.retention(x[at:at + n].to(dev).contiguous(), state, decay.to(dev), inv_freq, rot, 0.3, ctx,
                                 heads, d, dv, chunked=chunked).cpu())
        at += n
    assert at == T
    torch.testing.assert_close(torch.cat(got).double().view(T, heads, dv), want, rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(state[2].cpu().double(), S, rtol=2e-4, atol=2e-4)
    assert torch.all(state[1] == 9.0) and torch.all(state[3] == 9.0)


def test_retention_in_chunks_for_rows_of_unequal_length_side_by_side():
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(9)
    heads, d, dv = 2, 64, 32
    decay = torch.tensor([0.97, 0.999])
    lengths, prefixes = [130, 1, 64, 3], [0, 5, 2, 0]
    state = torch.randn(6, heads, d, dv, generator=g).to(dev)
    start = state.clone()
    xs = [torch.randn(n, heads * (2 * d + dv), generator=g) for n in lengths]
    ctx = step_ctx([(s, p, n) for s, p, n in zip([4, 2, 1, 5], prefixes, lengths)], dev)
    got = ops.retention(torch.cat(xs).to(dev), state, decay.to(dev), None, 0, 0.25, ctx, heads, d, dv, chunked=True).cpu()
    at = 0
    for x, slot, prefix in zip(xs, [4, 2, 1, 5], prefixes):
        T = x.shape[0]
        q = x[:, :heads * d].view(T, heads, d).double()
        k = x[:, heads * d:2 * heads * d].view(T, heads, d).double() * 0.25
        v = x[:, 2 * heads * d:].view(T, heads, dv).double()
        S0 = start[slot].cpu().double() if prefix else None
        want, S = P.retention_recurrence(q, k, v, decay.double(), S0=S0, return_state=True)
        torch.testing.assert_close(got[at:at + T].double().view(T, heads, dv), want, rtol=2e-4, atol=2e-4)
        torch.testing.assert_close(state[slot].cpu().double(), S, rtol=2e-4, atol=2e-4)
        at += T


# ----------------------------------------------------------------------------- models through the engine
PORTIONS = [2, 17, 3, 2, 16, 33, 2, 5, 64, 2, 9, 31]


def cut(total, pattern):
    sizes, left, k = [], total, 0
    while left:
        n = min(pattern[k % len(pattern)], left)
        if left - n == 1:
            n += 1
        sizes.append(n)
        left -= n
        k += 1
    return sizes


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4", "K5", "attention", "retention"])
def test_whole_decoded_and_in_portions(name, dtype, models):
    raw, w, folder = models[name]
    T = 150
    ids = K.tokens(raw["vocab"], T, 3)
    want = K.oracle(raw, w, ids)
    eng = K.make_engine(folder, dtype, page_size=8, pool_tokens=256)
    tol = K.tolerance(name, dtype)
    K.check(K.run_alone(eng, 1, ids, [T]), want, dtype, "whole", tol)
    K.check(K.run_alone(eng, 2, ids, [T - 40] + [1] * 40), want, dtype, "last 40 decoded", tol)
    K.check(K.run_alone(eng, 3, ids, cut(T, PORTIONS)), want, dtype, "in portions", tol)
    K.check(K.run_alone(eng, 4, ids[:24], [1] * 24), want[:24], dtype, "token by token from the first", tol)
    assert eng.cache.manager.check() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_with_sharp_scores_and_slow_decays(dtype, models):
    """Prompts of hundreds of tokens over many pages; scores so sharp (scale 3, cap 30) that the best key, wherever
    it lies, takes nearly all of a position's weight, and decays so slow that the first tokens still count at the end."""
    for name in ("attention", "retention"):
        raw, w, folder = models[name]
        T = 700
        ids = K.tokens(raw["vocab"], T, 11)
        want = K.oracle(raw, w, ids)
        eng = K.make_engine(folder, dtype, page_size=16, pool_tokens=768)
        tol = K.tolerance(name, dtype)
        K.check(K.run_alone(eng, 1, ids, [T]), want, dtype, name + " whole", tol)
        K.check(K.run_alone(eng, 2, ids, [T - 70, 37, 2] + [1] * 31), want, dtype, name + " tail decoded", tol)
        K.check(K.run_alone(eng, 3, ids, cut(T, [127, 2, 16, 129, 15, 1 + 16 * 7])), want, dtype, name + " in portions", tol)
        del eng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K1", "K2"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype, models):
    """Up to three live requests of unequal length in a pool that holds far less than all of them, two state slots
    fewer than requests: portions of some beside decoded tokens of others, and every position's logits as alone."""
    from llm_infer_rust_b200.engine import StepEntry
    from replay_driver import mixed_schedule
    raw, w, folder = models[name]
    lengths = {"a": 90, "b": 37, "c": 120, "d": 5, "e": 64, "f": 101}
    reqs = {r: (K.tokens(raw["vocab"], n, 20 + i), max(2, n - 12 - i)) for i, (r, n) in enumerate(lengths.items())}
    want = {r: K.oracle(raw, w, ids) for r, (ids, _) in reqs.items()}
    eng = K.make_engine(folder, dtype, page_size=8, pool_tokens=320, max_requests=3)
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
        K.check(np.concatenate(got[r]), want[r], dtype, f"request {r} in mixed batches")


def test_a_slot_that_is_used_again_starts_from_nothing(models):
    """One state slot: the second request gets the slot (and the pages) that the first one left full."""
    raw, w, folder = models["K1"]
    eng = K.make_engine(folder, "float32", page_size=4, pool_tokens=64, max_requests=1)
    first, second = K.tokens(raw["vocab"], 50, 1), K.tokens(raw["vocab"], 33, 2)
    K.check(K.run_alone(eng, 1, first, [20, 30]), K.oracle(raw, w, first), "float32", "first user of the slot")
    K.check(K.run_alone(eng, 2, second, [1, 1, 31]), K.oracle(raw, w, second), "float32", "second user of the slot")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, models):
    raw, w, folder = models["K1"]
    ids = K.tokens(raw["vocab"], 260, 8)
    eng = K.make_engine(folder, dtype, page_size=16, pool_tokens=320)
    K.check(K.run_alone(eng, 1, ids, [6] + [1] * 254), K.oracle(raw, w, ids), dtype, "254 tokens decoded one by one")


@pytest.mark.parametrize("dtype,graphs,portion_graphs", [("float32", 0, 0), ("bfloat16", 0, 0), ("bfloat16", 4, 0),
                                                         ("bfloat16", 4, 64)])
def test_greedy_generation_through_the_scheduler(dtype, graphs, portion_graphs, models):
    """``Engine.generate``: prompts cut by the scheduler's token budget, more prompts than state slots, decode
    graphs in bfloat16, and graphs of prompt portions whose shape comes again (captured on throw-away requests
    while live requests hold states).  float32: the tokens are the plain implementation's; bfloat16: every
    generated token is one whose plain logit is within a small margin of the best."""
    from llm_infer_rust_b200 import SamplingParams
    raw, w, folder = models["K3"]
    prompts = [K.tokens(raw["vocab"], n, 40 + n) for n in (5, 23, 1, 12, 30, 64, 50)]
    eng = K.make_engine(folder, dtype, page_size=8, pool_tokens=512, max_requests=3, cuda_graph_bs=graphs,
                        chunked_prefill_size=16, max_prefill_tokens_per_batch=16,
                        prefill_cuda_graph_max_tokens=portion_graphs)
    results = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    eng.check_kernel_errors()
    for prompt, res in zip(prompts, results):
        assert len(res.tokens) == 12
        logits = K.oracle(raw, w, prompt + res.tokens)
        for i, tok in enumerate(res.tokens):
            row = logits[len(prompt) - 1 + i]
            margin = 1e-4 if dtype == "float32" else 0.05 * max(1.0, np.abs(row).max())
            assert row[tok] >= row.max() - margin, f"token {i} of a prompt of {len(prompt)}: {tok} is not the best"


def test_trace_replay_as_a_user_runs_it(models, tmp_path):
    from replay_driver import Replay, run_alone
    raw, w, folder = models["K2"]
    ids = K.tokens(raw["vocab"], 70, 9)
    want = K.oracle(raw, w, ids)
    for dtype in ("bfloat16", "float32"):
        rp = Replay(folder, dtype, 128, str(tmp_path / dtype), raw["vocab"], ["--page-size", "8"])
        try:
            K.check(run_alone(rp, "x", ids, [33, 2, 3] + [1] * 32), want, dtype, "replay")
        finally:
            assert rp.close() == 0


def test_command_line_random_weights_mode_and_sampling(tmp_path):
    """The command line writes a random Kefetar model from a configuration and serves it; the same folder through
    ``Engine.generate`` gives the same tokens, and sampled generation repeats itself under a seed."""
    import json
    import os
    import subprocess
    import sys
    from llm_infer_rust_b200 import SamplingParams
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(K.CONFIGS["K2"]))
    made = tmp_path / "made"
    cmd = [sys.executable, "-m", "llm_infer_rust_b200", "--model-path", str(made), "--random-weights", "--config",
           str(cfg), "--seed", "5", "--dtype", "float32", "--page-size", "4", "--max-total-tokens", "256",
           "--max-running-req", "2", "--max-seq-len", "64", "--cuda-graph-bs", "0", "--prompt-ids", "1,2,3",
           "--prompt-ids", "9,8,7,6,5", "--max-tokens", "6", "--ignore-eos"]
    done = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    lines = [json.loads(x) for x in done.stdout.strip().splitlines()]
    assert sorted(os.listdir(made)) == ["config.json", "model.safetensors"]
    eng = K.make_engine(str(made), "float32", page_size=4, pool_tokens=256, max_requests=2)
    want = eng.generate([[1, 2, 3], [9, 8, 7, 6, 5]], SamplingParams(max_tokens=6, ignore_eos=True))
    assert [x["output_ids"] for x in lines] == [r.tokens for r in want]
    sp = SamplingParams(temperature=0.9, top_k=12, top_p=0.95, max_tokens=8, ignore_eos=True, seed=3)
    first = eng.generate([[4, 4, 4]], sp)[0].tokens
    assert eng.generate([[4, 4, 4]], sp)[0].tokens == first and len(first) == 8
    eng.check_kernel_errors()
