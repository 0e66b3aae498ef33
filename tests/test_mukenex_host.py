"""Mukenex on the host: configuration, registry, run list, weight plan, and the plain implementation's own checks."""
import copy
import math

import pytest
import torch

import mukenex_kit as M
import plain_mukenex as P
from llm_infer_rust_b200 import ConfigError, resolve_architecture
from llm_infer_rust_b200.config.mukenex import MukenexConfig

ALL = dict(M.CONFIGS, latent=M.ONLY_LATENT, blocks=M.ONLY_BLOCKS, lightning=M.ONLY_LIGHTNING)


def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_file():
    raw = M.CONFIGS["M1"]
    arch = resolve_architecture(raw)
    assert arch.name == "Mukenex"
    c = arch.parse_config(raw)
    assert (c.vocab, c.width, c.eps, c.streams, c.softcap) == (101, 44, 1e-5, 2, 12.0)
    assert [l.kind for l in c.layers] == ["attention", "lightning", "latent_attention", "lightning"]
    assert c.run == (0, 1, 2, 1, 2, 3)
    a, l = c.layers[0], c.layers[2]
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.mask) == (4, 2, 16, 8, 0.3, 7)
    assert (a.ff.kind, a.ff.ff, a.ff.experts, a.ff.top) == ("moe", 24, 5, 2)
    assert (l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.mask, l.rot_base, l.rot_dims) == (3, 8, 8, 12, 16, 9, 100.0, 4)
    assert l.ff is None and c.layers[1].decay == (0.9, 0.99) and c.layers[1].ff.kind == "dense"
    spec = arch.model_spec(c)
    assert [e.layer for e in spec.run_list] == [0, 1, 2, 1, 2, 3]
    assert spec.layers[0]["mixer"]["chunk"] == 7 and spec.layers[0]["mixer"].get("window") is None
    assert spec.layers[2]["mixer"]["window"] == 9 and spec.layers[2]["mixer"].get("chunk") is None
    assert "feed_forward" not in spec.layers[2].parts and spec.layers[0]["feed_forward"].kind == "table_experts"
    assert spec.lm_head["softcap"] == 12.0 and spec.final_norm["streams"] == 2
    # what the file does not mention does not exist
    plain = arch.parse_config(M.CONFIGS["M2"])
    assert plain.streams is None and plain.softcap is None and plain.run == (0, 1, 2)
    spec2 = arch.model_spec(plain)
    assert spec2.layers[0]["mixer_mix"]["fixed"] and spec2.lm_head.get("softcap") is None
    assert arch.parse_config(M.CONFIGS["M3"]).run == (0, 0, 0, 1, 2)
    assert arch.parse_config(M.CONFIGS["M4"]).run == (0, 1, 2)


@pytest.mark.parametrize("change,message", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda r: r["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda r: r["layers"][1].update(type="mamba"), "type"),
    (lambda r: r["layers"][1]["mlp"].update(kind="experts"), "mlp.kind"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda r: r["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r.update(streams=9), "streams"),
    (lambda r: r["loop"].update(stop=5), "loop"),
    (lambda r: r["loop"].update(times=0), "times"),
])
def test_configurations_that_are_refused(change, message):
    raw = copy.deepcopy(M.CONFIGS["M1"])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        MukenexConfig.parse(raw)


def test_the_weight_plan_names_exactly_the_tensors_of_a_checkpoint():
    for raw in ALL.values():
        arch = resolve_architecture(raw)
        plan = arch.weight_plan(arch.parse_config(raw))
        w = M.random_weights(raw, 1)
        named = {s.name: tuple(s.shape) for b in plan for s in b.sources}
        assert named == {n: tuple(t.shape) for n, t in w.items()}


def test_random_weights_mode_writes_a_folder_whose_table_rows_differ(tmp_path):
    from llm_infer_rust_b200.weights.random_init import random_tensors
    raw = M.CONFIGS["M1"]
    t = random_tensors(raw, 3, dtype="bfloat16")
    table = t["l0.mlp.table"]
    assert table.dtype == torch.int32 and tuple(table.shape) == (101, 2)
    assert int(table.min()) >= 0 and int(table.max()) < 5 and bool((table[:, 0] != table[:, 1]).all())
    assert torch.equal(t["l0.hc1.mix"].float(), torch.eye(2)) and float(t["l0.norm1"].abs().max()) == 0.0
    # a stream of such weights starts as the ordinary residual: in sums to one, out is one
    assert abs(float(t["l0.hc1.in"].float().sum()) - 1.0) < 1e-2 and float(t["l0.hc1.out"].float().min()) == 1.0


# ----------------------------------------------------------------------------- the plain implementation's own checks
def test_plain_masks_by_hand():
    w = P.window_mask(6, 3)
    assert w[5].tolist() == [False, False, False, True, True, True] and w[1].tolist() == [True, True] + [False] * 4
    c = P.chunk_mask(7, 3)
    assert c[3].tolist() == [False, False, False, True, False, False, False]
    assert c[5].tolist() == [False, False, False, True, True, True, False]
    assert c[2].tolist() == [True, True, True, False, False, False, False]


def test_plain_rotation_pairs_neighbours_and_leaves_the_rest():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 7.0]], [[1.0, 0.0, 0.0, 2.0, 5.0, 7.0]]], dtype=torch.float64)
    y = P.rotate_pairs(x, 100.0, 4)
    assert torch.equal(y[0], x[0])                                            # position 0: nothing turns
    a0, a1 = 1.0, 100.0 ** -0.5                                               # f_i = base^(-2i/dims)
    want = [math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 5.0, 7.0]
    torch.testing.assert_close(y[1, 0], torch.tensor(want, dtype=torch.float64))


def test_plain_sink_takes_weight_without_a_value():
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    k = torch.zeros(1, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[4.0, 8.0]]], dtype=torch.float64)
    mask = torch.ones(1, 1, dtype=torch.bool)
    out = P.masked_softmax_attention(q, k, v, 1.0, mask, sink=torch.tensor([math.log(3.0)]))
    torch.testing.assert_close(out[0, 0], v[0, 0] / 4.0)                      # e^0 / (e^0 + 3)
    torch.testing.assert_close(P.masked_softmax_attention(q, k, v, 1.0, mask)[0, 0], v[0, 0])


def test_plain_recurrence_by_hand_and_the_latent_identity():
    q = torch.ones(3, 1, 1, dtype=torch.float64)
    k = torch.ones(3, 1, 1, dtype=torch.float64)
    v = torch.tensor([1.0, 2.0, 4.0], dtype=torch.float64).reshape(3, 1, 1)
    o = P.decay_recurrence(q, k, v, [0.5])
    assert o.reshape(-1).tolist() == [1.0, 2.5, 5.25]
    # q . (W c) = (W^T q) . c: what lets an engine cache the latent alone
    g = torch.Generator().manual_seed(0)
    W, c, qq = (torch.randn(s, generator=g, dtype=torch.float64) for s in ((5, 3), (3,), (5,)))
    torch.testing.assert_close(qq @ (W @ c), (W.T @ qq) @ c)


def test_plain_streams_of_one_with_unit_coefficients_are_the_ordinary_residual():
    raw = copy.deepcopy(M.CONFIGS["M2"])
    w = M.random_weights(raw, 5)
    ids = M.tokens(raw["vocab"], 20, 1)
    base = P.forward(raw, w, ids)
    raw1 = dict(raw, streams=1)
    w1 = dict(w)
    for i, layer in enumerate(raw["layers"]):
        for q in ("hc1", "hc2") if layer.get("mlp") else ("hc1",):
            w1[f"l{i}.{q}.in"], w1[f"l{i}.{q}.out"], w1[f"l{i}.{q}.mix"] = torch.ones(1), torch.ones(1), torch.ones(1, 1)
    torch.testing.assert_close(P.forward(raw1, w1, ids), base)
    assert P.run_list(M.CONFIGS["M1"]) == [0, 1, 2, 1, 2, 3]
