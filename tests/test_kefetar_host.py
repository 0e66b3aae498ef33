"""Kefetar on the host: configuration, registry, weight plan, and the plain implementation's own checks."""
import copy

import pytest
import torch

import kefetar_kit as K
import plain_kefetar as P
from llm_infer_rust_b200 import ConfigError, resolve_architecture
from llm_infer_rust_b200.config.kefetar import KefetarConfig


def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_file():
    raw = K.CONFIGS["K1"]
    arch = resolve_architecture(raw)
    assert arch.name == "Kefetar"
    c = arch.parse_config(raw)
    assert (c.vocab, c.width, c.eps, c.canon_taps) == (97, 48, 1e-5, 4)
    assert [l.kind for l in c.layers] == ["retention", "attention", "attention", "retention", "attention"]
    a = c.layers[1]
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.scale, a.softcap, a.v_mix) == (4, 2, 16, 8, 3, 0.31, 20.0, True)
    assert (a.rot.base, a.rot.dims, a.rot.factor) == (10000.0, 8, 4.0)
    assert c.layers[0].decay == (0.9, 0.995) and c.layers[0].rot.factor == 1.0 and c.layers[2].ff is None
    spec = arch.model_spec(c)
    roles = [l["mixer"].get("v_mix") for l in spec.layers if l["mixer"].kind == "gated_conv_attention"]
    assert roles == ["source", "mix", "mix"]
    assert len(spec.position_encodings) == 3              # one for every distinct (base, dims, factor)
    assert "feed_forward" not in spec.layers[2].parts and "ff_conv" in spec.layers[1].parts
    # what the file does not mention does not exist
    spec2 = arch.model_spec(arch.parse_config(K.CONFIGS["K2"]))
    assert all("mixer_conv" not in l.parts for l in spec2.layers)
    m = spec2.layers[0]["mixer"]
    assert m.get("softcap") is None and m.get("position_encoding") is None and m.get("v_mix") is None
    assert m["conv_taps"] == 4 and spec2.layers[2]["mixer"]["conv_taps"] == 0
    one = arch.model_spec(arch.parse_config(K.CONFIGS["K4"]))                 # one tap is a convolution too
    assert one.layers[0]["mixer"]["conv_taps"] == 1 and one.layers[0]["mixer_conv"]["taps"] == 1


@pytest.mark.parametrize("change,message", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda r: r["layers"][0].update(type="mamba"), "type"),
    (lambda r: r["layers"][1]["mlp"].update(kind="experts"), "mlp.kind"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda r: r["layers"][4]["mixer"].update(vdim=10), "v_mix"),
    (lambda r: r["canon"].update(taps=9), "taps"),
])
def test_configurations_that_are_refused(change, message):
    raw = copy.deepcopy(K.CONFIGS["K1"])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        KefetarConfig.parse(raw)


def test_the_weight_plan_names_exactly_the_tensors_of_a_checkpoint():
    for raw in list(K.CONFIGS.values()) + [K.ONLY_ATTENTION, K.ONLY_RETENTION]:
        arch = resolve_architecture(raw)
        plan = arch.weight_plan(arch.parse_config(raw))
        weights = K.random_weights(raw, 0)
        named = {s.name: tuple(s.shape) for b in plan for s in b.sources}
        assert named == {n: tuple(t.shape) for n, t in weights.items()}


def test_a_checkpoint_with_single_numbers_is_written_and_read_back(tmp_path):
    from llm_infer_rust_b200.weights.safetensors_io import Checkpoint
    raw = K.CONFIGS["K2"]
    w = K.random_weights(raw, 3)
    ck = Checkpoint(K.write_model(str(tmp_path), raw, w))
    try:
        for name in ("final.norm", "l0.norm1", "l0.mlp.act", "l0.mix.q.conv"):
            got = ck.read(name)
            assert got.dtype == torch.bfloat16 and tuple(got.shape) == tuple(w[name].shape)
            assert torch.equal(got.float(), w[name])
    finally:
        ck.close()


# ----------------------------------------------------------------------------- the plain implementation itself
def test_plain_causal_taps_is_the_sum_it_says():
    g = torch.Generator().manual_seed(0)
    u, w = torch.randn(9, 5, generator=g, dtype=torch.float64), torch.randn(5, 3, generator=g, dtype=torch.float64)
    y = P.causal_taps(u, w)
    for t in range(9):
        want = sum(w[:, j] * u[t - 2 + j] for j in range(3) if t - 2 + j >= 0)
        assert torch.allclose(y[t], want)


def test_plain_retention_is_the_decayed_sum_over_the_past():
    g = torch.Generator().manual_seed(1)
    T, H, d, dv = 12, 2, 3, 4
    q, k = torch.randn(T, H, d, generator=g, dtype=torch.float64), torch.randn(T, H, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    decay = torch.tensor([0.8, 0.95], dtype=torch.float64)
    o = P.retention_recurrence(q, k, v, decay)
    for t in (0, 5, 11):
        for h in range(H):
            want = sum(decay[h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert torch.allclose(o[t, h], want)
    # cut in two with the state carried over
    o1, S = P.retention_recurrence(q[:7], k[:7], v[:7], decay, return_state=True)
    o2 = P.retention_recurrence(q[7:], k[7:], v[7:], decay, S0=S)
    assert torch.allclose(torch.cat([o1, o2]), o)


def test_plain_rotation_keeps_lengths_turns_by_the_position_and_leaves_the_rest():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(6, 2, 10, generator=g, dtype=torch.float64)
    y = P.rotate_half_split(x, 100.0, 4, factor=2.0)
    assert torch.allclose(y[..., 4:], x[..., 4:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[..., :4].norm(dim=-1), x[..., :4].norm(dim=-1))
    # pair (0, 2) at position 3 turns by 3 * 100^0 / 2, pair (1, 3) by 3 * 100^(-1/2) / 2
    for i, angle in ((0, 1.5), (1, 0.15)):
        a, b = x[3, 1, i], x[3, 1, i + 2]
        c, s = torch.cos(torch.tensor(angle, dtype=torch.float64)), torch.sin(torch.tensor(angle, dtype=torch.float64))
        assert torch.allclose(y[3, 1, i], a * c - b * s) and torch.allclose(y[3, 1, i + 2], b * c + a * s)


def test_plain_soft_cap_bounds_a_score_and_poly_norm_of_a_constant():
    q = torch.full((1, 1, 2), 100.0, dtype=torch.float64)
    out = P.capped_causal_attention(torch.cat([q, q]), torch.cat([q, -q]), torch.tensor([[[1.0]], [[3.0]]], dtype=torch.float64),
                                    1.0, 2.0)
    # second query: scores tanh-capped to +2 (key 0) and -2 (key 1): weights e^2 : e^-2
    want = (torch.exp(torch.tensor(2.0)) * 1.0 + torch.exp(torch.tensor(-2.0)) * 3.0) / (2 * torch.cosh(torch.tensor(2.0)))
    assert torch.allclose(out[1, 0, 0], want.double())
    z = torch.full((2, 8), 2.0, dtype=torch.float64)
    got = P.poly_norm(z, torch.tensor([1.0, 10.0, 100.0, 0.5], dtype=torch.float64), 0.0)
    assert torch.allclose(got, torch.full_like(z, 111.5))
