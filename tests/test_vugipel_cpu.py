"""The plain Vugipel restatement (tests/vugipel_plain.py) against hand-made cases, and the synthetic checkpoint layout. Runs without a GPU."""
import json
import math

import torch

from tests import vugipel_plain as P
from uzu_b200 import safetensors_io as st
from uzu_b200 import synth

F64 = torch.float64


def test_norm_weight_is_a_distance_from_one():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    assert torch.allclose(P.offset_norm(x, torch.zeros(2), 0.0), x / math.sqrt(12.5))
    assert torch.allclose(P.offset_norm(x, torch.tensor([1.0, -1.0]), 0.0), torch.tensor([[6.0 / math.sqrt(12.5), 0.0]], dtype=F64))


def test_min_gru_candidate_and_gate():
    zl = torch.tensor([[0.0, 0.0, 50.0, -50.0]], dtype=F64)
    u = torch.tensor([[0.0, -1e-9, 2.0, 2.0]], dtype=F64)
    S, last = P.min_gru_scan(zl, u, torch.tensor([1.0, 1.0, 9.0, 9.0], dtype=F64))
    assert torch.allclose(S[0], torch.tensor([0.75, 0.75, 2.5, 9.0], dtype=F64))
    assert torch.equal(S[0], last)
    # two steps equal one call over two rows
    zl2, u2 = torch.randn(2, 3, dtype=F64), torch.randn(2, 3, dtype=F64)
    both, _ = P.min_gru_scan(zl2, u2, torch.zeros(3, dtype=F64))
    a, s = P.min_gru_scan(zl2[:1], u2[:1], torch.zeros(3, dtype=F64))
    b, _ = P.min_gru_scan(zl2[1:], u2[1:], s)
    assert torch.equal(both, torch.cat([a, b]))


def test_window_keeps_the_first_tokens():
    assert P.visible(10, 10, 3, 2) and P.visible(10, 8, 3, 2) and not P.visible(10, 7, 3, 2)
    assert P.visible(10, 1, 3, 2) and not P.visible(10, 2, 3, 2) and not P.visible(4, 5, 3, 2)
    assert P.visible(2, 0, 1, 0) is False and P.visible(2, 2, 1, 0)


def test_attention_weights_sum_to_one_over_visible_keys_only():
    g = torch.Generator().manual_seed(0)
    T = 12
    q, k = torch.randn(T, 2, 4, generator=g, dtype=F64), torch.randn(T, 1, 4, generator=g, dtype=F64)
    v = torch.ones(T, 1, 3, dtype=F64)
    pos = list(range(T))
    out = P.window_softmax_attention(q, k, v, pos, pos, 2, 1, 0.5, torch.tensor([1.0, 2.0]), 5.0, 3, 1)
    assert torch.allclose(out, torch.ones_like(out))
    v = torch.zeros(T, 1, 3, dtype=F64)
    v[4] = 1.0                              # position 4 is outside the window of 3 from position 7 on, and not a kept token
    out = P.window_softmax_attention(q, k, v, pos, pos, 2, 1, 0.5, torch.tensor([1.0, 2.0]), 5.0, 3, 1)
    assert (out[7:] == 0).all() and (out[4:7] > 0).all() and (out[:4] == 0).all()


def test_soft_cap_bounds_the_scores():
    q = torch.tensor([[[100.0]], [[100.0]]], dtype=F64)
    k = torch.tensor([[[1.0]], [[-1.0]]], dtype=F64)
    v = torch.tensor([[[1.0]], [[0.0]]], dtype=F64)
    out = P.window_softmax_attention(q, k, v, [0, 1], [0, 1], 1, 1, 1.0, torch.ones(1), 2.0, 8, 0)
    # scores +-100 are capped to +-2: the weights are e^2 and e^-2, not 1 and 0
    assert abs(float(out[1, 0, 0]) - math.exp(2) / (math.exp(2) + math.exp(-2))) < 1e-9


def test_values_turned_by_their_position_and_back_carry_the_distance():
    g = torch.Generator().manual_seed(1)
    v = torch.randn(6, 1, 8, generator=g, dtype=F64)
    turned = P.rotate_pairs(v, list(range(6)), 100.0, 8)
    # what position 5 reads of position 2 after turning back is the value turned by 2 - 5
    back = P.rotate_pairs(turned[2:3], [5], 100.0, 8, sign=-1.0)
    assert torch.allclose(back, P.rotate_pairs(v[2:3], [-3], 100.0, 8))
    # partial rotation leaves the tail alone
    part = P.rotate_pairs(v, list(range(6)), 100.0, 4)
    assert torch.equal(part[..., 4:], v[..., 4:]) and not torch.allclose(part[1:, :, :4], v[1:, :, :4])
    # pairs are neighbours (2i, 2i+1): channel 0 and 1 mix, channel 0 and 4 do not
    e0 = torch.zeros(1, 1, 8, dtype=F64)
    e0[0, 0, 0] = 1.0
    r = P.rotate_pairs(e0, [1], 100.0, 8)
    assert abs(float(r[0, 0, 0]) - math.cos(1.0)) < 1e-12 and abs(float(r[0, 0, 1]) - math.sin(1.0)) < 1e-12 and float(r[0, 0, 4]) == 0.0


def test_retention_closed_form():
    g = torch.Generator().manual_seed(2)
    T, H, d, dv = 7, 2, 3, 4
    q, k, v = torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, dv, generator=g, dtype=F64)
    decay = [0.5, 1.0]
    out, last = P.retention_scan(q, k, v, decay, torch.zeros(H, d, dv, dtype=F64))
    for h in range(H):
        for t in range(T):
            want = sum(decay[h] ** (t - j) * float(q[t, h] @ k[j, h]) / math.sqrt(d) * v[j, h] for j in range(t + 1))
            assert torch.allclose(out[t, h], want)
    a, s = P.retention_scan(q[:3], k[:3], v[:3], decay, torch.zeros(H, d, dv, dtype=F64))
    b, s2 = P.retention_scan(q[3:], k[3:], v[3:], decay, s)
    assert torch.allclose(torch.cat([a, b]), out) and torch.allclose(s2, last)


def test_router_weight_sits_on_the_expert_input():
    W = {"router": torch.tensor([[2.0], [2.0], [-1.0]]), "e0.gate": torch.tensor([[1.0]]), "e0.up": torch.tensor([[1.0]]), "e0.down": torch.tensor([[1.0]]),
         "e1.gate": torch.tensor([[1.0]]), "e1.up": torch.tensor([[1.0]]), "e1.down": torch.tensor([[5.0]]),
         "e2.gate": torch.tensor([[1.0]]), "e2.up": torch.tensor([[1.0]]), "e2.down": torch.tensor([[100.0]])}
    h = torch.tensor([[1.0]], dtype=F64)
    s = 1.0 / (1.0 + math.exp(-2.0))
    unit = s * (s / (1.0 + math.exp(-s)))              # silu(s) * s: the weight went through the expert, not around it
    one = P.routed_experts(h, W, "", P.moe_mlp(1, 3, 1))
    assert abs(float(one) - unit) < 1e-12              # equal logits: the lower index
    two = P.routed_experts(h, W, "", P.moe_mlp(1, 3, 2))
    assert abs(float(two) - 6.0 * unit) < 1e-12        # weights are not renormalised


def test_portions_and_whole_prompt_agree():
    cfg = P.make_config(40, 50, [P.mingru_layer(24, P.moe_mlp(12, 3, 2)),
                                 P.parallel_layer(4, 2, 8, 6, 5, 2, 3, 6, 4, [0.9, 0.5, 1.0], mlp=P.moe_mlp(8, 2, 1), rot_dims=4)])
    w = P.random_weights(cfg, 1)
    toks = list(range(1, 31))
    whole = P.forward(cfg, w, toks)
    state = P.State(cfg)
    parts = [P.forward(cfg, w, toks[a:b], state) for a, b in ((0, 2), (2, 3), (3, 17), (17, 30))]
    assert torch.allclose(torch.cat(parts), whole, atol=1e-10)


def test_synthetic_checkpoint_layout(tmp_path):
    cfg = synth.vugipel_config(32, 40, [
        synth.vugipel_mingru_layer(20, synth.vugipel_moe_mlp(10, 3, 2)),
        synth.vugipel_parallel_layer(4, 2, 8, 6, 5, 1, 2, 10, 12, None, rot_dims=4),
    ])
    path = synth.write_vugipel_model(cfg, tmp_path / "m", seed=2)
    assert json.loads((path / "config.json").read_text())["architecture"] == "Vugipel"
    tensors, dtypes, _ = st.load(path / "model.safetensors")
    assert set(dtypes.values()) == {"BF16"}
    assert tensors["l0.mix.z"].shape == (20, 32) and tensors["l0.mix.x.b"].shape == (20,) and tensors["l0.mix.o"].shape == (32, 20)
    assert tensors["l0.mlp.router"].shape == (3, 32) and tensors["l0.mlp.e2.down"].shape == (32, 10) and "l0.mlp.router.b" not in tensors
    assert tensors["l1.mix.left.q"].shape == (32, 32) and tensors["l1.mix.left.k"].shape == (16, 32) and tensors["l1.mix.left.v.b"].shape == (12,)
    assert tensors["l1.mix.left.q.norm"].shape == (8,) and tensors["l1.mix.left.temp"].shape == (4,) and tensors["l1.mix.left.o"].shape == (32, 24)
    assert tensors["l1.mix.right.k"].shape == (20, 32) and tensors["l1.mix.right.g"].shape == (24, 32) and tensors["l1.mix.right.o"].shape == (32, 24)
    assert "l1.norm2" not in tensors and len(cfg["layers"][1]["mixer"]["right"]["decay"]) == 2
    # the oracle runs on what the file holds
    w = {k: torch.from_numpy(synth.st_bits_to_f32(v)) for k, v in tensors.items()}
    out = P.forward(cfg, w, [1, 2, 3, 4])
    assert out.shape == (4, 40) and torch.isfinite(out).all()
    preset = synth.vugipel_preset(256, 100, blocks=2, experts=4, top=2)
    assert [L["type"] for L in preset["layers"]] == ["mingru", "parallel", "mingru", "parallel"]
