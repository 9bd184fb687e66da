"""The plain restatement of the Vakesun design against hand-made cases, and the checkpoint writer's layout. No GPU."""
import math

import numpy as np
import torch

from tests import vakesun_plain as P
from uzu_b200 import safetensors_io as st
from uzu_b200 import synth

F64 = torch.float64


def small_config():
    return P.make_config(48, 61, [
        P.latent_layer(3, 8, 6, 16, 12, 5, 20),
        P.attention_layer(4, 2, 8, 6, None, rot_dims=4, scaling={"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}),
        P.mlstm_layer(2, 8, 6, None),
        P.latent_layer(2, 4, 8, 16, 8, 9, 24, kv_from=0),
    ], residual_mult=0.3, embedding_scale=0.5, side_dim=4)


def test_dynamic_tanh_takes_no_mean_and_no_variance():
    W = {"n": torch.tensor([2.0, 1.0, 1.0]), "n.b": torch.tensor([0.5, 0.0, -1.0]), "n.alpha": torch.tensor(0.5)}
    out = P.dyt(torch.tensor([[100.0, 0.0, -2.0]]), W, "n")
    assert torch.allclose(out, torch.tensor([[2.5, 0.0, -math.tanh(1.0) - 1.0]], dtype=F64))
    # scaling the row changes the result (an RMS norm would not notice)
    assert not torch.allclose(P.dyt(torch.tensor([[1.0, 2.0, 3.0]]), W, "n"), P.dyt(torch.tensor([[2.0, 4.0, 6.0]]), W, "n"))


def test_gelu_tanh_values():
    z = torch.tensor([0.0, 1.0, -1.0, 3.0], dtype=F64)
    ref = [0.0, 0.8411919906082768, -0.15880800939172324, 2.996362607454593]
    assert torch.allclose(P.gelu_tanh(z), torch.tensor(ref, dtype=F64), atol=1e-12)


def test_rotation_pairs_are_halves_and_the_rest_passes():
    rot = {"base": 100.0, "dims": 4}
    x = torch.zeros(2, 1, 6, dtype=F64)
    x[:, 0, 0] = 1.0
    x[:, 0, 5] = 7.0
    y = P.rotate_halves(x, [0, 3], rot)
    assert torch.allclose(y[0], x[0])                                 # position 0 turns nothing
    assert abs(float(y[1, 0, 0]) - math.cos(3.0)) < 1e-12 and abs(float(y[1, 0, 2]) - math.sin(3.0)) < 1e-12      # channel 0 pairs with 2
    assert float(y[1, 0, 1]) == 0.0 and float(y[1, 0, 3]) == 0.0 and float(y[1, 0, 5]) == 7.0


def test_blended_frequencies():
    rot = {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 16, "fast": 2.0, "slow": 0.5}}
    f, mult = P.rot_frequencies(rot)
    where = lambda t: 8 * math.log(16 / (2 * math.pi * t)) / (2 * math.log(10000.0))
    lo, hi = max(math.floor(where(2.0)), 0), min(math.ceil(where(0.5)), 7)
    for i, fi in enumerate(f):
        plain = 10000.0 ** (-2 * i / 8)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert abs(fi - (plain / 4 * ramp + plain * (1 - ramp))) < 1e-15
    assert abs(mult - (0.1 * math.log(4.0) + 1)) < 1e-15
    assert f[0] == 1.0 and f[-1] < 10000.0 ** (-6 / 8)                 # fast pairs stay, slow pairs are stretched
    assert P.rot_frequencies({"base": 10.0, "dims": 4}) == ([1.0, 10.0 ** -0.5], 1.0)


def test_sink_only_enlarges_the_denominator_and_window_edges():
    q = torch.ones(6, 1, 2, dtype=F64)
    k = torch.zeros(6, 1, 2, dtype=F64)                               # every score is 0
    v = torch.eye(6, dtype=F64)[:, None, :]                           # the output lists the weights
    pos = list(range(6))
    o = P.softmax_attention(q, k, v, pos, pos, 5.0, window=3, sink=torch.tensor([math.log(2.0)]))
    # position 5 sees 3, 4, 5 (itself and the window - 1 before it); with the sink e^ln2 = 2 the denominator is 3 + 2
    assert torch.allclose(o[5, 0], torch.tensor([0, 0, 0, 0.2, 0.2, 0.2], dtype=F64))
    assert torch.allclose(o[1, 0], torch.tensor([0.25, 0.25, 0, 0, 0, 0], dtype=F64))
    assert torch.allclose(P.softmax_attention(q, k, v, pos, pos, 5.0)[5, 0], torch.full((6,), 1 / 6, dtype=F64))


def test_grouped_heads_read_their_group():
    q = torch.zeros(1, 4, 2, dtype=F64)
    k = torch.zeros(1, 2, 2, dtype=F64)
    v = torch.tensor([[[1.0], [2.0]]], dtype=F64)
    o = P.softmax_attention(q, k, v, [0], [0], 1.0)
    assert o[0, :, 0].tolist() == [1.0, 1.0, 2.0, 2.0]


def test_matrix_memory_first_steps_by_hand():
    """The running maximum starts at 0: with i = -3 and f = log sigmoid(2) the first maximum is f (not i), the gain e^(i - f)."""
    i = torch.tensor([[-3.0]], dtype=F64)
    f = torch.nn.functional.logsigmoid(torch.tensor([[2.0]], dtype=F64))
    q, k, v = torch.tensor([[[2.0, 0.0]]], dtype=F64), torch.tensor([[[1.0, 1.0]]], dtype=F64), torch.tensor([[[3.0]]], dtype=F64)
    o, (S, n, m) = P.mlstm_scan(q, k, v, i, f)
    assert abs(float(m) - float(f)) < 1e-15
    gain = math.exp(-3.0 - float(f))
    assert torch.allclose(S[0], gain * torch.tensor([[3.0], [3.0]], dtype=F64)) and torch.allclose(n[0], gain * torch.tensor([1.0, 1.0], dtype=F64))
    den = max(abs(gain * 2.0), math.exp(-float(f))) + 1e-6
    assert abs(float(o[0, 0, 0]) - gain * 3.0 * 2.0 / den) < 1e-12
    ig, fg = P.mlstm_gates(torch.tensor([1000.0]), torch.tensor([-1000.0]), 15.0)
    assert abs(float(ig) - 15.0) < 1e-9 and abs(float(fg) + 15.0) < 1e-6      # the cap, then log sigmoid(-15) ~ -15


def test_a_borrower_reads_the_lenders_latents():
    cfg = small_config()
    w = P.random_weights(cfg, 0)
    toks = list(range(20))
    a, layers_a, _ = P.forward(cfg, w, toks)
    w2 = dict(w)
    w2["l0.mix.dkv.norm"] = w["l0.mix.dkv.norm"] * 2
    w2["l0.mix.uk"], w2["l0.mix.uv"] = w["l0.mix.uk"] / 2, w["l0.mix.uv"] / 2        # layer 0 itself is unchanged ...
    b, layers_b, _ = P.forward(cfg, w2, toks)
    assert torch.allclose(layers_a[2], layers_b[2], atol=1e-9)
    assert (layers_a[3] - layers_b[3]).abs().max() > 1e-3                               # ... but the borrower sees doubled latents
    assert "l3.mix.dkv" not in w


def test_portions_equal_the_whole_prompt():
    cfg = small_config()
    w = P.random_weights(cfg, 1)
    toks = [int(x) for x in np.random.default_rng(0).integers(0, 61, 40)]
    whole, _, _ = P.forward(cfg, w, toks)
    state, parts = None, []
    for lo, hi in ((0, 7), (7, 8), (8, 10), (10, 31), (31, 40)):
        o, _, state = P.forward(cfg, w, toks[lo:hi], state)
        parts.append(o)
    assert (torch.cat(parts) - whole).abs().max() < 1e-11


def test_token_input_uses_the_layers_columns():
    cfg = small_config()
    w = P.random_weights(cfg, 2)
    x = torch.randn(3, 48, dtype=F64)
    a = P.token_side(x, [5, 6, 7], w, "l1.", 1, 4, 1e-6)
    w2 = dict(w)
    t = w["side.embed"].clone()
    t[:, 0:4] = 0                                                      # layer 0's columns do not reach layer 1
    w2["side.embed"] = t
    assert torch.equal(a, P.token_side(x, [5, 6, 7], w2, "l1.", 1, 4, 1e-6))
    t[:, 4:8] *= 2                                                     # a factor on the gated unit leaves the unit-RMS result alone (but for eps)
    assert torch.allclose(a, P.token_side(x, [5, 6, 7], w2, "l1.", 1, 4, 1e-6), atol=1e-3)
    assert torch.allclose((a / w["l1.side.norm"].to(F64)).pow(2).mean(-1), torch.ones(3, dtype=F64), atol=1e-3)


def test_checkpoint_writer_matches_the_design(tmp_path):
    cfg = synth.vakesun_config(48, 61, [
        synth.vakesun_latent_layer(3, 8, 6, 16, 12, 5, synth.vakesun_dense_mlp(20)),
        synth.vakesun_attention_layer(4, 2, 8, 6, None, rot_dims=4),
        synth.vakesun_mlstm_layer(2, 8, 6, None),
        synth.vakesun_latent_layer(2, 4, 8, 16, 8, 9, synth.vakesun_dense_mlp(24), kv_from=0),
    ], side_dim=4)
    path = synth.write_vakesun_model(cfg, tmp_path / "m", seed=3)
    tensors, dtypes, _ = st.load(path / "model.safetensors")
    ref = P.random_weights(P.make_config(48, 61, [
        P.latent_layer(3, 8, 6, 16, 12, 5, 20), P.attention_layer(4, 2, 8, 6, None, rot_dims=4), P.mlstm_layer(2, 8, 6, None),
        P.latent_layer(2, 4, 8, 16, 8, 9, 24, kv_from=0)], side_dim=4), 0)
    assert set(tensors) == set(ref)
    for name, v in tensors.items():
        assert tuple(v.shape) == tuple(ref[name].shape) and dtypes[name] == "BF16", name
    w = {k: torch.from_numpy(np.asarray(synth.st_bits_to_f32(np.asarray(v))).reshape(v.shape).copy()) for k, v in tensors.items()}
    logits, layers, _ = P.forward(cfg, w, [1, 2, 3, 4, 5])
    assert torch.isfinite(logits).all() and layers.shape == (4, 5, 48)
