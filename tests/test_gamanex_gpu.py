"""Gamanex (sigmoid attention, gated parallel sublayers, routed experts) on the GPU against the plain float64 restatement in
tests/gamanex_plain.py.

Kernel-level tests feed one mechanism through the C ABI; engine-level tests write a small random checkpoint from the oracle's own
random weights, run it through the engine's passes / slots / decode graph and compare logits. Engines run in true f32 (tight bounds: a
mask, cache or slot fault is orders of magnitude above them) and in the serving precisions (bf16 products and caches).
"""
import ctypes as C
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import gamanex_plain as P
from uzu_b200 import binding as B
from uzu_b200 import safetensors_io as st
from uzu_b200 import synth

pytestmark = pytest.mark.gpu
F64 = torch.float64
ROOT = Path(__file__).resolve().parents[1]


def t64(a):
    return torch.from_numpy(np.asarray(a)).to(F64)


def bf16_exact(a):
    return synth.st_bits_to_f32(synth.f32_to_bf16_bits(np.asarray(a, np.float32)))


def run(ctx, fn, *args):
    with ctx.command_buffer(fn) as cmd:
        cmd.encode(fn, *args)


def close(got, ref, tol, what=""):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    scale = max(float(np.sqrt((ref ** 2).mean())), 1e-6)
    err = float(np.abs(got - ref).max()) / scale
    assert err <= tol, f"{what}: max error {err:.3e} of the rms exceeds {tol:.1e}"


# ---- kernels, one mechanism each ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,n", [(1, 96), (5, 90), (33, 2500)])
def test_one_sum_of_squares_two_scaled_copies(ctx, rows, n):
    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, n), dtype=np.float32) * 3
    w1, w2 = rng.standard_normal(n, dtype=np.float32), rng.standard_normal(n, dtype=np.float32)
    bx, b1, b2, o1, o2 = ctx.upload(x), ctx.upload(w1), ctx.upload(w2), ctx.upload(np.zeros_like(x)), ctx.upload(np.zeros_like(x))
    a = B.GroupRmsNormArgs(input=bx.ptr, scales=b1.ptr, output=o1.ptr, rows=rows, n=n, groups=1, in_stride=n, out_stride=n, epsilon=1e-3,
                           scales2=b2.ptr, output2=o2.ptr)
    run(ctx, "uzu_group_rms_norm_encode", C.byref(a))
    close(o1.numpy(np.float32, x.shape), P.rms_norm(t64(x), t64(w1), 1e-3).numpy(), 2e-6, "first copy")
    close(o2.numpy(np.float32, x.shape), P.rms_norm(t64(x), t64(w2), 1e-3).numpy(), 2e-6, "second copy")


@pytest.mark.parametrize("m", [1, 5, 40, 100, 130])
@pytest.mark.parametrize("f32_weights", [True, False])
def test_squared_relu_operand_and_gated_scaled_accumulation(ctx, m, f32_weights):
    """D += scale[c] * sigmoid(gate[r, c] + bias[c]) * (relu(A)^2 . W^T): the operand is a column range of a wider block that also holds the gate."""
    rng = np.random.default_rng(m)
    n, k = 70, 128
    block = rng.standard_normal((m, k + n + 3), dtype=np.float32)      # [operand | 3 unused | gate logits]
    w = bf16_exact(rng.standard_normal((n, k)) / 8)
    bias, scale = rng.standard_normal(n, dtype=np.float32), rng.standard_normal(n, dtype=np.float32)
    d0 = rng.standard_normal((m, n), dtype=np.float32)
    bb, bw = ctx.upload(block), ctx.upload(w if f32_weights else synth.f32_to_bf16_bits(w))
    bbias, bscale, bd = ctx.upload(bias), ctx.upload(scale), ctx.upload(d0)
    ws = ctx.upload(np.zeros((m, k), np.uint16))
    a = B.DenseLinearArgs(a=bb.ptr, w=bw.ptr, d=bd.ptr, gate=bb.ptr + 4 * (k + 3), gate_ld=block.shape[1], gate_bias=bbias.ptr, col_scale=bscale.ptr,
                          workspace=ws.ptr, m=m, n=n, k=k, lda=block.shape[1], ldd=n, batch=1, weights_dt=B.DT_F32 if f32_weights else B.DT_BF16,
                          accumulate=1, scale=1.0, a_op=2)
    run(ctx, "uzu_dense_linear_encode", C.byref(a))
    act = torch.relu(t64(block[:, :k])) ** 2
    if not f32_weights and m >= 32:
        act = t64(bf16_exact(act.numpy()))
    ref = t64(d0) + t64(scale) * torch.sigmoid(t64(block[:, k + 3:]) + t64(bias)) * (act @ t64(w).T)
    close(bd.numpy(np.float32, d0.shape), ref.numpy(), 5e-6, "gated accumulation")


@pytest.mark.parametrize("m", [1, 7, 20])
def test_silu_gated_unit(ctx, m):
    """Standalone over a [gate | up] block, and as the paired epilogue of the short-pass product."""
    rng = np.random.default_rng(m)
    f, k = 37, 64
    gu = rng.standard_normal((m, 2 * f), dtype=np.float32) * 2
    bg, bo = ctx.upload(gu), ctx.upload(np.zeros((m, f), np.float32))
    run(ctx, "uzu_silu_glu_encode", bg.ptr, bo.ptr, m, f)
    g, u = t64(gu[:, :f]), t64(gu[:, f:])
    close(bo.numpy(np.float32, (m, f)), (g * torch.sigmoid(g) * u).numpy(), 2e-6, "silu unit")
    if m <= 8:
        x = rng.standard_normal((m, k), dtype=np.float32)
        w = bf16_exact(rng.standard_normal((2 * f, k)) / 4)
        bx, bw, bd = ctx.upload(x), ctx.upload(synth.f32_to_bf16_bits(w)), ctx.upload(np.zeros((m, f), np.float32))
        a = B.DenseLinearArgs(a=bx.ptr, w=bw.ptr, d=bd.ptr, m=m, n=f, k=k, lda=k, ldd=f, batch=1, weights_dt=B.DT_BF16, scale=1.0, pair_rows=f, glu_kind=1)
        run(ctx, "uzu_dense_linear_encode", C.byref(a))
        g, u = t64(x) @ t64(w[:f]).T, t64(x) @ t64(w[f:]).T
        close(bd.numpy(np.float32, (m, f)), (g * torch.sigmoid(g) * u).numpy(), 5e-6, "paired silu unit")


@pytest.mark.parametrize("rows,experts,top,stride", [(1, 10, 4, 10), (9, 5, 5, 9), (70, 40, 1, 64), (1024, 7, 3, 7), (6, 130, 8, 130)])
def test_router_picks_the_largest_and_sorts_pairs_by_expert(ctx, rows, experts, top, stride):
    rng = np.random.default_rng(rows + experts)
    z = rng.standard_normal((rows, stride), dtype=np.float32)
    z[:, :experts] = np.round(z[:, :experts] * 4) / 4              # many equal logits: the lower index must win
    bias = (np.round(rng.standard_normal(experts) * 2) / 4).astype(np.float32)
    bz, bb = ctx.upload(z), ctx.upload(bias)
    off, rmap, ppos = ctx.upload(np.zeros(experts + 1, np.uint32)), ctx.upload(np.zeros(rows * top, np.uint32)), ctx.upload(np.zeros(rows * top, np.uint32))
    pw = ctx.upload(np.zeros(rows * top, np.float32))
    a = B.TopkRouteArgs(logits=bz.ptr, bias=bb.ptr, group_offsets=off.ptr, rows_map=rmap.ptr, pair_pos=ppos.ptr, pair_weight=pw.ptr, rows=rows, top=top,
                        experts=experts, logits_stride=stride)
    run(ctx, "uzu_topk_route_encode", C.byref(a))
    W = {"mlp.router": torch.eye(experts, dtype=F64), "mlp.router.b": t64(bias)}
    idx, wt = P.route(t64(z[:, :experts]), W, "", top)
    offsets, rows_map, pair_pos, weight = off.numpy(np.uint32), rmap.numpy(np.uint32), ppos.numpy(np.uint32).reshape(rows, top), pw.numpy(np.float32).reshape(rows, top)
    close(weight, wt.numpy(), 2e-6, "weights of the chosen experts")
    counts = np.bincount(idx.numpy().ravel(), minlength=experts)
    assert offsets.tolist() == np.concatenate([[0], np.cumsum(counts)]).tolist()
    seen = np.zeros(rows * top, bool)
    for r in range(rows):
        for s in range(top):
            e, at = int(idx[r, s]), int(pair_pos[r, s])
            assert offsets[e] <= at < offsets[e + 1] and rows_map[at] == r and not seen[at], (r, s, e, at)
            seen[at] = True
    for e in range(experts):                                       # token order inside an expert's list
        assert np.all(np.diff(rows_map[offsets[e]:offsets[e + 1]].astype(np.int64)) > 0)


def test_weighted_gated_combination_of_expert_rows(ctx):
    rng = np.random.default_rng(8)
    rows, top, n = 11, 3, 50
    pairs = rng.standard_normal((rows * top, n), dtype=np.float32)
    pos = rng.permutation(rows * top).astype(np.uint32)
    w = rng.random(rows * top, dtype=np.float32)
    gate = rng.standard_normal((rows, n + 6), dtype=np.float32)
    bias, scale, x0 = rng.standard_normal(n, dtype=np.float32), rng.standard_normal(n, dtype=np.float32), rng.standard_normal((rows, n), dtype=np.float32)
    bp, bpos, bw, bg, bb, bs, bx = map(ctx.upload, (pairs, pos, w, gate, bias, scale, x0))
    a = B.RoutedCombineArgs(pairs=bp.ptr, pair_pos=bpos.ptr, pair_weight=bw.ptr, gate=bg.ptr + 4 * 6, gate_bias=bb.ptr, col_scale=bs.ptr, output=bx.ptr,
                            rows=rows, top=top, n=n, gate_ld=n + 6, accumulate=1, weight=1.0)
    run(ctx, "uzu_routed_combine_gated_encode", C.byref(a))
    mix = (t64(w).reshape(rows, top, 1) * t64(pairs)[torch.from_numpy(pos.astype(np.int64))].reshape(rows, top, n)).sum(1)
    ref = t64(x0) + t64(scale) * torch.sigmoid(t64(gate[:, 6:]) + t64(bias)) * mix
    close(bx.numpy(np.float32, x0.shape), ref.numpy(), 3e-6, "combine")


def attention_gpu(ctx, q, k, v, qw, kw, r1, r2, pb, *, heads, kv_heads, dim, vdim, scale, eps, temp, prefix, cache, f32_cache=True, splits=0, own=True, chunk_tiles=0):
    """Feeds raw projections [T, ...] of the tokens at positions prefix .. prefix + T - 1 through prepare + attend. `cache` is (keys, values)
    device buffers that persist between calls."""
    T = q.shape[0]
    qn, kn, vn = heads * dim, kv_heads * dim, kv_heads * vdim
    block = np.concatenate([q, k, v], axis=1).astype(np.float32)
    bb, bqw, bkw = ctx.upload(block), ctx.upload(qw.astype(np.float32)), ctx.upload(kw.astype(np.float32))
    query, out = ctx.upload(np.zeros((T, qn), np.float32)), ctx.upload(np.zeros((T, heads * vdim), np.float32))
    dt = B.DT_F32 if f32_cache else B.DT_BF16
    pa = B.SigmoidAttentionPrepareArgs(q=bb.ptr, k=bb.ptr + 4 * qn if own else 0, v=bb.ptr + 4 * (qn + kn) if own else 0, q_scales=bqw.ptr, k_scales=bkw.ptr,
                                       query=query.ptr, keys=cache[0].ptr, values=cache[1].ptr, rows=T, q_n=qn, k_n=kn, v_n=vn,
                                       q_stride=block.shape[1], k_stride=block.shape[1], v_stride=block.shape[1], prefix=prefix, cache_dt=dt,
                                       temp_every=temp[1] if temp else 0, temp_coef=temp[0] if temp else 0.0, epsilon=eps)
    run(ctx, "uzu_sigmoid_attention_prepare_encode", C.byref(pa))
    b1, b2, b3 = ctx.upload(r1.astype(np.float32)), ctx.upload(r2.astype(np.float32)), ctx.upload(pb.astype(np.float32))
    parts = ctx.upload(np.zeros(max(1, T * heads * max(splits, 1, (prefix + T + 63) // 64) * vdim), np.float32))
    tickets = ctx.upload(np.zeros(T * heads, np.uint32))
    aa = B.SigmoidAttentionArgs(query=query.ptr, keys=cache[0].ptr, values=cache[1].ptr, out=out.ptr, dist_r1=b1.ptr, dist_r2=b2.ptr, head_bias=b3.ptr,
                                partials=parts.ptr, tickets=tickets.ptr, rows=T, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, prefix=prefix,
                                cache_dt=dt, scale=scale, splits=splits, chunk_tiles=chunk_tiles)
    run(ctx, "uzu_sigmoid_attention_encode", C.byref(aa))
    assert not tickets.numpy(np.uint32).any(), "every ticket returns to zero"
    return out.numpy(np.float32, (T, heads * vdim)).copy(), query.numpy(np.float32, (T, qn)).copy()


def attention_plain(q, k, v, qw, kw, r1, r2, pb, *, heads, kv_heads, dim, vdim, scale, eps, temp, prefix, round_cache=False):
    """q rows are the last len(q) positions of the k / v rows (all positions from 0)."""
    n, T = k.shape[0], q.shape[0]
    qq = P.rms_norm(t64(q), t64(qw), eps)
    pos = list(range(n - T, n))
    if temp:
        qq = qq * P.query_temperature(pos, temp[0], temp[1])[:, None]
    kk, vv = P.rms_norm(t64(k), t64(kw), eps), t64(v)
    if round_cache:
        kk, vv = t64(bf16_exact(kk.numpy())), t64(bf16_exact(vv.numpy()))
    return P.sigmoid_attention(qq, kk, vv, pos, list(range(n)), heads, kv_heads, dim, vdim, scale, t64(r1), t64(r2), t64(pb)).numpy(), qq.numpy()


def new_cache(ctx, positions, kv_heads, dim, vdim, f32_cache):
    e = np.float32 if f32_cache else np.uint16
    return ctx.upload(np.zeros((positions, kv_heads * dim), e)), ctx.upload(np.zeros((positions, kv_heads * vdim), e))


@pytest.mark.parametrize("T,prefix,heads,kv_heads,dim,vdim,temp", [
    (1, 0, 2, 2, 8, 8, None), (1, 77, 6, 2, 16, 24, (0.4, 7)), (40, 0, 4, 1, 32, 16, (0.25, 16)), (70, 130, 3, 3, 9, 7, (1.5, 1)),
    (200, 65, 8, 4, 64, 64, (0.35, 128)), (130, 2, 2, 1, 128, 96, None), (17, 300, 1, 1, 260, 40, (0.1, 50)),
    (64, 0, 2, 2, 16, 16, None), (100, 40, 4, 2, 32, 48, (0.2, 30)), (260, 1000, 2, 1, 96, 80, (0.15, 512)), (129, 63, 3, 1, 80, 112, None)])
@pytest.mark.parametrize("f32_cache", [True, False])
def test_sigmoid_attention_kernels(ctx, T, prefix, heads, kv_heads, dim, vdim, temp, f32_cache):
    """A prefix pass, then the pass under test on top of it (prompt portion or one decoded token), with and without key splits."""
    rng = np.random.default_rng(T + prefix + dim)
    n = prefix + T
    q, k, v = (rng.standard_normal((n, c), dtype=np.float32) for c in (heads * dim, kv_heads * dim, kv_heads * vdim))
    qw, kw = 1 + 0.2 * rng.standard_normal(heads * dim), 1 + 0.2 * rng.standard_normal(kv_heads * dim)
    r1, r2, pb = np.abs(rng.standard_normal(heads)) * 0.5, np.abs(rng.standard_normal(heads)) * 0.3 + 0.05, rng.standard_normal(heads) - 1
    kw_ = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=1.3 / np.sqrt(dim), eps=1e-5, temp=temp)
    ref, ref_q = attention_plain(q[prefix:], k, v, qw, kw, r1, r2, pb, prefix=prefix, round_cache=not f32_cache, **kw_)
    for splits in (0, 2, 5, 64):
        cache = new_cache(ctx, n + 3, kv_heads, dim, vdim, f32_cache)
        if prefix:
            attention_gpu(ctx, q[:prefix], k[:prefix], v[:prefix], qw, kw, r1, r2, pb, prefix=0, cache=cache, f32_cache=f32_cache, **kw_)
        got, got_q = attention_gpu(ctx, q[prefix:], k[prefix:], v[prefix:], qw, kw, r1, r2, pb, prefix=prefix, cache=cache, f32_cache=f32_cache,
                                   splits=splits, **kw_)
        close(got_q, ref_q, 3e-6, "normed query with temperature")
        close(got, ref, 2e-5 if f32_cache else 2e-4, f"attention, splits {splits}")
    if not f32_cache and T >= 64:                  # tensor-pipe passes with the key tiles of a row tile cut into chunks
        for chunk_tiles in (1, 2, 5):
            got, _ = attention_gpu(ctx, q[prefix:], k[prefix:], v[prefix:], qw, kw, r1, r2, pb, prefix=prefix, cache=cache, f32_cache=False, own=False,
                                   chunk_tiles=chunk_tiles, **kw_)
            close(got, ref, 2e-4, f"attention, chunks of {chunk_tiles} key tiles")


@pytest.mark.parametrize("far", [0, 1, 31, 32, 33, 500])
@pytest.mark.parametrize("f32_cache", [True, False])
def test_one_far_key_among_hundreds_and_the_causal_edge(ctx, far, f32_cache):
    """Every key but one scores far below zero; the one at position `far` scores high. Queries before it must not see it (also not the query one
    place before), queries from it on get its value times a weight that falls with the distance. Prompt rows and one decoded row."""
    rng = np.random.default_rng(far)
    heads, dim, vdim, n, T = 2, 16, 16, 640, 130
    k = rng.standard_normal((n, dim), dtype=np.float32) * 0.05
    k[:, 3] = 0
    k[far] = 0
    k[far, 3] = 30.0
    q = rng.standard_normal((n, heads * dim), dtype=np.float32) * 0.05
    q[:, 3] = 4.0
    q[:, dim + 3] = 4.0
    v = rng.standard_normal((n, vdim), dtype=np.float32)
    r1, r2, pb = np.array([0.0, 0.8]), np.array([0.0, 0.5]), np.array([-14.0, -12.0])
    kw_ = dict(heads=heads, kv_heads=1, dim=dim, vdim=vdim, scale=1.0, eps=1e-6, temp=None)
    qw, kw = np.ones(heads * dim), np.ones(dim)
    ref, _ = attention_plain(q, k, v, qw, kw, r1, r2, pb, prefix=0, round_cache=not f32_cache, **kw_)
    assert np.abs(ref[far:]).max() > 0.2 and (far == 0 or np.abs(ref[:far]).max() < 1e-3), "the far key must matter, and only from its place on"
    for prefix in sorted({0, max(far - 1, 0), min(far + 1, n - T), n - T, n - 1}):
        cache = new_cache(ctx, n, 1, dim, vdim, f32_cache)
        if prefix:
            attention_gpu(ctx, q[:prefix], k[:prefix], v[:prefix], qw, kw, r1, r2, pb, prefix=0, cache=cache, f32_cache=f32_cache, **kw_)
        hi = min(n, prefix + T) if prefix < n - 1 else n
        for splits in (0, 3):
            got, _ = attention_gpu(ctx, q[prefix:hi], k[prefix:hi], v[prefix:hi], qw, kw, r1, r2, pb, prefix=prefix, cache=cache, f32_cache=f32_cache,
                                   splits=splits, **kw_)
            assert np.abs(got - ref[prefix:hi]).max() < 2e-4, (far, prefix, splits)


def test_borrowing_layer_writes_no_cache_rows(ctx):
    rng = np.random.default_rng(1)
    heads, dim, vdim, T = 2, 8, 8, 5
    q, k, v = (rng.standard_normal((T, c), dtype=np.float32) for c in (heads * dim, dim, vdim))
    cache = new_cache(ctx, T, 1, dim, vdim, True)
    kw_ = dict(heads=heads, kv_heads=1, dim=dim, vdim=vdim, scale=0.3, eps=1e-5, temp=None)
    z = np.zeros(heads)
    first, _ = attention_gpu(ctx, q, k, v, np.ones(heads * dim), np.ones(dim), z, z, z, prefix=0, cache=cache, **kw_)
    again, _ = attention_gpu(ctx, q, k * 0 + 9, v * 0 + 9, np.ones(heads * dim), np.ones(dim), z, z, z, prefix=0, cache=cache, own=False, **kw_)
    assert np.array_equal(first, again)


# ---- whole models through the engine ----------------------------------------------------------------------------------------------
def config_a():
    """Every size differs from every other; grouped key heads; two borrowers of one lender; experts with top 3 and top 1; a layer without
    feed-forward and one without temperature."""
    return P.make_config(96, 211, [
        P.attention_layer(6, 2, 16, 24, scale=0.21, q_temp=(0.4, 7), mlp=P.dense_mlp(56)),
        P.attention_layer(6, 2, 16, 24, scale=0.3, q_temp=(0.2, 5), kv_from=0, mlp=P.moe_mlp(28, 6, 3)),
        P.attention_layer(3, 3, 20, 12, mlp=None),
        P.attention_layer(2, 2, 16, 24, scale=0.25, q_temp=(0.4, 7), kv_from=0, mlp=P.moe_mlp(44, 4, 1)),
    ], eps=1e-4, logit_scale=0.7)


def config_b():
    """One head, all experts chosen (5 of 5) and one of two, temperature that changes at every position, wide cache rows (few tokens per
    cache page), logit scale 1, a borrower right after a borrower."""
    return P.make_config(64, 130, [
        P.attention_layer(1, 1, 500, 24, q_temp=(0.5, 1), mlp=P.moe_mlp(12, 5, 5)),
        P.attention_layer(1, 1, 500, 24, kv_from=0, mlp=P.moe_mlp(20, 2, 1)),
        P.attention_layer(1, 1, 500, 24, kv_from=0, q_temp=(0.1, 300), mlp=P.dense_mlp(40)),
        P.attention_layer(4, 4, 8, 8, mlp=P.dense_mlp(24)),
    ], eps=1e-6, logit_scale=1.0)


def config_c():
    """Sizes that fit no vector width: width 90, odd head sizes 9 / 7 (bf16 rows that start at odd elements), odd feed-forwards, 3 experts."""
    return P.make_config(90, 77, [
        P.attention_layer(4, 2, 9, 7, scale=0.4, q_temp=(0.35, 3), mlp=P.moe_mlp(11, 3, 2)),
        P.attention_layer(2, 1, 18, 20, q_temp=(0.15, 64), mlp=P.dense_mlp(51)),
        P.attention_layer(4, 2, 9, 7, scale=0.2, kv_from=0, mlp=None),
    ], eps=1e-5, logit_scale=0.3)


def write_model(path, config, weights):
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config))
    st.save(path / "model.safetensors", {k: st.as_bf16(synth.f32_to_bf16_bits(v.to(torch.float32).numpy())) for k, v in weights.items()})
    return path


class Pair:
    """A checkpoint on disk, the engine on it and the oracle on the same (bf16-exact) tensors."""

    def __init__(self, ctx, tmp_path, config, seed=0, f32=True, weights=None, max_context=4096, **kw):
        self.config = config
        self.weights = weights or P.random_weights(config, seed)
        path = write_model(tmp_path / f"m{seed}{int(f32)}", config, self.weights)
        self.engine = B.Engine(ctx, path, max_context_length=max_context, storage_f32=f32, **kw)
        self.f32 = f32
        self.tol = 2e-4 if f32 else 6e-2

    def reference(self, tokens, layers=None):
        return P.forward(self.config, self.weights, list(tokens), layers).numpy()

    def check(self, got, ref, what):
        got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
        d = (got - ref) - (got - ref).mean(-1, keepdims=True)
        err = np.sqrt((d * d).mean(-1)) / max(float(ref.std()), 1e-6)
        # bf16 products can turn a router's close call the other way for a token or two: there the bound holds for nine rows in ten (the f32
        # engine, where a close call needs a gap of 1e-6, is held to it in every row)
        worst = err.max() if self.f32 else np.quantile(err, 0.9)
        assert worst <= self.tol, f"{what}: row {int(err.argmax())} differs by {err.max():.3e} of the logits' spread (bound {self.tol:.0e})"

    def close(self):
        self.engine.close()


def tokens_for(config, n, seed=0):
    return np.random.default_rng(seed).integers(0, config["vocab"], n).tolist()


@pytest.mark.parametrize("make", [config_a, config_b, config_c])
@pytest.mark.parametrize("f32", [True, False])
def test_prompt_logits_and_layers(ctx, tmp_path, make, f32):
    pr = Pair(ctx, tmp_path, make(), seed=1, f32=f32)
    toks = tokens_for(pr.config, 70 if f32 else 150, 1)     # bf16: 150 rows take the tensor-pipe products and attention
    pr.engine.debug_layer_outputs(True)
    s = pr.engine.slot_acquire()
    got = pr.engine.forward_rows(toks, list(range(len(toks))), slot=s)
    layers = pr.engine.debug_layer_outputs(True)
    ref_layers = []
    ref = pr.reference(toks, ref_layers)
    for i, (g, r) in enumerate(zip(layers, ref_layers)):
        if f32:
            close(g, r.numpy(), 1e-5, f"residual after layer {i}")
        else:                                   # see Pair.check: nine rows in ten
            row_err = np.abs(g - r.numpy()).max(-1) / np.sqrt((r.numpy() ** 2).mean())
            assert np.quantile(row_err, 0.9) <= 1e-1, f"residual after layer {i}"
    pr.check(got, ref, "prompt logits")
    pr.close()


@pytest.mark.parametrize("make", [config_a, config_b, config_c])
@pytest.mark.parametrize("f32", [True, False])
def test_decode_and_portions_match_the_whole_prompt(ctx, tmp_path, make, f32):
    """Prefill + token-by-token decoding, and portions of 2, 3, 1, 33, 2, ... tokens, give the logits of the whole prompt."""
    pr = Pair(ctx, tmp_path, make(), seed=2, f32=f32)
    n = 90
    toks = tokens_for(pr.config, n, 2)
    ref = pr.reference(toks)
    s = pr.engine.slot_acquire()
    parts = [pr.engine.forward_rows(toks[:50], list(range(50)), slot=s)]
    parts += [pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(50, n)]
    pr.check(np.concatenate(parts), ref, "prefill + decode")
    pr.engine.slot_release(s)
    s = pr.engine.slot_acquire()                 # the same slot again: its cache rows start over
    parts, p, k = [], 0, 0
    sizes = [2, 3, 1, 33, 2, 9, 32, 2]
    while p < n:
        c = min(sizes[k % len(sizes)], n - p)
        parts.append(pr.engine.forward_rows(toks[p:p + c], list(range(c)), slot=s))
        p, k = p + c, k + 1
    pr.check(np.concatenate(parts), ref, "portions")
    pr.close()


def test_slots_interleaved_and_reused(ctx, tmp_path):
    """Three unequal requests advance in turns in their own slots; one ends early and its slot serves a new request. Each equals its solo run."""
    pr = Pair(ctx, tmp_path, config_a(), seed=3, f32=True)
    reqs = {name: tokens_for(pr.config, n, 10 + i) for i, (name, n) in enumerate([("a", 41), ("b", 7), ("c", 64), ("d", 23)])}
    refs = {name: pr.reference(t) for name, t in reqs.items()}
    got = {name: [] for name in reqs}
    at = {name: 0 for name in reqs}
    slot = {}
    live, waiting = ["a", "b", "c"], ["d"]
    step = {"a": 5, "b": 2, "c": 1, "d": 4}
    while live:
        for name in list(live):
            if name not in slot:
                slot[name] = pr.engine.slot_acquire()
            c = min(step[name], len(reqs[name]) - at[name])
            got[name].append(pr.engine.forward_rows(reqs[name][at[name]:at[name] + c], list(range(c)), slot=slot[name]))
            at[name] += c
            if at[name] == len(reqs[name]):
                pr.engine.slot_release(slot[name])
                live.remove(name)
                if waiting:
                    live.append(waiting.pop())
    assert slot["d"] == slot["b"]                # the freed slot was handed out again
    for name in reqs:
        pr.check(np.concatenate(got[name]), refs[name], f"request {name}")
    pr.close()


def test_long_context_page_and_pass_edges(ctx, tmp_path):
    """1100 tokens: past the 1024-row pass and, with 500-wide f32 key rows, past the first cache page (lender and borrowers); then 40 decoded
    tokens. Rows just before and after both edges are compared, in the prompt and decoded."""
    pr = Pair(ctx, tmp_path, config_b(), seed=4, f32=True)
    n = 1140
    toks = tokens_for(pr.config, n, 4)
    ref = pr.reference(toks)
    s = pr.engine.slot_acquire()
    rows = [0, 1, 2, 1014, 1015, 1016, 1017, 1022, 1023, 1024, 1025, 1047, 1048, 1049, 1099]
    got = pr.engine.forward_rows(toks[:1100], rows, slot=s)
    pr.check(got, ref[rows], "long prompt")
    dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(1100, n)])
    pr.check(dec, ref[1100:], "decoding after a long prompt")
    pr.engine.slot_release(s)
    s = pr.engine.slot_acquire()                 # decode across the edges: prompt of 1010, then one by one over 1024 and the page's end
    pr.engine.forward_rows(toks[:1010], [], slot=s)
    dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(1010, 1060)])
    pr.check(dec, ref[1010:1060], "decoding over the edges")
    pr.close()


def marker_model(marker=7):
    """Two layers, the second borrowing the first's cache. Input coordinate 0 is non-zero for the marker token only and key channel 3 reads
    it; coordinate 1 is the same for every token and query channel 3 of every head reads it. With a head bias far below zero only the
    marker's key gets a weight worth mentioning, at any distance."""
    cfg = P.make_config(48, 60, [P.attention_layer(2, 1, 8, 12, scale=1.0, mlp=None),
                                 P.attention_layer(2, 1, 8, 12, scale=1.0, kv_from=0, q_temp=(0.2, 100), mlp=P.dense_mlp(20))], eps=1e-6, logit_scale=1.0)
    w = {k: v.to(torch.float32) for k, v in P.random_weights(cfg, 5).items()}
    w["embed"][:, 0] = 0.0
    w["embed"][:, 1] = 3.0
    w["embed"][marker] = 0.0
    w["embed"][marker, 0] = 5.0
    w["embed"][marker, 1] = 3.0
    w["l0.norm1"][:] = 1.0
    w["l0.mix.k.norm"][:] = 1.0
    w["l0.mix.k"] *= 0.05
    w["l0.mix.k"][:, 0] = 0.0
    w["l0.mix.k"][3, :] = 0.0
    w["l0.mix.k"][3, 0] = 10.0
    for p in ("l0.", "l1."):
        w[p + "mix.q.norm"][:] = 1.0
        w[p + "mix.q"] *= 0.05
        for h in range(2):
            w[p + "mix.q"][h * 8 + 3, :] = 0.0
            w[p + "mix.q"][h * 8 + 3, 1] = 6.0
        w[p + "mix.pb"][:] = -9.0
        w[p + "mix.r1"][:] = 0.05
        w[p + "mix.o"] *= 3.0
        w[p + "ls1"][:] = 1.0
    return cfg, {k: v.to(torch.bfloat16) for k, v in w.items()}, marker


def test_far_token_decides_the_logits(ctx, tmp_path):
    """A marker token somewhere in a 700-token prompt (position 0, 1, 31, 32, 33, 400) changes the last logits strongly; the engine agrees
    with the oracle for each place, in the prompt's last row and in 10 decoded tokens."""
    cfg, w, marker = marker_model()
    pr = Pair(ctx, tmp_path, cfg, seed=5, f32=True, weights=w)
    base = [x if x != marker else 8 for x in tokens_for(cfg, 700, 5)]
    without = pr.reference(base)
    for place in (0, 1, 31, 32, 33, 400):
        toks = list(base)
        toks[place] = marker
        ref = pr.reference(toks)
        moved = np.sqrt(((ref[689:] - without[689:]) ** 2).mean(-1)).max() / ref.std()
        assert moved > 0.3, "the marker must matter for this test to mean anything"
        s = pr.engine.slot_acquire()
        got = pr.engine.forward_rows(toks[:690], [689], slot=s)
        dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(690, 700)])
        pr.engine.slot_release(s)
        pr.check(got, ref[689:690], f"marker at {place}, prompt")
        pr.check(dec, ref[690:], f"marker at {place}, decoded")
    pr.close()


@pytest.mark.parametrize("graph", [True, False])
def test_greedy_generation_through_the_stream(ctx, tmp_path, graph):
    """prefill() + next()/flush() (the engine's generation entry point; CUDA-graph decode when `graph`), 300 tokens. The oracle reads the whole
    sequence once: every chosen token must be its best at that place within the rounding of the bf16 logits the sampler reads."""
    pr = Pair(ctx, tmp_path, config_a(), seed=6, f32=True, use_cuda_graph=graph)
    prompt = tokens_for(pr.config, 12, 6)
    steps = 300 if graph else 40
    out = pr.engine.generate(prompt, steps)
    assert len(out) == steps
    ref = pr.reference(prompt + out)
    for i, tok in enumerate(out):
        z = ref[len(prompt) - 1 + i]
        assert z[tok] >= z.max() - 2.0 ** -7 * np.abs(z).max() - 1e-3, f"token {i}: the engine chose {tok}, the oracle's best is {int(z.argmax())}"
    # the stream's state is the context so far: feeding one more token gives the oracle's logits
    pr.check(pr.engine.forward_rows([out[-1]], [0]), ref[-1:], "the stream's state after generation")
    pr.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_command_line(tmp_path, dtype):
    """bin/trace_run as a user starts it: two requests one after the other, each in portions down to two tokens and single decoded tokens,
    logits of the wanted places in <step>.f32; the second request reuses the first one's slot."""
    import subprocess
    import sys
    cfg = config_a()
    w = P.random_weights(cfg, 9)
    model = write_model(tmp_path / "model", cfg, w)
    reqs = {"a": tokens_for(cfg, 57, 1), "b": tokens_for(cfg, 31, 2)}
    lines, wanted = [], []
    step = 0
    for rid, toks in reqs.items():
        at, sizes, k = 0, [2, 19, 1, 3, 1, 1, 40], 0
        while at < len(toks):
            c = min(sizes[k % len(sizes)], len(toks) - at)
            want = list(range(c)) if k % 2 == 0 else [c - 1]
            lines.append(json.dumps({"step": step, "entries": [{"id": rid, "tokens": toks[at:at + c], "want": want}],
                                     "end": [rid] if at + c == len(toks) else []}))
            wanted.append((step, rid, [at + x for x in want]))
            at, k, step = at + c, k + 1, step + 1
    out = tmp_path / "out"
    root = ROOT
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(step)]
    refs = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    V = cfg["vocab"]
    errs = []
    for s, rid, places in wanted:
        got = np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(len(places), V).astype(np.float64)
        d = got - refs[rid][places]
        d = d - d.mean(-1, keepdims=True)
        errs += list(np.sqrt((d * d).mean(-1)) / refs[rid].std())
    errs = np.array(errs)
    if dtype == "float32":
        assert errs.max() < 2e-4, errs.max()
    else:
        assert np.quantile(errs, 0.9) < 6e-2, np.quantile(errs, 0.9)
