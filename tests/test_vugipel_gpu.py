"""Vugipel (minGRU, window attention with rotated values beside retention, sigmoid-routed experts weighted on their input) on the GPU
against the plain float64 restatement in tests/vugipel_plain.py.

Kernel-level tests feed one mechanism through the C ABI; engine-level tests write a small random checkpoint, run it through the engine's
passes / slots / decode graph and compare logits. Engines run in true f32 (tight bounds: a mask, window, state or slot fault is orders of
magnitude above them) and in the serving precisions (bf16 products and caches).
"""
import ctypes as C
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import vugipel_plain as P
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
@pytest.mark.parametrize("rows,n", [(1, 37), (5, 200), (8, 70), (64, 96), (300, 33), (1024, 130)])
def test_min_gru_scan_one_launch_and_carried_state(ctx, rows, n):
    """Strided operands inside a wider block; the launch over all rows (chunks composed in order) and the same rows in two launches with the
    state carried both equal the token-by-token scan."""
    rng = np.random.default_rng(rows + n)
    ld = 3 * n + 5
    block = (rng.standard_normal((rows, ld)) * 2).astype(np.float32)           # [z logits | candidates | gate | unused]
    s0 = rng.standard_normal(n).astype(np.float32)
    S, last = P.min_gru_scan(t64(block[:, :n]), t64(block[:, n:2 * n]), t64(s0))
    ref = (S * P.silu(t64(block[:, 2 * n:3 * n]))).numpy()
    for cut in sorted({rows, rows // 3, 1} - {0}):
        bb, bs, bo = ctx.upload(block), ctx.upload(s0), ctx.upload(np.zeros((rows, n), np.float32))
        for lo, hi in ((0, cut), (cut, rows)):
            if hi > lo:
                a = B.MinGruArgs(z_logit=bb.ptr + 4 * lo * ld, u=bb.ptr + 4 * (lo * ld + n), gate=bb.ptr + 4 * (lo * ld + 2 * n), state=bs.ptr,
                                 out=bo.ptr + 4 * lo * n, rows=hi - lo, n=n, z_stride=ld, u_stride=ld, gate_stride=ld, out_stride=n)
                run(ctx, "uzu_min_gru_encode", C.byref(a))
        close(bo.numpy(np.float32, (rows, n)), ref, 3e-6, f"scan cut at {cut}")
        close(bs.numpy(np.float32, (n,)), last.numpy(), 3e-6, f"state cut at {cut}")


def test_min_gru_candidate_branches_and_saturated_gates(ctx):
    """u = 0 takes the linear branch (1/2), u just below 0 the sigmoid; a gate logit of +-40 keeps or replaces the state entirely."""
    zl = np.array([[40.0, -40.0, 0.0, 0.0, 40.0]], np.float32)
    u = np.array([[0.0, 3.0, -1e-6, 2.5, -30.0]], np.float32)
    s0 = np.array([7.0, 7.0, 1.0, 1.0, 7.0], np.float32)
    bz, bu, bs, bo = ctx.upload(zl), ctx.upload(u), ctx.upload(s0), ctx.upload(np.zeros((1, 5), np.float32))
    a = B.MinGruArgs(z_logit=bz.ptr, u=bu.ptr, gate=0, state=bs.ptr, out=bo.ptr, rows=1, n=5)
    run(ctx, "uzu_min_gru_encode", C.byref(a))
    close(bo.numpy(np.float32, (1, 5)), [[0.5, 7.0, 0.75, 2.0, 0.0]], 1e-6, "branches")


@pytest.mark.parametrize("rows,heads,dim,vdim", [(1, 3, 64, 48), (17, 2, 9, 7), (100, 2, 128, 64), (40, 1, 48, 96), (33, 5, 20, 33)])
def test_retention_state_and_outputs(ctx, rows, heads, dim, vdim):
    """Decays of 1 (nothing forgotten), 1/2 and close to 1; key size != value size; one launch equals two launches with the state carried."""
    rng = np.random.default_rng(rows + dim)
    ld = heads * (2 * dim + vdim) + 3
    block = rng.standard_normal((rows, ld)).astype(np.float32)
    decay = np.array(([1.0, 0.5, 0.96875, 0.75, 0.999])[:heads], np.float32)
    s0 = rng.standard_normal((heads, dim, vdim)).astype(np.float32)
    q = t64(block[:, :heads * dim]).reshape(rows, heads, dim)
    k = t64(block[:, heads * dim:2 * heads * dim]).reshape(rows, heads, dim)
    v = t64(block[:, 2 * heads * dim:2 * heads * dim + heads * vdim]).reshape(rows, heads, vdim)
    ref, last = P.retention_scan(q, k, v, decay, t64(s0))
    for cut in sorted({rows, rows // 2} - {0}):
        bb, bd, bs, bo = ctx.upload(block), ctx.upload(decay), ctx.upload(s0), ctx.upload(np.zeros((rows, heads * vdim), np.float32))
        for lo, hi in ((0, cut), (cut, rows)):
            if hi > lo:
                a = B.RetentionArgs(q=bb.ptr + 4 * lo * ld, k=bb.ptr + 4 * (lo * ld + heads * dim), v=bb.ptr + 4 * (lo * ld + 2 * heads * dim), decay=bd.ptr,
                                    state=bs.ptr, out=bo.ptr + 4 * lo * heads * vdim, rows=hi - lo, heads=heads, dim=dim, vdim=vdim, q_stride=ld, k_stride=ld,
                                    v_stride=ld, out_stride=heads * vdim, key_scale=1.0 / math.sqrt(dim))
                run(ctx, "uzu_retention_encode", C.byref(a))
        close(bo.numpy(np.float32, (rows, heads * vdim)), ref.reshape(rows, -1).numpy(), 5e-6, f"outputs cut at {cut}")
        close(bs.numpy(np.float32, s0.shape), last.numpy(), 5e-6, f"state cut at {cut}")


def test_retention_remembers_a_far_token(ctx):
    """600 tokens with keys orthogonal to the query except token 3: with decay 1 the output is exactly that token's value, with decay d it is
    d^(596) of it."""
    rows, dim, vdim = 600, 16, 8
    q = np.zeros((rows, 2 * dim), np.float32); k = np.zeros((rows, 2 * dim), np.float32)
    v = np.random.default_rng(0).standard_normal((rows, 2 * vdim)).astype(np.float32)
    q[:, 0] = q[:, dim] = 1.0
    k[:, 1] = k[:, dim + 1] = 1.0
    k[3, 0] = k[3, dim] = 4.0
    decay = np.array([1.0, 0.99], np.float32)
    bq, bk, bv, bd = ctx.upload(q), ctx.upload(k), ctx.upload(v), ctx.upload(decay)
    bs, bo = ctx.upload(np.zeros((2, dim, vdim), np.float32)), ctx.upload(np.zeros((rows, 2 * vdim), np.float32))
    a = B.RetentionArgs(q=bq.ptr, k=bk.ptr, v=bv.ptr, decay=bd.ptr, state=bs.ptr, out=bo.ptr, rows=rows, heads=2, dim=dim, vdim=vdim, key_scale=0.25)
    run(ctx, "uzu_retention_encode", C.byref(a))
    out = bo.numpy(np.float32, (rows, 2 * vdim))
    close(out[599, :vdim], v[3, :vdim], 1e-6, "decay 1")
    close(out[599, vdim:], v[3, vdim:] * 0.99 ** 596, 1e-5, "decay 0.99")
    assert np.abs(out[2]).max() == 0.0


def test_head_norm_with_silu_gate(ctx):
    rng = np.random.default_rng(3)
    rows, heads, dim = 6, 3, 33
    x = rng.standard_normal((rows, heads * dim)).astype(np.float32) * 4
    g = rng.standard_normal((rows, heads * dim + 2)).astype(np.float32) * 2
    bx, bg, bo = ctx.upload(x), ctx.upload(g), ctx.upload(np.zeros_like(x))
    a = B.HeadNormGateArgs(x=bx.ptr, scales=0, gate=bg.ptr, out=bo.ptr, rows=rows, heads=heads, dim=dim, x_stride=heads * dim, gate_stride=heads * dim + 2,
                           out_stride=heads * dim, normalize=1, epsilon=1e-3, gate_op=1)
    run(ctx, "uzu_head_norm_gate_encode", C.byref(a))
    ref = P.unit_rms(t64(x).reshape(rows, heads, dim), 1e-3).reshape(rows, -1) * P.silu(t64(g[:, :heads * dim]))
    close(bo.numpy(np.float32, x.shape), ref.numpy(), 3e-6, "unit rms * silu(gate)")


@pytest.mark.parametrize("rows,experts,top", [(1, 12, 1), (7, 5, 5), (40, 6, 2), (300, 9, 3)])
@pytest.mark.parametrize("f32_weights", [True, False])
def test_sigmoid_router_weights_scale_the_expert_input(ctx, rows, experts, top, f32_weights):
    """Router: the `top` largest logits, weight = sigmoid of each on its own. The gate / up product of a pair is multiplied by the pair's weight
    before the unit (the weight sits on the expert's input), in the short-pass paired form and in the grouped form."""
    rng = np.random.default_rng(rows + experts)
    W, f = 64, 24
    h = rng.standard_normal((rows, W)).astype(np.float32)
    z = rng.standard_normal((rows, experts)).astype(np.float32) * 2
    gu = bf16_exact(rng.standard_normal((experts, 2 * f, W)) / 6)
    bz = ctx.upload(z)
    off, rmap, ppos = ctx.upload(np.zeros(experts + 1, np.uint32)), ctx.upload(np.zeros(rows * top, np.uint32)), ctx.upload(np.zeros(rows * top, np.uint32))
    pw, cw = ctx.upload(np.zeros(rows * top, np.float32)), ctx.upload(np.zeros(rows * top, np.float32))
    scratch = ctx.upload(np.zeros(rows * top, np.uint16))          # with it, the 300-row case makes its choice over many CTAs
    ra = B.TopkRouteArgs(logits=bz.ptr, bias=0, group_offsets=off.ptr, rows_map=rmap.ptr, pair_pos=ppos.ptr, pair_weight=pw.ptr, rows=rows, top=top,
                         experts=experts, logits_stride=experts, weight_kind=1, compact_weight=cw.ptr, scratch=scratch.ptr)
    run(ctx, "uzu_topk_route_encode", C.byref(ra))
    pos, weights, compact = ppos.numpy(np.uint32, (rows, top)), pw.numpy(np.float32, (rows, top)), cw.numpy(np.float32, (rows * top,))
    order = np.argsort(-z, axis=1, kind="stable")[:, :top]
    close(weights, 1.0 / (1.0 + np.exp(-np.take_along_axis(z.astype(np.float64), order, 1))), 2e-6, "sigmoid weights, largest first")
    np.testing.assert_array_equal(compact[pos.reshape(-1)], weights.reshape(-1))
    offsets, rows_of = off.numpy(np.uint32, (experts + 1,)), rmap.numpy(np.uint32, (rows * top,))
    for e in range(experts):                                       # the pairs of an expert, in token order
        want = [r for r in range(rows) if e in order[r]]
        assert rows_of[offsets[e]:offsets[e + 1]].tolist() == want, f"expert {e}"
    bh, bw = ctx.upload(h), ctx.upload(gu if f32_weights else synth.f32_to_bf16_bits(gu))
    paired = rows <= 8
    bd = ctx.upload(np.zeros((rows * top, f if paired else 2 * f), np.float32))
    a = B.DenseLinearArgs(a=bh.ptr, w=bw.ptr, d=bd.ptr, group_offsets=off.ptr, rows_map=rmap.ptr, w_z_stride=2 * f * W, m=rows, n=f if paired else 2 * f,
                          k=W, lda=W, ldd=f if paired else 2 * f, batch=experts, weights_dt=B.DT_F32 if f32_weights else B.DT_BF16, scale=1.0,
                          pair_rows=f if paired else 0, glu_kind=1, row_scale=cw.ptr)
    run(ctx, "uzu_dense_linear_encode", C.byref(a))
    got = bd.numpy(np.float32, (rows * top, f if paired else 2 * f))
    for r in range(rows):
        for s in range(top):
            e = order[r, s]
            y = t64(h[r]) * float(weights[r, s])
            g, u = t64(gu[e, :f]) @ y, t64(gu[e, f:]) @ y
            ref = (P.silu(g) * u) if paired else torch.cat([g, u])
            close(got[pos[r, s]], ref.numpy(), 2e-5 if f32_weights or rows < 32 else 2e-2, f"pair ({r}, {s})")


@pytest.mark.parametrize("m", [3, 40, 130, 300])
@pytest.mark.parametrize("f32_weights", [True, False])
def test_product_with_bias_row_scale_and_share(ctx, m, f32_weights):
    """D += share * row_scale[r] * (A . W^T) + bias: the stacked projections' biases and an output projection's share of a sum, in the short-pass,
    tile, tensor-pipe and tensor-memory forms (the last from 128 rows on with bf16 weights)."""
    rng = np.random.default_rng(m)
    n, k = 192, 128
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = bf16_exact(rng.standard_normal((n, k)) / 8)
    bias, rs = rng.standard_normal(n).astype(np.float32), (0.2 + rng.random(m)).astype(np.float32)
    d0 = rng.standard_normal((m, n)).astype(np.float32)
    bx, bw = ctx.upload(x), ctx.upload(w if f32_weights else synth.f32_to_bf16_bits(w))
    bb, br, bd, ws = ctx.upload(bias), ctx.upload(rs), ctx.upload(d0), ctx.upload(np.zeros((m, k), np.uint16))
    a = B.DenseLinearArgs(a=bx.ptr, w=bw.ptr, d=bd.ptr, bias=bb.ptr, row_scale=br.ptr, workspace=ws.ptr, m=m, n=n, k=k, lda=k, ldd=n, batch=1,
                          weights_dt=B.DT_F32 if f32_weights else B.DT_BF16, accumulate=1, scale=0.8)
    run(ctx, "uzu_dense_linear_encode", C.byref(a))
    act = t64(x) if f32_weights or m < 32 else t64(bf16_exact(x))
    ref = t64(d0) + 0.8 * t64(rs)[:, None] * (act @ t64(w).T) + t64(bias)
    close(bd.numpy(np.float32, d0.shape), ref.numpy(), 5e-6, "bias, row scale, share")
    assert ctx.lib.uzu_debug_dense_umma_error() == 0


def rope_table(positions, pairs, base, dims):
    ang = np.arange(positions, dtype=np.float64)[:, None] * base ** (-2.0 * np.arange(pairs, dtype=np.float64) / dims)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def window_attention_gpu(ctx, q, k, v, cache, *, prefix, heads, kv_heads, dim, vdim, rot_dims, base, scale, temp, softcap, window, keep_first, qw, kw, eps,
                         f32_cache=True, splits=0, rotate_values=True):
    """One pass of T tokens at positions prefix ..; `cache` = (keys, values) device buffers that already hold positions < prefix."""
    T = q.shape[0]
    positions = prefix + T
    cs, sn = rope_table(positions, rot_dims // 2, base, rot_dims)
    vc, vs = rope_table(positions, vdim // 2, base, vdim)
    bq, bk, bv = ctx.upload(q.astype(np.float32)), ctx.upload(k.astype(np.float32)), ctx.upload(v.astype(np.float32))
    bqw, bkw = ctx.upload(qw.astype(np.float32)), ctx.upload(kw.astype(np.float32))
    bcs, bsn, bvc, bvs = ctx.upload(cs), ctx.upload(sn), ctx.upload(vc), ctx.upload(vs)
    query, out = ctx.upload(np.zeros((T, heads * dim), np.float32)), ctx.upload(np.zeros((T, heads * vdim), np.float32))
    dt = B.DT_F32 if f32_cache else B.DT_BF16
    vp = vdim // 2 if rotate_values else 0
    pa = B.WindowAttentionPrepareArgs(q=bq.ptr, k=bk.ptr, v=bv.ptr, q_scales=bqw.ptr, k_scales=bkw.ptr, query=query.ptr, keys=cache[0].ptr, values=cache[1].ptr,
                                      cosines=bcs.ptr, sines=bsn.ptr, v_cosines=bvc.ptr, v_sines=bvs.ptr, rows=T, heads=heads, kv_heads=kv_heads, dim=dim,
                                      vdim=vdim, rot_pairs=rot_dims // 2, v_pairs=vp, prefix=prefix, cache_dt=dt, epsilon=eps)
    run(ctx, "uzu_window_attention_prepare_encode", C.byref(pa))
    btemp = ctx.upload(np.asarray(temp, np.float32))
    parts = ctx.upload(np.zeros(max(T * heads * max(splits, 1) * (vdim + 2), 4), np.float32))
    tickets = ctx.upload(np.zeros(T * heads, np.uint32))
    aa = B.WindowAttentionArgs(query=query.ptr, keys=cache[0].ptr, values=cache[1].ptr, out=out.ptr, head_temp=btemp.ptr, v_cosines=bvc.ptr, v_sines=bvs.ptr,
                               partials=parts.ptr, tickets=tickets.ptr, rows=T, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, prefix=prefix, cache_dt=dt,
                               window=window, keep_first=keep_first, v_pairs=vp, scale=scale, softcap=softcap, splits=splits)
    run(ctx, "uzu_window_attention_encode", C.byref(aa))
    assert not tickets.numpy(np.uint32, (T * heads,)).any(), "tickets must be zero again"
    return out.numpy(np.float32, (T, heads * vdim))


def window_attention_plain(q, k, v, *, heads, kv_heads, dim, vdim, rot_dims, base, scale, temp, softcap, window, keep_first, qw, kw, eps,
                           round_cache=False, rotate_values=True):
    """All positions 0 .. T-1 at once"""
    T = q.shape[0]
    pos = list(range(T))
    qq = P.rotate_pairs(P.unit_rms(t64(q).reshape(T, heads, dim), eps) * t64(qw), pos, base, rot_dims)
    kk = P.rotate_pairs(P.unit_rms(t64(k).reshape(T, kv_heads, dim), eps) * t64(kw), pos, base, rot_dims)
    vv = t64(v).reshape(T, kv_heads, vdim)
    if rotate_values:
        vv = P.rotate_pairs(vv, pos, base, vdim)
    if round_cache:
        kk, vv = t64(bf16_exact(kk.numpy())), t64(bf16_exact(vv.numpy()))
    o = P.window_softmax_attention(qq, kk, vv, pos, pos, heads, kv_heads, scale, temp, softcap if softcap > 0 else 1e30, window if window else 1 << 30,
                                   keep_first)
    if rotate_values:
        o = P.rotate_pairs(o, pos, base, vdim, sign=-1.0)
    return o.reshape(T, heads * vdim).numpy()


def new_cache(ctx, positions, kv_heads, dim, vdim, f32_cache):
    dt = np.float32 if f32_cache else np.uint16
    return ctx.upload(np.zeros((positions, kv_heads * dim), dt)), ctx.upload(np.zeros((positions, kv_heads * vdim), dt))


@pytest.mark.parametrize("T,prefix,heads,kv_heads,dim,vdim,rot_dims,window,keep", [
    (40, 0, 4, 2, 16, 24, 16, 7, 2), (9, 31, 6, 2, 48, 80, 48, 20, 5), (70, 5, 2, 2, 10, 6, 4, 16, 0), (33, 0, 3, 1, 64, 32, 32, 1, 3),
    (130, 20, 2, 1, 128, 128, 64, 50, 1), (20, 0, 1, 1, 9, 14, 8, 0, 0), (25, 40, 2, 2, 24, 8, 24, 100, 5), (12, 3, 2, 1, 300, 40, 300, 6, 6),
    (200, 0, 4, 2, 64, 32, 64, 70, 3), (150, 37, 2, 1, 48, 80, 32, 20, 3), (300, 100, 2, 2, 16, 16, 8, 0, 0), (260, 0, 1, 1, 32, 64, 32, 1, 70),
    (70, 700, 2, 1, 64, 64, 64, 128, 5), (64, 1, 2, 2, 16, 112, 16, 63, 65)])
@pytest.mark.parametrize("f32_cache", [True, False])
def test_window_attention_kernels(ctx, T, prefix, heads, kv_heads, dim, vdim, rot_dims, window, keep, f32_cache):
    """Prompt rows on an empty cache and rows after a prefix, windows shorter and longer than the context, windows of one key, no window,
    more kept tokens than the window is long, partial rotation, odd head sizes, grouped heads; with key splits of 0 / 2 / 5 / 64. bf16 caches
    with passes of >= 64 rows and head sizes in multiples of 16 take the tensor-pipe kernel (no splits), the rest the plain one."""
    rng = np.random.default_rng(T + dim)
    n = prefix + T
    q, k, v = (rng.standard_normal((n, w)).astype(np.float32) * 2 for w in (heads * dim, kv_heads * dim, kv_heads * vdim))
    qw, kw = 1 + 0.3 * rng.standard_normal(dim), 1 + 0.3 * rng.standard_normal(dim)
    temp = 0.5 + rng.random(heads)
    kwargs = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot_dims=rot_dims, base=500.0, scale=dim ** -0.5, temp=temp, softcap=6.0, window=window,
                  keep_first=keep, qw=qw, kw=kw, eps=1e-5)
    ref = window_attention_plain(q, k, v, round_cache=not f32_cache, **kwargs)
    for splits in (0, 2, 5, 64):
        cache = new_cache(ctx, n, kv_heads, dim, vdim, f32_cache)
        if prefix:
            window_attention_gpu(ctx, q[:prefix], k[:prefix], v[:prefix], cache, prefix=0, f32_cache=f32_cache, **kwargs)
        got = window_attention_gpu(ctx, q[prefix:], k[prefix:], v[prefix:], cache, prefix=prefix, f32_cache=f32_cache, splits=splits, **kwargs)
        close(got, ref[prefix:], 2e-5 if f32_cache else 2e-3, f"splits {splits}")


def test_window_attention_without_cap_and_value_rotation(ctx):
    rng = np.random.default_rng(5)
    T, heads, dim, vdim = 30, 2, 16, 12
    q, k, v = (rng.standard_normal((T, w)).astype(np.float32) for w in (heads * dim, heads * dim, heads * vdim))
    kwargs = dict(heads=heads, kv_heads=heads, dim=dim, vdim=vdim, rot_dims=8, base=100.0, scale=0.9, temp=np.ones(heads), softcap=0.0, window=9, keep_first=1,
                  qw=np.ones(dim), kw=np.ones(dim), eps=1e-6, rotate_values=False)
    got = window_attention_gpu(ctx, q, k, v, new_cache(ctx, T, heads, dim, vdim, True), prefix=0, **kwargs)
    close(got, window_attention_plain(q, k, v, **kwargs), 2e-5, "plain values, no cap")


@pytest.mark.parametrize("f32_cache", [True, False])
@pytest.mark.parametrize("decoded", [True, False])
def test_one_key_at_the_edges_of_the_window_and_of_the_kept_tokens(ctx, f32_cache, decoded):
    """Among 700 keys one is made to stand out (its score is far above the others: key and query share one large channel, no rotation on
    it). Queried from position p, the output is that key's value when it is visible and something else when it is not: the key sits just
    inside / just outside the window, is the last kept token / the first one not kept, or is position 0 far outside the window."""
    heads, dim, vdim, window, keep = 2, 16, 16, 64, 3         # bf16 prompt rows take the tensor-pipe kernel, everything else the plain one
    rng = np.random.default_rng(11)
    n = 700
    for place, p, seen in [(n - window, n - 1, True), (n - window - 1, n - 1, False), (keep - 1, n - 1, True), (keep, n - 1, False), (0, 500, True),
                           (500 - window, 500, False), (500 - window + 1, 500, True), (n - 1, n - 1, True)]:
        q = np.zeros((n, heads * dim), np.float32)
        k = rng.standard_normal((n, heads * dim)).astype(np.float32) * 0.1
        v = rng.standard_normal((n, heads * vdim)).astype(np.float32)
        q[:, dim - 1] = q[:, 2 * dim - 1] = 3.0                  # the last channel is outside the rotated ones; no other key has anything there
        k[:, dim - 1] = k[:, 2 * dim - 1] = 0.0
        k[place, dim - 1] = k[place, 2 * dim - 1] = 3.0
        kwargs = dict(heads=heads, kv_heads=heads, dim=dim, vdim=vdim, rot_dims=dim - 2, base=1000.0, scale=1.0, temp=np.ones(heads), softcap=30.0, window=window,
                      keep_first=keep, qw=np.ones(dim), kw=np.ones(dim), eps=1e-6)
        ref = window_attention_plain(q, k, v, round_cache=not f32_cache, **kwargs)
        cache = new_cache(ctx, n, heads, dim, vdim, f32_cache)
        if decoded:
            window_attention_gpu(ctx, q[:p], k[:p], v[:p], cache, prefix=0, f32_cache=f32_cache, **kwargs)
            got = window_attention_gpu(ctx, q[p:p + 1], k[p:p + 1], v[p:p + 1], cache, prefix=p, f32_cache=f32_cache, splits=4, **kwargs)[0]
        else:
            got = window_attention_gpu(ctx, q[:p + 1], k[:p + 1], v[:p + 1], cache, prefix=0, f32_cache=f32_cache, **kwargs)[p]
        close(got, ref[p], 3e-5 if f32_cache else 3e-3, f"key {place} from {p}")
        # the reference itself must show the difference this test is about
        unrot = P.rotate_pairs(t64(ref[p]).reshape(1, heads, vdim), [p], 1000.0, vdim).reshape(heads, vdim)
        turned = P.rotate_pairs(t64(v[place]).reshape(1, heads, vdim), [place], 1000.0, vdim).reshape(heads, vdim)
        is_that_value = float((unrot - turned).abs().max()) < 0.01
        assert is_that_value == seen, (place, p)


# ---- whole models through the engine ----------------------------------------------------------------------------------------------
def config_a():
    """Every size differs from every other; grouped key heads; window 11 with 2 kept tokens; partial rotation; experts with top 2 of 6 and 1 of 4;
    a layer without feed-forward; layer order gru, parallel, parallel, gru."""
    return P.make_config(96, 211, [
        P.mingru_layer(56, P.moe_mlp(20, 6, 2)),
        P.parallel_layer(6, 2, 16, 32, 11, 2, 3, 20, 12, [0.9, 0.96875, 1.0], mlp=P.moe_mlp(28, 4, 1), rot_dims=8, base=300.0, scale=0.21, softcap=8.0,
                         left_scale=0.7, right_scale=1.2),
        P.parallel_layer(2, 2, 24, 10, 40, 0, 2, 12, 28, [0.5, 0.99], mlp=None, softcap=25.0, left_scale=1.3, right_scale=0.6),
        P.mingru_layer(72, P.moe_mlp(12, 3, 3)),
    ], eps=1e-4)


def config_b():
    """One attention head and one retention head, all experts chosen (5 of 5) and one of two, a window of one key beside 5 kept tokens, wide
    cache rows (few tokens per cache page), a window longer than any test context, two parallel layers in a row."""
    return P.make_config(64, 130, [
        P.parallel_layer(1, 1, 500, 24, 1, 5, 1, 40, 8, [0.998], mlp=P.moe_mlp(12, 5, 5), rot_dims=64, scale=0.05, softcap=50.0),
        P.parallel_layer(4, 4, 8, 8, 5000, 1, 4, 8, 8, [0.75, 0.875, 0.9375, 1.0], mlp=P.moe_mlp(20, 2, 1), right_scale=0.5),
        P.mingru_layer(64, None),
    ], eps=1e-6)


def config_c():
    """Sizes that fit no vector width: width 90, head sizes 10 / 6 and 18 / 22 (bf16 rows that start at odd words), odd feed-forwards, 3 experts,
    retention keys of 9 with values of 7, a gru of 35 followed by a single expert (plain products that add straight into the residual)."""
    return P.make_config(90, 77, [
        P.parallel_layer(4, 2, 10, 6, 9, 3, 3, 9, 7, [0.9, 0.95, 0.99], mlp=P.moe_mlp(11, 3, 2), rot_dims=6, base=50.0, scale=0.4, softcap=12.0),
        P.mingru_layer(35, P.moe_mlp(51, 1, 1)),
        P.parallel_layer(2, 1, 18, 22, 30, 1, 1, 33, 5, [0.97], mlp=None, left_scale=0.5, right_scale=2.0),
    ], eps=1e-5)


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
        return P.forward(self.config, self.weights, list(tokens), None, layers).numpy()

    def check(self, got, ref, what):
        got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
        d = (got - ref) - (got - ref).mean(-1, keepdims=True)
        err = np.sqrt((d * d).mean(-1)) / max(float(ref.std()), 1e-6)
        # bf16 products can turn a router's close call the other way for a token, and the recurrent states carry that token's residual on to
        # every later one: there the bound holds for the median row (the f32 engine, where a close call needs a gap of 1e-6, is held to it
        # in every row)
        worst = err.max() if self.f32 else np.quantile(err, 0.5)
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
            close(g, r.numpy(), 3e-5, f"residual after layer {i}")
        else:                                   # see Pair.check: the median row
            row_err = np.abs(g - r.numpy()).max(-1) / np.sqrt((r.numpy() ** 2).mean())
            assert np.quantile(row_err, 0.5) <= 1e-1, f"residual after layer {i}"
    pr.check(got, ref, "prompt logits")
    pr.close()


@pytest.mark.parametrize("make", [config_a, config_b, config_c])
@pytest.mark.parametrize("f32", [True, False])
def test_decode_and_portions_match_the_whole_prompt(ctx, tmp_path, make, f32):
    """Prefill + token-by-token decoding (the window passes over decoded tokens), and portions of 2, 3, 1, 33, 2, ... tokens cut in the middle
    of windows, give the logits of the whole prompt."""
    pr = Pair(ctx, tmp_path, make(), seed=2, f32=f32)
    n = 170
    toks = tokens_for(pr.config, n, 2)
    ref = pr.reference(toks)
    s = pr.engine.slot_acquire()
    parts = [pr.engine.forward_rows(toks[:50], list(range(50)), slot=s)]
    parts += [pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(50, n)]
    pr.check(np.concatenate(parts), ref, "prefill + decode")
    pr.engine.slot_release(s)
    s = pr.engine.slot_acquire()                 # the same slot again: its cache rows and states start over
    parts, p, k = [], 0, 0
    sizes = [2, 3, 1, 33, 2, 70, 9, 32, 2]       # 70 rows after a prefix of 41: the tensor-pipe attention with rows before it in the cache
    while p < n:
        c = min(sizes[k % len(sizes)], n - p)
        parts.append(pr.engine.forward_rows(toks[p:p + c], list(range(c)), slot=s))
        p, k = p + c, k + 1
    pr.check(np.concatenate(parts), ref, "portions")
    pr.engine.slot_release(s)
    s = pr.engine.slot_acquire()                 # from the very first token one by one
    parts = [pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(30)]
    pr.check(np.concatenate(parts), ref[:30], "one by one from the start")
    pr.close()


def test_slots_interleaved_and_reused(ctx, tmp_path):
    """Three unequal requests advance in turns in their own slots; one ends early and its slot serves a new request, whose recurrent states
    and cache must start from nothing. Each equals its solo run."""
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
    """1100 tokens: past the 1024-row pass and, with 500-wide f32 key rows, past the first cache page; the kept tokens stay visible from
    there. Then 40 decoded tokens. Rows just before and after both edges are compared, in the prompt and decoded."""
    pr = Pair(ctx, tmp_path, config_b(), seed=4, f32=True)
    n = 1140
    toks = tokens_for(pr.config, n, 4)
    ref = pr.reference(toks)
    s = pr.engine.slot_acquire()
    rows = [0, 1, 2, 4, 5, 6, 1014, 1015, 1016, 1017, 1022, 1023, 1024, 1025, 1047, 1048, 1049, 1099]
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
    """One parallel layer (window 16, 2 kept tokens) whose attention finds the marker token wherever it is visible: input coordinate 0 is
    non-zero for the marker only and an unrotated key channel reads it; coordinate 1 is the same for every token and the same query channel
    reads it. The retention side is switched off (share 0) so that only the window decides."""
    cfg = P.make_config(48, 60, [P.parallel_layer(2, 1, 8, 12, 16, 2, 1, 4, 4, [0.9], mlp=P.moe_mlp(20, 2, 1), rot_dims=4, scale=1.0, softcap=40.0,
                                                  left_scale=1.0, right_scale=0.0)], eps=1e-6)
    w = {k: v.to(torch.float32) for k, v in P.random_weights(cfg, 5).items()}
    w["embed"][:, 0] = 0.0
    w["embed"][:, 1] = 3.0
    w["embed"][marker] = 0.0
    w["embed"][marker, 0] = 5.0
    w["embed"][marker, 1] = 3.0
    w["l0.norm1"][:] = 0.0
    l = "l0.mix.left."
    w[l + "k.norm"][:] = 1.0
    w[l + "q.norm"][:] = 1.0
    w[l + "temp"][:] = 1.0
    for name, heads in (("k", 1), ("q", 2)):
        w[l + name] *= 0.05
        w[l + name + ".b"][:] = 0.0
        for h in range(heads):
            w[l + name][h * 8 + 7, :] = 0.0
    w[l + "k"][7, 0] = 10.0
    for h in range(2):
        w[l + "q"][h * 8 + 7, 1] = 6.0
    w[l + "o"] *= 3.0
    return cfg, {k: v.to(torch.bfloat16) for k, v in w.items()}, marker


def test_marker_token_inside_and_outside_the_window(ctx, tmp_path):
    """A marker token in a 300-token prompt. Seen from the last rows it matters when it is one of the kept tokens (0, 1) or inside the window
    (285 .. ), and must NOT matter when it is the first token not kept (2) or just outside the window: the engine agrees with the oracle for
    each place, in the prompt's last row and in 10 decoded tokens."""
    cfg, w, marker = marker_model()
    pr = Pair(ctx, tmp_path, cfg, seed=5, f32=True, weights=w)
    base = [x if x != marker else 8 for x in tokens_for(cfg, 300, 5)]
    without = pr.reference(base)
    n, window = 300, 16
    for place, matters in ((0, True), (1, True), (2, False), (n - 11 - window, False), (n - 11 - window + 1, True), (n - 12, True)):
        toks = list(base)
        toks[place] = marker
        ref = pr.reference(toks)
        moved = np.sqrt(((ref[n - 11] - without[n - 11]) ** 2).mean()) / ref.std()
        assert (moved > 0.2) == matters, (place, moved)
        s = pr.engine.slot_acquire()
        got = pr.engine.forward_rows(toks[:n - 10], [n - 11], slot=s)
        dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(n - 10, n)])
        pr.engine.slot_release(s)
        pr.check(got, ref[n - 11:n - 10], f"marker at {place}, prompt")
        pr.check(dec, ref[n - 10:], f"marker at {place}, decoded")
    pr.close()


def test_recurrent_states_carry_a_far_token(ctx, tmp_path):
    """With the attention share at zero and a gru layer, what the first token was still decides the last logits 400 tokens later through the
    retention state (decay 1) -- in one pass, in portions, and decoded."""
    cfg = P.make_config(40, 50, [P.parallel_layer(2, 1, 8, 6, 4, 0, 2, 8, 10, [1.0, 0.999], mlp=None, left_scale=0.0, right_scale=1.0),
                                 P.mingru_layer(24, P.moe_mlp(16, 2, 1))], eps=1e-5)
    pr = Pair(ctx, tmp_path, cfg, seed=8, f32=True)
    toks = tokens_for(cfg, 400, 8)
    other = [(toks[0] + 1) % 50] + toks[1:]
    ref, ref_other = pr.reference(toks), pr.reference(other)
    assert np.abs(ref[-1] - ref_other[-1]).max() > 5e-3 * ref.std(), "the first token must still matter"
    s = pr.engine.slot_acquire()
    parts = [pr.engine.forward_rows(toks[:150], [], slot=s), pr.engine.forward_rows(toks[150:390], [239], slot=s)]
    parts += [pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(390, 400)]
    pr.check(np.concatenate([x for x in parts if x.size]), ref[389:], "first token after 400")
    pr.close()


@pytest.mark.parametrize("graph", [True, False])
def test_greedy_generation_through_the_stream(ctx, tmp_path, graph):
    """prefill() + next()/flush() (the engine's generation entry point; CUDA-graph decode when `graph`), 300 tokens: the window (11 and 40)
    passes over decoded tokens many times. The oracle reads the whole sequence once: every chosen token must be its best at that place within
    the rounding of the bf16 logits the sampler reads."""
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


def test_snapshot_and_restore_rewind_cache_and_states(ctx, tmp_path):
    pr = Pair(ctx, tmp_path, config_c(), seed=7, f32=True)
    toks = tokens_for(pr.config, 60, 7)
    ref = pr.reference(toks)
    pr.engine.forward_rows(toks[:40], [])
    pr.engine.snapshot()
    first = pr.engine.forward_rows(toks[40:], list(range(20)))
    pr.engine.restore()
    again = pr.engine.forward_rows(toks[40:], list(range(20)))
    pr.check(first, ref[40:], "after the snapshot")
    np.testing.assert_array_equal(first, again)
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
        assert np.quantile(errs, 0.5) < 6e-2, errs.max()
