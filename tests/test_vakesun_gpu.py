"""Vakesun (sandwich layers with Dynamic Tanh norms, softmax attention with a half-split rotation, a matrix memory with exponential gates,
windowed latent attention with sinks and head gates that may read another layer's latents, a per-layer token input) on the GPU against the
plain float64 restatement in tests/vakesun_plain.py.

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

from tests import vakesun_plain as P
from uzu_b200 import binding as B
from uzu_b200 import safetensors_io as st
from uzu_b200 import synth

pytestmark = pytest.mark.gpu
F64 = torch.float64
ROOT = Path(__file__).resolve().parents[1]


def t64(a):
    return torch.from_numpy(np.asarray(a)).to(F64)


def bf16_exact(a):
    return synth.st_bits_to_f32(synth.f32_to_bf16_bits(np.asarray(a, np.float32))).reshape(np.shape(a))


def run(ctx, fn, *args):
    with ctx.command_buffer(fn) as cmd:
        cmd.encode(fn, *args)


def close(got, ref, tol, what=""):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    scale = max(float(np.sqrt((ref ** 2).mean())), 1e-6)
    err = float(np.abs(got - ref).max()) / scale
    assert err <= tol, f"{what}: max error {err:.3e} of the rms exceeds {tol:.1e}"


# ---- kernels, one mechanism each ---------------------------------------------------------------------------------------------------
def plain_norm(kind, x, w, b, alpha, eps):
    y = torch.tanh(alpha * x) if kind == 1 else P.unit_rms(x, eps)
    return y * w + b


@pytest.mark.parametrize("rows,n", [(1, 7), (5, 90), (33, 320), (3, 2500)])
@pytest.mark.parametrize("kind,next_kind", [(1, 1), (0, 1), (1, 0), (0, 0)])
def test_norm_then_add_then_next_norm(ctx, rows, n, kind, next_kind):
    """norm alone; norm added into a residual with a factor; the same followed by the next norm of the updated residual. Dynamic Tanh takes
    no mean and no variance: a row of large values saturates at +-w + b."""
    rng = np.random.default_rng(rows + n + kind)
    ld = n + 3
    x = (rng.standard_normal((rows, ld)) * 3).astype(np.float32)
    x[0, : min(4, n)] = [50.0, -50.0, 1e-3, 0.0][: min(4, n)]
    w, b, nw, nb = (rng.standard_normal(n).astype(np.float32) for _ in range(4))
    res = rng.standard_normal((rows, n)).astype(np.float32)
    alpha, nalpha, eps, mult = 0.37, 1.7, 1e-3, 0.3
    bx, bw, bb, bnw, bnb = ctx.upload(x), ctx.upload(w), ctx.upload(b), ctx.upload(nw), ctx.upload(nb)
    normed = plain_norm(kind, t64(x[:, :n]), t64(w), t64(b), alpha, eps)
    out = ctx.upload(np.zeros((rows, n), np.float32))
    a = B.NormAddArgs(input=bx.ptr, weight=bw.ptr, bias=bb.ptr, output=out.ptr, rows=rows, n=n, in_stride=ld, kind=kind, alpha=alpha, epsilon=eps)
    run(ctx, "uzu_norm_add_encode", C.byref(a))
    close(out.numpy(np.float32, (rows, n)), normed.numpy(), 3e-6, "norm alone")
    updated = t64(res) + mult * normed
    for with_next in (False, True):
        br, out = ctx.upload(res), ctx.upload(np.zeros((rows, n), np.float32))
        a = B.NormAddArgs(input=bx.ptr, weight=bw.ptr, bias=bb.ptr, residual=br.ptr, output=out.ptr if with_next else 0, next_weight=bnw.ptr, next_bias=bnb.ptr,
                          rows=rows, n=n, in_stride=ld, kind=kind, next_kind=next_kind, alpha=alpha, epsilon=eps, mult=mult, next_alpha=nalpha)
        run(ctx, "uzu_norm_add_encode", C.byref(a))
        close(br.numpy(np.float32, (rows, n)), updated.numpy(), 3e-6, "residual")
        if with_next:
            close(out.numpy(np.float32, (rows, n)), plain_norm(next_kind, updated, t64(nw), t64(nb), nalpha, eps).numpy(), 5e-6, "next norm")


@pytest.mark.parametrize("f32_table", [True, False])
def test_token_gate_and_scaled_embedding(ctx, f32_table):
    rng = np.random.default_rng(1)
    rows, n, vocab, stride, column = 9, 13, 40, 45, 26
    z = (rng.standard_normal((rows, n)) * 3).astype(np.float32)
    table = bf16_exact(rng.standard_normal((vocab, stride)))
    toks = rng.integers(0, vocab, rows).astype(np.uint32)
    bz, bt, bk, bo = ctx.upload(z), ctx.upload(table if f32_table else synth.f32_to_bf16_bits(table).reshape(table.shape)), ctx.upload(toks), ctx.upload(np.zeros_like(z))
    dt = B.DT_F32 if f32_table else B.DT_BF16
    a = B.TokenGateArgs(z=bz.ptr, token_ids=bk.ptr, table=bt.ptr, out=bo.ptr, rows=rows, n=n, vocab=vocab, table_stride=stride, column=column, weights_dt=dt)
    run(ctx, "uzu_token_gate_encode", C.byref(a))
    close(bo.numpy(np.float32, z.shape), (P.gelu_tanh(t64(z)) * t64(table[toks, column:column + n])).numpy(), 3e-6, "gelu_tanh(z) * table row")
    out = ctx.upload(np.zeros((rows, stride), np.float32))
    run(ctx, "uzu_embedding_f32_scaled_encode", bk.ptr, bt.ptr, dt, out.ptr, rows, vocab, stride, 0.375)
    np.testing.assert_array_equal(out.numpy(np.float32, (rows, stride)), table[toks] * np.float32(0.375))


@pytest.mark.parametrize("m,n,k", [(1, 90, 77), (1, 320, 2048), (5, 33, 200), (40, 130, 96), (100, 64, 64)])
@pytest.mark.parametrize("f32_weights", [True, False])
def test_product_epilogues_norm_add_next_norm_and_token_gate(ctx, m, n, k, f32_weights):
    """The output projection of a sandwich sublayer in short passes: product -> Dynamic Tanh norm -> residual add with a factor -> the next
    reader's norm, in the product's epilogue (one-row, few-row, tile and tensor-pipe kernels); and the token-gated gelu unit as an epilogue."""
    rng = np.random.default_rng(m + n)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = bf16_exact(rng.standard_normal((n, k)) / 4)
    pw, pb, nw, nb = (rng.standard_normal(n).astype(np.float32) for _ in range(4))
    res = rng.standard_normal((m, n)).astype(np.float32)
    act = t64(x) if f32_weights or m < 32 else t64(bf16_exact(x))
    y = act @ t64(w).T
    updated = t64(res) + 0.3 * (torch.tanh(0.8 * y) * t64(pw) + t64(pb))
    bx, bw = ctx.upload(x), ctx.upload(w if f32_weights else synth.f32_to_bf16_bits(w).reshape(w.shape))
    dt = B.DT_F32 if f32_weights else B.DT_BF16
    bpw, bpb, bnw, bnb, br, bo = ctx.upload(pw), ctx.upload(pb), ctx.upload(nw), ctx.upload(nb), ctx.upload(res), ctx.upload(np.zeros((m, n), np.float32))
    a = B.DenseLinearArgs(a=bx.ptr, w=bw.ptr, d=br.ptr, m=m, n=n, k=k, lda=k, ldd=n, batch=1, weights_dt=dt, scale=1.0, post_weight=bpw.ptr, post_bias=bpb.ptr,
                          next_weight=bnw.ptr, next_bias=bnb.ptr, next_out=bo.ptr, post_alpha=0.8, post_mult=0.3, next_alpha=1.4)
    run(ctx, "uzu_dense_linear_encode", C.byref(a))
    close(br.numpy(np.float32, (m, n)), updated.numpy(), 1e-5, "residual")
    close(bo.numpy(np.float32, (m, n)), (torch.tanh(1.4 * updated) * t64(nw) + t64(nb)).numpy(), 1e-5, "next norm")
    vocab, stride, column = 30, n + 7, 5
    table = bf16_exact(rng.standard_normal((vocab, stride)))
    toks = rng.integers(0, vocab, m).astype(np.uint32)
    bt, bk, bd = ctx.upload(table if f32_weights else synth.f32_to_bf16_bits(table).reshape(table.shape)), ctx.upload(toks), ctx.upload(np.zeros((m, n), np.float32))
    a = B.DenseLinearArgs(a=bx.ptr, w=bw.ptr, d=bd.ptr, m=m, n=n, k=k, lda=k, ldd=n, batch=1, weights_dt=dt, scale=1.0, token_ids=bk.ptr, token_table=bt.ptr,
                          token_gate_dt=dt, token_table_stride=stride, token_column=column, token_vocab=vocab)
    run(ctx, "uzu_dense_linear_encode", C.byref(a))
    close(bd.numpy(np.float32, (m, n)), (P.gelu_tanh(y) * t64(table[toks, column:column + n])).numpy(), 1e-5, "token gate")


def test_latent_prepare_norms_cache_row_and_query_latent_in_one_launch(ctx):
    rng = np.random.default_rng(2)
    rows, rank, q_rank, ld, prefix = 7, 27, 19, 60, 3
    proj = (rng.standard_normal((rows, ld)) * 3).astype(np.float32)           # [query latent | kv latent | other]
    cw = (1 + 0.3 * rng.standard_normal(rank)).astype(np.float32)
    qw = (1 + 0.3 * rng.standard_normal(q_rank)).astype(np.float32)
    bp, bcw, bqw = ctx.upload(proj), ctx.upload(cw), ctx.upload(qw)
    cache, qo = ctx.upload(np.zeros((prefix + rows, rank), np.float32)), ctx.upload(np.zeros((rows, q_rank), np.float32))
    a = B.LatentPrepareArgs(kv=bp.ptr + 4 * q_rank, cache=cache.ptr, latent_scales=bcw.ptr, rows=rows, heads=4, dim=8, rot_dim=0, rank=rank, kv_stride=ld,
                            prefix=prefix, cache_dt=B.DT_F32, epsilon=1e-4, q_latent=bp.ptr, q_latent_scales=bqw.ptr, q_latent_out=qo.ptr, q_rank=q_rank, q_latent_stride=ld)
    run(ctx, "uzu_latent_prepare_encode", C.byref(a))
    got = cache.numpy(np.float32, (prefix + rows, rank))
    assert not got[:prefix].any()
    close(got[prefix:], (P.unit_rms(t64(proj[:, q_rank:q_rank + rank]), 1e-4) * t64(cw)).numpy(), 3e-6, "cache rows")
    close(qo.numpy(np.float32, (rows, q_rank)), (P.unit_rms(t64(proj[:, :q_rank]), 1e-4) * t64(qw)).numpy(), 3e-6, "query latent")


def rot_table(positions, rot):
    f, mult = P.rot_frequencies(rot)
    ang = np.arange(positions, dtype=np.float64)[:, None] * np.asarray(f, np.float64)[None, :]
    return (np.cos(ang) * mult).astype(np.float32), (np.sin(ang) * mult).astype(np.float32)


def attention_gpu(ctx, q, k, v, cache, *, prefix, heads, kv_heads, dim, vdim, rot, scale, qw, kw, eps, f32_cache=True, splits=0):
    """One pass of T tokens at positions prefix ..; `cache` = (keys, values) device buffers that already hold positions < prefix."""
    T = q.shape[0]
    pairs = rot["dims"] // 2 if rot else 0
    cs, sn = rot_table(prefix + T, rot) if rot else (np.zeros(1, np.float32),) * 2
    bq, bk, bv = ctx.upload(q.astype(np.float32)), ctx.upload(k.astype(np.float32)), ctx.upload(v.astype(np.float32))
    bqw, bkw, bcs, bsn = ctx.upload(qw.astype(np.float32)), ctx.upload(kw.astype(np.float32)), ctx.upload(cs), ctx.upload(sn)
    query, out = ctx.upload(np.zeros((T, heads * dim), np.float32)), ctx.upload(np.zeros((T, heads * vdim), np.float32))
    dt = B.DT_F32 if f32_cache else B.DT_BF16
    pa = B.WindowAttentionPrepareArgs(q=bq.ptr, k=bk.ptr, v=bv.ptr, q_scales=bqw.ptr, k_scales=bkw.ptr, query=query.ptr, keys=cache[0].ptr, values=cache[1].ptr,
                                      cosines=bcs.ptr, sines=bsn.ptr, rows=T, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot_pairs=pairs,
                                      prefix=prefix, cache_dt=dt, epsilon=eps, rot_halves=1)
    run(ctx, "uzu_window_attention_prepare_encode", C.byref(pa))
    parts = ctx.upload(np.zeros(max(T * heads * max(splits, 1) * (vdim + 2), 4), np.float32))
    tickets = ctx.upload(np.zeros(T * heads, np.uint32))
    aa = B.WindowAttentionArgs(query=query.ptr, keys=cache[0].ptr, values=cache[1].ptr, out=out.ptr, partials=parts.ptr, tickets=tickets.ptr, rows=T, heads=heads,
                               kv_heads=kv_heads, dim=dim, vdim=vdim, prefix=prefix, cache_dt=dt, scale=scale, splits=splits)
    run(ctx, "uzu_window_attention_encode", C.byref(aa))
    return out.numpy(np.float32, (T, heads * vdim))


def attention_plain(q, k, v, *, heads, kv_heads, dim, vdim, rot, scale, qw, kw, eps, round_cache=False):
    T = q.shape[0]
    pos = list(range(T))
    qq = P.unit_rms(t64(q).reshape(T, heads, dim), eps) * t64(qw)
    kk = P.unit_rms(t64(k).reshape(T, kv_heads, dim), eps) * t64(kw)
    if rot:
        qq, kk = P.rotate_halves(qq, pos, rot), P.rotate_halves(kk, pos, rot)
    vv = t64(v).reshape(T, kv_heads, vdim)
    if round_cache:
        kk, vv = t64(bf16_exact(kk.numpy())), t64(bf16_exact(vv.numpy()))
    return P.softmax_attention(qq, kk, vv, pos, pos, scale).reshape(T, heads * vdim).numpy()


def new_cache(ctx, positions, kv_heads, dim, vdim, f32_cache):
    dt = np.float32 if f32_cache else np.uint16
    return ctx.upload(np.zeros((positions, kv_heads * dim), dt)), ctx.upload(np.zeros((positions, kv_heads * vdim), dt))


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


@pytest.mark.parametrize("T,prefix,heads,kv_heads,dim,vdim,rot", [
    (40, 0, 4, 2, 16, 24, {"base": 500.0, "dims": 16}), (9, 31, 6, 2, 48, 80, {"base": 1e4, "dims": 20, "scaling": YARN}),
    (70, 5, 2, 2, 10, 6, {"base": 50.0, "dims": 4}), (130, 20, 2, 1, 128, 128, {"base": 1e6, "dims": 64, "scaling": YARN}), (20, 0, 1, 1, 9, 14, None),
    (200, 300, 4, 1, 64, 32, {"base": 1e4, "dims": 64, "scaling": {"factor": 16.0, "original": 32, "fast": 4.0, "slow": 2.0}})])
@pytest.mark.parametrize("f32_cache", [True, False])
def test_attention_with_half_split_rotation(ctx, T, prefix, heads, kv_heads, dim, vdim, rot, f32_cache):
    """Channel i turns with channel i + dims / 2 (not with its neighbour), channels from dims on pass unchanged; blended frequencies and the
    factor on cos / sin; grouped heads; prompt rows and rows after a prefix, with key splits, on the plain and the tensor-pipe kernel."""
    rng = np.random.default_rng(T + dim)
    n = prefix + T
    q, k, v = (rng.standard_normal((n, w)).astype(np.float32) * 2 for w in (heads * dim, kv_heads * dim, kv_heads * vdim))
    kwargs = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=rot, scale=dim ** -0.5 * 1.3, qw=1 + 0.3 * rng.standard_normal(dim),
                  kw=1 + 0.3 * rng.standard_normal(dim), eps=1e-5)
    ref = attention_plain(q, k, v, round_cache=not f32_cache, **kwargs)
    for splits in (0, 3, 64):
        cache = new_cache(ctx, n, kv_heads, dim, vdim, f32_cache)
        if prefix:
            attention_gpu(ctx, q[:prefix], k[:prefix], v[:prefix], cache, prefix=0, f32_cache=f32_cache, **kwargs)
        got = attention_gpu(ctx, q[prefix:], k[prefix:], v[prefix:], cache, prefix=prefix, f32_cache=f32_cache, splits=splits, **kwargs)
        # (bf16 caches: a key or value element that rounds the other way in f32 than in the float64 restatement moves an output by a few 1e-3)
        close(got, ref[prefix:], 3e-5 if f32_cache else 1e-2, f"splits {splits}")


@pytest.mark.parametrize("T,prefix,heads,dim,vdim,window", [(40, 0, 3, 16, 24, 7), (200, 0, 4, 64, 32, 70), (150, 130, 2, 128, 128, 50), (70, 64, 2, 16, 16, 0), (5, 90, 2, 10, 6, 33)])
@pytest.mark.parametrize("f32_cache", [True, False])
def test_softmax_attention_with_sink_and_head_gate(ctx, T, prefix, heads, dim, vdim, window, f32_cache):
    """The window-attention kernels (plain with key splits, and the tensor-pipe one for bf16 passes of >= 64 rows) with a sink term per head
    and a sigmoid gate per head, as the expanded form of latent attention uses them; the caches are addressed from a later row on (the
    pointer names where row 0 WOULD be), as a temporary copy of the visible range is."""
    rng = np.random.default_rng(T + dim)
    n = prefix + T
    q = rng.standard_normal((n, heads, dim)).astype(np.float32)
    k, v = rng.standard_normal((n, heads, dim)).astype(np.float32), rng.standard_normal((n, heads, vdim)).astype(np.float32)
    if not f32_cache:
        k, v = bf16_exact(k), bf16_exact(v)
    sink = (rng.standard_normal(heads) * 2).astype(np.float32)
    gate = (rng.standard_normal((n, heads + 2)) * 2).astype(np.float32)
    pos = list(range(n))
    ref = (P.softmax_attention(t64(q), t64(k), t64(v), pos, pos, 0.3, window=window, sink=t64(sink)) * torch.sigmoid(t64(gate[:, :heads]))[:, :, None]).numpy()
    lo = (max(0, prefix + 1 - window) if window else 0) // 64 * 64
    as_cache = (lambda x: x) if f32_cache else (lambda x: synth.f32_to_bf16_bits(x).reshape(x.shape))
    bk, bv = ctx.upload(as_cache(k[lo:].reshape(n - lo, -1))), ctx.upload(as_cache(v[lo:].reshape(n - lo, -1)))
    size = 4 if f32_cache else 2
    bq, bs, bg = ctx.upload(q[prefix:]), ctx.upload(sink), ctx.upload(gate[prefix:])
    for splits in (1, 3):
        out, parts, tickets = ctx.upload(np.zeros((T, heads * vdim), np.float32)), ctx.upload(np.zeros(T * heads * splits * (vdim + 2), np.float32)), ctx.upload(np.zeros(T * heads, np.uint32))
        a = B.WindowAttentionArgs(query=bq.ptr, keys=bk.ptr - lo * heads * dim * size, values=bv.ptr - lo * heads * vdim * size, out=out.ptr, partials=parts.ptr,
                                  tickets=tickets.ptr, rows=T, heads=heads, kv_heads=heads, dim=dim, vdim=vdim, prefix=prefix,
                                  cache_dt=B.DT_F32 if f32_cache else B.DT_BF16, window=window, scale=0.3, splits=splits, sinks=bs.ptr, head_gate=bg.ptr,
                                  head_gate_stride=heads + 2)
        run(ctx, "uzu_window_attention_encode", C.byref(a))
        # (the tensor-pipe kernel carries query and weights as two bf16 numbers each: 2^-16 relative)
        close(out.numpy(np.float32, (T, heads, vdim)), ref[prefix:], 3e-5 if f32_cache else 1e-4, f"splits {splits}")


@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (300, 200, 192), (1000, 96, 512)])
def test_product_of_bf16_rows_on_tensor_memory_and_bf16_copy(ctx, m, n, k):
    """A = rows of a bf16 cache, read as they are by the tensor-memory product; the f32 result copied to bf16 column ranges."""
    rng = np.random.default_rng(m)
    x, w = bf16_exact(rng.standard_normal((m, k))), bf16_exact(rng.standard_normal((n, k)) / 8)
    bx, bw = ctx.upload(synth.f32_to_bf16_bits(x).reshape(x.shape)), ctx.upload(synth.f32_to_bf16_bits(w).reshape(w.shape))
    bd, ws = ctx.upload(np.zeros((m, n), np.float32)), ctx.upload(np.zeros(16, np.uint16))
    a = B.DenseLinearArgs(a=bx.ptr, w=bw.ptr, d=bd.ptr, workspace=ws.ptr, m=m, n=n, k=k, lda=k, ldd=n, batch=1, weights_dt=B.DT_BF16, scale=1.0, a_bf16=1)
    run(ctx, "uzu_dense_linear_encode", C.byref(a))
    ref = (t64(x) @ t64(w).T).numpy()
    close(bd.numpy(np.float32, (m, n)), ref, 5e-6, "product")
    assert ctx.lib.uzu_debug_dense_umma_error() == 0
    half = n // 2
    bo = ctx.upload(np.zeros((m, n - half), np.uint16))
    run(ctx, "uzu_rows_to_bf16_encode", bd.ptr + 4 * half, n, bo.ptr, m, n - half)
    np.testing.assert_array_equal(bo.numpy(np.uint16, (m, n - half)), synth.f32_to_bf16_bits(bd.numpy(np.float32, (m, n))[:, half:]).reshape(m, n - half))


def test_rotation_layout_is_halves_not_neighbours(ctx):
    """One query / key pair with a single non-zero channel each: under the half-split layout channel 0 pairs with channel dims / 2."""
    dim, rot = 8, {"base": 10.0, "dims": 8}
    q = np.zeros((3, dim), np.float32); q[:, 0] = 1.0
    cache = new_cache(ctx, 3, 1, dim, 4, True)
    attention_gpu(ctx, q, q, np.ones((3, 4), np.float32), cache, prefix=0, heads=1, kv_heads=1, dim=dim, vdim=4, rot=rot, scale=1.0, qw=np.ones(dim), kw=np.ones(dim), eps=0.0)
    keys = cache[0].numpy(np.float32, (3, dim))
    norm = math.sqrt(dim)                                     # unit rms of a one-hot row
    for p in range(3):
        assert abs(keys[p, 0] - norm * math.cos(p)) < 1e-5 and abs(keys[p, 4] - norm * math.sin(p)) < 1e-5
        assert np.abs(np.delete(keys[p], [0, 4])).max() == 0.0


@pytest.mark.parametrize("f32_cache", [True, False])
@pytest.mark.parametrize("decoded", [True, False])
def test_attention_finds_one_far_key_among_hundreds(ctx, f32_cache, decoded):
    """Among 900 keys one stands out (a large channel outside the rotated ones that only it and the query have): from the last position
    the output is that key's value, wherever it sits: position 0, 1, the rows around a tile's edge, far back, the row before the query."""
    heads, kv, dim, vdim, n = 2, 1, 16, 16, 900
    rng = np.random.default_rng(3)
    rot = {"base": 1000.0, "dims": 12}
    for place in (0, 1, 63, 64, 65, 511, n - 2):
        q = np.zeros((n, heads * dim), np.float32)
        k = rng.standard_normal((n, kv * dim)).astype(np.float32) * 0.05
        v = rng.standard_normal((n, kv * vdim)).astype(np.float32)
        q[:, dim - 1] = q[:, 2 * dim - 1] = 1.0
        k[:, dim - 1] = 0.0
        k[place, dim - 1] = 1.0
        kwargs = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, rot=rot, scale=3.0, qw=np.ones(dim), kw=np.ones(dim), eps=1e-6)
        ref = attention_plain(q, k, v, round_cache=not f32_cache, **kwargs)
        cache = new_cache(ctx, n, kv, dim, vdim, f32_cache)
        if decoded:
            attention_gpu(ctx, q[:n - 1], k[:n - 1], v[:n - 1], cache, prefix=0, f32_cache=f32_cache, **kwargs)
            got = attention_gpu(ctx, q[n - 1:], k[n - 1:], v[n - 1:], cache, prefix=n - 1, f32_cache=f32_cache, splits=7, **kwargs)[0]
        else:
            got = attention_gpu(ctx, q, k, v, cache, prefix=0, f32_cache=f32_cache, **kwargs)[n - 1]
        close(got, ref[n - 1], 3e-5 if f32_cache else 3e-3, f"key {place}")
        assert np.abs(ref[n - 1, :vdim] - v[place]).max() < 0.02, "the reference itself must have found the key"


@pytest.mark.parametrize("rows,heads,cap", [(1, 3, 15.0), (31, 2, 2.0), (32, 1, 15.0), (33, 5, 0.0), (300, 4, 6.0)])
def test_exponential_gates_and_running_maximum(ctx, rows, heads, cap):
    """Log gates with the cap, the running maximum carried over launches, and its start at 0 (not at minus infinity): with very negative
    input gates the first maxima are f_1, f_1 + f_2, ... and the gain exp(i - m) stays tiny."""
    rng = np.random.default_rng(rows)
    ld = 2 * heads + 3
    pre = (rng.standard_normal((rows, ld)) * 4).astype(np.float32)
    pre[: min(rows, 3), :heads] = -9.0
    i_log, f_log = P.mlstm_gates(t64(pre[:, :heads]), t64(pre[:, heads:2 * heads]), cap) if cap else (t64(pre[:, :heads]), torch.nn.functional.logsigmoid(t64(pre[:, heads:2 * heads])))
    m = torch.zeros(heads, dtype=F64)
    decay, gain, floor = [], [], []
    for t in range(rows):
        m_new = torch.maximum(f_log[t] + m, i_log[t])
        decay.append(torch.exp(f_log[t] + m - m_new)); gain.append(torch.exp(i_log[t] - m_new)); floor.append(torch.exp(-m_new))
        m = m_new
    for cut in sorted({rows, rows // 3, 1} - {0}):
        bp, bs = ctx.upload(pre), ctx.upload(np.zeros(heads, np.float32))
        bd, bg, bf = (ctx.upload(np.zeros((rows, heads), np.float32)) for _ in range(3))
        for lo, hi in ((0, cut), (cut, rows)):
            if hi > lo:
                a = B.ExpGatesArgs(i_pre=bp.ptr + 4 * lo * ld, f_pre=bp.ptr + 4 * (lo * ld + heads), state=bs.ptr, token_decay=bd.ptr + 4 * lo * heads,
                                   token_gain=bg.ptr + 4 * lo * heads, floor=bf.ptr + 4 * lo * heads, rows=hi - lo, heads=heads, i_stride=ld, f_stride=ld, cap=cap)
                run(ctx, "uzu_exp_gates_encode", C.byref(a))
        for name, buf, ref in (("decay", bd, decay), ("gain", bg, gain), ("floor", bf, floor)):
            close(buf.numpy(np.float32, (rows, heads)), torch.stack(ref).numpy(), 1e-5, f"{name} cut at {cut}")
        close(bs.numpy(np.float32, (heads,)), m.numpy(), 3e-6, "running maximum")


def mlstm_gpu(ctx, q, k, v, i_pre, f_pre, gate, weight, state, m_state, *, heads, dim, vdim, cap, eps, cuts):
    """exp gates -> gated linear recurrence with its normaliser column -> division, unit RMS, weight, sigmoid gate; in launches cut at `cuts`"""
    rows = q.shape[0]
    bq, bk, bv, bi, bf, bgt, bw = (ctx.upload(np.ascontiguousarray(x, np.float32)) for x in (q, k, v, i_pre, f_pre, gate, weight))
    bs, bm = ctx.upload(np.ascontiguousarray(state, np.float32)), ctx.upload(np.ascontiguousarray(m_state, np.float32))
    fac = [ctx.upload(np.zeros((rows, heads), np.float32)) for _ in range(4)]
    raw, out = ctx.upload(np.zeros((rows, heads * vdim), np.float32)), ctx.upload(np.zeros((rows, heads * vdim), np.float32))
    edges = [0] + list(cuts) + [rows]
    for lo, hi in zip(edges[:-1], edges[1:]):
        if hi <= lo:
            continue
        n, oh = hi - lo, 4 * lo * heads
        ga = B.ExpGatesArgs(i_pre=bi.ptr + oh, f_pre=bf.ptr + oh, state=bm.ptr, token_decay=fac[0].ptr + oh, token_gain=fac[1].ptr + oh, floor=fac[2].ptr + oh,
                            rows=n, heads=heads, cap=cap)
        run(ctx, "uzu_exp_gates_encode", C.byref(ga))
        ra = B.RetentionArgs(q=bq.ptr + 4 * lo * heads * dim, k=bk.ptr + 4 * lo * heads * dim, v=bv.ptr + 4 * lo * heads * vdim, state=bs.ptr,
                             out=raw.ptr + 4 * lo * heads * vdim, rows=n, heads=heads, dim=dim, vdim=vdim, key_scale=1.0, query_scale=dim ** -0.5,
                             token_decay=fac[0].ptr + oh, token_gain=fac[1].ptr + oh, norm_out=fac[3].ptr + oh)
        run(ctx, "uzu_retention_encode", C.byref(ra))
        na = B.HeadNormGateArgs(x=raw.ptr + 4 * lo * heads * vdim, scales=bw.ptr, gate=bgt.ptr + 4 * lo * heads * vdim, out=out.ptr + 4 * lo * heads * vdim, rows=n,
                                heads=heads, dim=vdim, normalize=1, epsilon=eps, gate_op=0, denom=fac[3].ptr + oh, denom_floor=fac[2].ptr + oh, denom_epsilon=1e-6)
        run(ctx, "uzu_head_norm_gate_encode", C.byref(na))
    return out.numpy(np.float32, (rows, heads * vdim)), bs.numpy(np.float32, np.shape(state)), bm.numpy(np.float32, (heads,))


@pytest.mark.parametrize("rows,heads,dim,vdim", [(1, 3, 64, 48), (17, 2, 9, 7), (100, 2, 128, 64), (40, 1, 48, 96), (33, 5, 20, 31), (50, 2, 16, 32)])
def test_matrix_memory_against_the_token_by_token_scan(ctx, rows, heads, dim, vdim):
    """Key size != value size, odd sizes, a value width that fills its last block of 32 columns (the normaliser then opens one more); one
    launch equals launches of 1, 2 and the rest with matrix, normaliser and maximum carried; a state that is not zero at the start."""
    rng = np.random.default_rng(rows + dim)
    q, k = (rng.standard_normal((rows, heads * dim)).astype(np.float32) for _ in range(2))
    v, gate = (rng.standard_normal((rows, heads * vdim)).astype(np.float32) for _ in range(2))
    i_pre, f_pre = (rng.standard_normal((rows, heads)) * 3).astype(np.float32), (2 + rng.standard_normal((rows, heads)) * 3).astype(np.float32)
    weight = (1 + 0.3 * rng.standard_normal(heads * vdim)).astype(np.float32)
    S0, n0, m0 = rng.standard_normal((heads, dim, vdim)).astype(np.float32), rng.standard_normal((heads, dim)).astype(np.float32), rng.standard_normal(heads).astype(np.float32)
    cap, eps = 15.0, 1e-5
    il, fl = P.mlstm_gates(t64(i_pre), t64(f_pre), cap)
    o, (S, nn, m) = P.mlstm_scan(t64(q).reshape(rows, heads, dim) * dim ** -0.5, t64(k).reshape(rows, heads, dim), t64(v).reshape(rows, heads, vdim), il, fl,
                                 (t64(S0), t64(n0), t64(m0)))
    ref = (P.unit_rms(o, eps).reshape(rows, -1) * t64(weight) * torch.sigmoid(t64(gate))).numpy()
    state0 = np.concatenate([S0, n0[:, :, None]], axis=2)                 # [heads, dim, vdim + 1]: the normaliser is the last column
    for cuts in ((), (1,), (1, 3), (rows // 2,)):
        cuts = tuple(c for c in cuts if c < rows)
        got, state, mm = mlstm_gpu(ctx, q, k, v, i_pre, f_pre, gate, weight, state0, m0, heads=heads, dim=dim, vdim=vdim, cap=cap, eps=eps, cuts=cuts)
        close(got, ref, 2e-5, f"outputs, cuts {cuts}")
        close(state[:, :, :vdim], S.numpy(), 2e-5, "matrix")
        close(state[:, :, vdim], nn.numpy(), 2e-5, "normaliser")
        close(mm, m.numpy(), 3e-6, "maximum")


def test_matrix_memory_remembers_a_far_token_and_floors_its_denominator(ctx):
    """600 tokens whose keys are orthogonal to the query except token 3, forget gates wide open: the output direction is that token's
    value. And with every key orthogonal to the query the normaliser product is 0, so the denominator is exp(-m) + 1e-6, not 0."""
    rows, dim, vdim = 600, 16, 8
    rng = np.random.default_rng(0)
    q = np.zeros((rows, dim), np.float32); k = np.zeros((rows, dim), np.float32)
    v = rng.standard_normal((rows, vdim)).astype(np.float32)
    q[:, 0] = 1.0; k[:, 1] = 1.0; k[3, 0] = 4.0
    i_pre, f_pre = np.zeros((rows, 1), np.float32), np.full((rows, 1), 14.0, np.float32)
    one = np.ones((rows, vdim), np.float32) * 30.0            # sigmoid gate ~ 1
    got, _, _ = mlstm_gpu(ctx, q, k, v, i_pre, f_pre, one, np.ones(vdim, np.float32), np.zeros((1, dim, vdim + 1), np.float32), np.zeros(1, np.float32),
                          heads=1, dim=dim, vdim=vdim, cap=15.0, eps=1e-6, cuts=(200,))
    unit = v[3] / np.sqrt((v[3] ** 2).mean())
    close(got[599], unit, 1e-4, "far token")
    assert np.abs(got[2]).max() == 0.0 and np.isfinite(got).all()


def latent_gpu(ctx, query, cache, *, prefix, heads, rank, scale, window, sink, gate, f32_cache, splits):
    T = query.shape[0]
    bq, bo = ctx.upload(query.astype(np.float32)), ctx.upload(np.zeros((T, heads * rank), np.float32))
    bs = ctx.upload(np.asarray(sink, np.float32)) if sink is not None else None
    bg = ctx.upload(np.ascontiguousarray(gate, np.float32)) if gate is not None else None
    parts = ctx.upload(np.zeros(max(T * heads * max(splits, 1) * (rank + 2), 4), np.float32))
    a = B.LatentAttentionArgs(query=bq.ptr, cache=cache.ptr, out=bo.ptr, partials=parts.ptr, rows=T, heads=heads, rank=rank, rot_dim=0, prefix=prefix,
                              cache_dt=B.DT_F32 if f32_cache else B.DT_BF16, scale=scale, splits=splits, sinks=bs.ptr if bs else 0, head_gate=bg.ptr if bg else 0,
                              window=window, head_gate_stride=gate.shape[1] if gate is not None else 0)
    run(ctx, "uzu_latent_attention_encode", C.byref(a))
    return bo.numpy(np.float32, (T, heads, rank))


def latent_plain(query, c, *, heads, scale, window, sink, gate):
    """query [n, heads, rank] (already folded with the key up-projection), c [n, rank]: every head scores against and sums the same rows"""
    n = c.shape[0]
    pos = list(range(n))
    o = P.softmax_attention(t64(query), t64(c)[:, None, :], t64(c)[:, None, :], pos, pos, scale, window=window, sink=t64(sink) if sink is not None else None)
    if gate is not None:
        o = o * torch.sigmoid(t64(gate[:, :heads]))[:, :, None]
    return o.numpy()


@pytest.mark.parametrize("T,prefix,heads,rank,window", [(40, 0, 3, 16, 7), (1, 99, 9, 128, 72), (70, 5, 2, 27, 1), (33, 64, 8, 64, 33), (5, 300, 6, 96, 0),
                                                         (200, 0, 4, 32, 64), (2, 31, 1, 512, 32), (64, 130, 10, 40, 100)])
@pytest.mark.parametrize("f32_cache", [True, False])
def test_latent_attention_window_sink_and_head_gate(ctx, T, prefix, heads, rank, window, f32_cache):
    """A sliding window (1 key, shorter and longer than the context, none), a sink per head that only enlarges the denominator, a gate per
    head; rows after a prefix; key splits of 0 / 2 / 5 / 64; more heads than one CTA's eight; rows that fit no vector width."""
    rng = np.random.default_rng(T + rank)
    n = prefix + T
    c = bf16_exact(rng.standard_normal((n, rank))) if not f32_cache else rng.standard_normal((n, rank)).astype(np.float32)
    query = rng.standard_normal((n, heads, rank)).astype(np.float32)
    sink = (rng.standard_normal(heads) * 2).astype(np.float32)
    gate = (rng.standard_normal((n, heads + 3)) * 2).astype(np.float32)
    scale = 1.5 / math.sqrt(rank)
    ref = latent_plain(query, c, heads=heads, scale=scale, window=window, sink=sink, gate=gate)
    cache = ctx.upload(c if f32_cache else synth.f32_to_bf16_bits(c).reshape(c.shape))
    for splits in (0, 2, 5, 64):
        got = latent_gpu(ctx, query[prefix:], cache, prefix=prefix, heads=heads, rank=rank, scale=scale, window=window, sink=sink, gate=gate[prefix:],
                         f32_cache=f32_cache, splits=splits)
        close(got, ref[prefix:], 2e-5, f"splits {splits}")
    plain = latent_gpu(ctx, query[prefix:], cache, prefix=prefix, heads=heads, rank=rank, scale=scale, window=window, sink=None, gate=None, f32_cache=f32_cache, splits=0)
    close(plain, latent_plain(query, c, heads=heads, scale=scale, window=window, sink=None, gate=None)[prefix:], 2e-5, "no sink, no gate")


def test_sink_counts_once_and_is_not_scaled(ctx):
    """One visible key with score 0 and a sink s: the weight of the key is 1 / (1 + e^s), whatever the scale."""
    c = np.zeros((1, 8), np.float32); c[0, 0] = 1.0
    q = np.zeros((1, 2, 8), np.float32)
    cache = ctx.upload(c)
    got = latent_gpu(ctx, q, cache, prefix=0, heads=2, rank=8, scale=123.0, window=4, sink=[0.0, math.log(3.0)], gate=None, f32_cache=True, splits=0)
    np.testing.assert_allclose(got[0, :, 0], [0.5, 0.25], rtol=1e-6)


@pytest.mark.parametrize("f32_cache", [True, False])
@pytest.mark.parametrize("decoded", [True, False])
def test_one_latent_row_just_inside_and_just_outside_the_window(ctx, f32_cache, decoded):
    """Among 700 cached rows one stands out (the query is aligned with it). From position p the output is that row when p - j < window and
    not otherwise: the row sits at the window's first place, one before it, at a tile's edge inside the window, or is the query's own."""
    heads, rank, window, n = 2, 32, 72, 700
    rng = np.random.default_rng(4)
    for place, p, seen in [(n - window, n - 1, True), (n - window - 1, n - 1, False), (0, n - 1, False), (n - 1, n - 1, True), (500 - window + 1, 500, True),
                           (500 - window, 500, False), (639, n - 1, True), (640, n - 1, True), (0, window - 1, True), (0, window, False)]:
        c = rng.standard_normal((n, rank)).astype(np.float32) * 0.05
        c[:, 0] = 0.0
        c[place, 0] = 4.0
        if not f32_cache:
            c = bf16_exact(c)
        query = np.zeros((n, heads, rank), np.float32)
        query[:, :, 0] = 3.0
        sink = np.array([-1.0, 0.5], np.float32)
        ref = latent_plain(query, c, heads=heads, scale=1.0, window=window, sink=sink, gate=None)
        cache = ctx.upload(c if f32_cache else synth.f32_to_bf16_bits(c).reshape(c.shape))
        if decoded:
            got = latent_gpu(ctx, query[p:p + 1], cache, prefix=p, heads=heads, rank=rank, scale=1.0, window=window, sink=sink, gate=None, f32_cache=f32_cache, splits=4)[0]
        else:
            lo = max(0, p - 99)
            got = latent_gpu(ctx, query[lo:p + 1], cache, prefix=lo, heads=heads, rank=rank, scale=1.0, window=window, sink=sink, gate=None, f32_cache=f32_cache, splits=0)[-1]
        close(got, ref[p], 3e-5, f"row {place} from {p}")
        assert (ref[p, 0, 0] > 3.5) == seen, (place, p)


# ---- whole models through the engine ----------------------------------------------------------------------------------------------
def config_a():
    """Every size differs from every other; grouped key heads; a borrower of layer 0's latents; partial rotation with blended frequencies;
    a matrix memory without feed-forward; order latent, attention, mlstm, latent (borrower), attention."""
    return P.make_config(96, 211, [
        P.latent_layer(5, 12, 20, 40, 24, 11, 56),
        P.attention_layer(6, 2, 16, 32, 44, rot_dims=8, base=300.0, scaling={"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}, scale=0.21),
        P.mlstm_layer(3, 20, 12, None, gate_cap=15.0),
        P.latent_layer(3, 8, 28, 40, 16, 30, 36, kv_from=0, scale=0.4),
        P.attention_layer(2, 2, 24, 10, None, rot_dims=24, base=1e4),
    ], eps=1e-4, residual_mult=0.3, embedding_scale=0.5, side_dim=8)


def config_b():
    """One head everywhere it can be, heads == kv_heads, a window of one key and a window longer than any test context, wide latent rows
    (few tokens per cache page), no rotation in one attention layer, factor 1 on the additions and on the embedding, two matrix memories
    in a row, a borrower right after its lender and a second borrower of the same lender."""
    return P.make_config(64, 130, [
        P.mlstm_layer(1, 40, 8, 24, gate_cap=4.0),
        P.mlstm_layer(4, 8, 8, None),
        P.latent_layer(1, 24, 16, 500, 32, 1, 12),
        P.latent_layer(4, 8, 8, 500, 8, 5000, 20, kv_from=2),
        P.attention_layer(1, 1, 64, 24, 16, rot_dims=0),
        P.latent_layer(2, 16, 12, 500, 12, 3, None, kv_from=2),
    ], eps=1e-6, residual_mult=1.0, embedding_scale=1.0, side_dim=4)


def config_c():
    """Sizes that fit no vector width: width 90, head sizes 10 / 6 and 18 / 22 (bf16 rows that start at odd words), a latent of 27, odd
    feed-forwards, a token input of 3 channels, a matrix memory with keys of 9 and values of 7."""
    return P.make_config(90, 77, [
        P.attention_layer(4, 2, 10, 6, 11, rot_dims=6, base=50.0, scale=0.4),
        P.latent_layer(3, 10, 6, 27, 9, 9, 51),
        P.mlstm_layer(3, 9, 7, 13, gate_cap=30.0),
        P.attention_layer(2, 1, 18, 22, None, rot_dims=18, base=1e5, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}),
    ], eps=1e-5, residual_mult=0.7, embedding_scale=2.0, side_dim=3)


def config_d():
    """Latent sizes the expanded prompt form takes (latent 64 / 128, head sizes in multiples of 16): windows shorter and longer than a pass,
    a borrower with other head sizes than its lender, no window at all."""
    return P.make_config(128, 150, [
        P.latent_layer(4, 16, 32, 64, 24, 20, 40),
        P.mlstm_layer(2, 16, 16, None),
        P.latent_layer(2, 32, 16, 64, 16, 100, 24, kv_from=0),
        P.latent_layer(3, 16, 16, 128, 32, 100000, None),
        P.attention_layer(4, 2, 32, 16, 36, rot_dims=16, base=1e4),
    ], eps=1e-5, residual_mult=0.4, embedding_scale=1.0, side_dim=16)


def write_model(path, config, weights):
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config))
    st.save(path / "model.safetensors", {k: st.as_bf16(synth.f32_to_bf16_bits(v.to(torch.float32).numpy()).reshape(tuple(v.shape))) for k, v in weights.items()})
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

    def reference(self, tokens, with_layers=False):
        logits, layers, _ = P.forward(self.config, self.weights, list(tokens))
        return (logits.numpy(), layers.numpy()) if with_layers else logits.numpy()

    def check(self, got, ref, what):
        got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
        d = (got - ref) - (got - ref).mean(-1, keepdims=True)
        err = np.sqrt((d * d).mean(-1)) / max(float(ref.std()), 1e-6)
        # bf16 products: the bound holds for the median row and 2.5 times it for nine rows in ten. Single rows are ill-conditioned by design:
        # the token input is a unit-RMS vector spanned by a few gated channels, and where these are all near zero its direction follows the
        # rounding (the f32 engine, held to its bound in every row, is the test of masks, states and slots).
        if self.f32:
            assert err.max() <= self.tol, f"{what}: row {int(err.argmax())} differs by {err.max():.3e} of the logits' spread (bound {self.tol:.0e})"
        else:
            assert np.median(err) <= self.tol and np.quantile(err, 0.9) <= 2.5 * self.tol, \
                f"{what}: median / 90 % of the rows differ by {np.median(err):.3e} / {np.quantile(err, 0.9):.3e} of the logits' spread (bound {self.tol:.0e})"

    def close(self):
        self.engine.close()


def tokens_for(config, n, seed=0):
    return np.random.default_rng(seed).integers(0, config["vocab"], n).tolist()


@pytest.mark.parametrize("make", [config_a, config_b, config_c, config_d])
@pytest.mark.parametrize("f32", [True, False])
def test_prompt_logits_and_layers(ctx, tmp_path, make, f32):
    pr = Pair(ctx, tmp_path, make(), seed=1, f32=f32)
    toks = tokens_for(pr.config, 70 if f32 else 150, 1)     # bf16: 150 rows take the tensor-pipe products and attention (and expanded latents)
    pr.engine.debug_layer_outputs(True)
    s = pr.engine.slot_acquire()
    got = pr.engine.forward_rows(toks, list(range(len(toks))), slot=s)
    layers = pr.engine.debug_layer_outputs(True)
    ref, ref_layers = pr.reference(toks, with_layers=True)
    for i, (g, r) in enumerate(zip(layers, ref_layers)):
        if f32:
            close(g, r, 1e-4, f"residual after layer {i}")
        else:                                   # bf16 products: the root mean square of the difference, not its largest element
            assert np.sqrt(((g - r) ** 2).mean() / (r ** 2).mean()) <= 3e-2, f"residual after layer {i}"
    pr.check(got, ref, "prompt logits")
    pr.close()


@pytest.mark.parametrize("make", [config_a, config_b, config_c, config_d])
@pytest.mark.parametrize("f32", [True, False])
def test_decode_and_portions_match_the_whole_prompt(ctx, tmp_path, make, f32):
    """Prefill + token-by-token decoding (the windows pass over decoded tokens), and portions of 2, 3, 1, 33, 2, ... tokens cut in the middle
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
    pr.engine.slot_release(s)
    s = pr.engine.slot_acquire()                 # long portions after a prefix: 90 + 80 rows see windows that start before their pass
    parts = [pr.engine.forward_rows(toks[:90], list(range(90)), slot=s), pr.engine.forward_rows(toks[90:], list(range(n - 90)), slot=s)]
    pr.check(np.concatenate(parts), ref, "two long portions")
    pr.close()


def test_slots_interleaved_and_reused(ctx, tmp_path):
    """Three unequal requests advance in turns in their own slots; one ends early and its slot serves a new request, whose matrix memory,
    running maximum and caches must start from nothing. Each equals its solo run."""
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
    """1100 tokens: past the 1024-row pass and, with 500-wide f32 latent rows, past the first cache page (lender and both borrowers). Then
    40 decoded tokens. Rows just before and after both edges are compared, in the prompt and decoded."""
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


def marker_model(kind, marker=7):
    """One layer whose mixer finds the marker token wherever it is visible. Dynamic Tanh with a small alpha is nearly linear, so input
    coordinate 0 (non-zero for the marker only) reaches one key channel and coordinate 1 (the same for every token) the same query
    channel. kind "latent": a window of 16 with a borrower behind it that sees the same rows; kind "attention": no window."""
    if kind == "latent":
        layers = [P.latent_layer(2, 8, 12, 8, 8, 16, 20, scale=1.0), P.latent_layer(2, 8, 6, 8, 8, 16, None, scale=1.0, kv_from=0)]
    else:
        layers = [P.attention_layer(2, 1, 8, 12, 20, rot_dims=4, base=100.0, scale=1.0)]
    cfg = P.make_config(48, 60, layers, eps=1e-6, residual_mult=1.0, embedding_scale=1.0, side_dim=4)
    w = {k: v.to(torch.float32) for k, v in P.random_weights(cfg, 5).items()}
    w["embed"][:, 0] = 0.0
    w["embed"][:, 1] = 3.0
    w["embed"][marker] = 0.0
    w["embed"][marker, 0] = 5.0
    w["embed"][marker, 1] = 3.0
    w["l0.norm1"][:] = 1.0
    w["l0.norm1.b"][:] = 0.0
    w["l0.norm1.alpha"] = torch.tensor(0.125)
    if kind == "latent":
        for l in ("l0.", "l1."):
            w[l + "mix.dq"] *= 0.05
            w[l + "mix.dq"][7, :] = 0.0
            w[l + "mix.dq"][7, 1] = 6.0                      # query latent channel 7 reads the constant coordinate
            w[l + "mix.dq.norm"][:] = 1.0
            w[l + "mix.uq"] *= 0.05
            w[l + "mix.uk"] *= 0.05
            for h in range(2):
                w[l + "mix.uq"][h * 8 + 7, :] = 0.0
                w[l + "mix.uq"][h * 8 + 7, 7] = 2.0
                w[l + "mix.uk"][h * 8 + 7, :] = 0.0
                w[l + "mix.uk"][h * 8 + 7, 7] = 4.0          # key channel 7 of every head reads latent channel 7
            w[l + "mix.sink"][:] = -2.0
            w[l + "mix.o"] *= 3.0
        w["l0.mix.dkv"] *= 0.05
        w["l0.mix.dkv"][7, :] = 0.0
        w["l0.mix.dkv"][7, 0] = 10.0                         # latent channel 7 reads the marker's coordinate
        w["l0.mix.dkv.norm"][:] = 1.0
    else:
        l = "l0.mix."
        w[l + "k.norm"][:] = 1.0
        w[l + "q.norm"][:] = 1.0
        for name, heads in (("k", 1), ("q", 2)):
            w[l + name] *= 0.05
            for h in range(heads):
                w[l + name][h * 8 + 7, :] = 0.0
        w[l + "k"][7, 0] = 10.0
        for h in range(2):
            w[l + "q"][h * 8 + 7, 1] = 6.0
        w[l + "o"] *= 3.0
    return cfg, {k: v.to(torch.bfloat16) for k, v in w.items()}, marker


def test_marker_token_inside_and_outside_the_latent_window(ctx, tmp_path):
    """A marker token in a 300-token prompt. Seen from the last rows it matters when it is inside the window (285 ..) and must NOT matter
    one place before it or at position 0: the engine agrees with the oracle for each place, in the prompt's last row and in 10 decoded
    tokens (the lender's window and the borrower's both slide over them)."""
    cfg, w, marker = marker_model("latent")
    pr = Pair(ctx, tmp_path, cfg, seed=5, f32=True, weights=w)
    base = [x if x != marker else 8 for x in tokens_for(cfg, 300, 5)]
    without = pr.reference(base)
    n, window = 300, 16
    for place, matters in ((0, False), (n - 11 - window, False), (n - 11 - window + 1, True), (n - 12, True)):
        toks = list(base)
        toks[place] = marker
        ref = pr.reference(toks)
        moved = np.sqrt(((ref[n - 11] - without[n - 11]) ** 2).mean()) / ref.std()
        assert (moved > 0.05) == matters, (place, moved)
        s = pr.engine.slot_acquire()
        got = pr.engine.forward_rows(toks[:n - 10], [n - 11], slot=s)
        dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(n - 10, n)])
        pr.engine.slot_release(s)
        pr.check(got, ref[n - 11:n - 10], f"marker at {place}, prompt")
        pr.check(dec, ref[n - 10:], f"marker at {place}, decoded")
    pr.close()


def test_marker_token_far_back_in_full_attention(ctx, tmp_path):
    """Without a window the marker matters from anywhere: position 0, 1 and 400 tokens back, from a prompt row and from decoded rows."""
    cfg, w, marker = marker_model("attention")
    pr = Pair(ctx, tmp_path, cfg, seed=5, f32=True, weights=w)
    n = 420
    base = [x if x != marker else 8 for x in tokens_for(cfg, n, 6)]
    without = pr.reference(base)
    for place in (0, 1, 19, n - 12):
        toks = list(base)
        toks[place] = marker
        ref = pr.reference(toks)
        assert np.sqrt(((ref[n - 11] - without[n - 11]) ** 2).mean()) / ref.std() > 0.05, place
        s = pr.engine.slot_acquire()
        got = pr.engine.forward_rows(toks[:n - 10], [n - 11], slot=s)
        dec = np.concatenate([pr.engine.forward_rows(toks[p:p + 1], [0], slot=s) for p in range(n - 10, n)])
        pr.engine.slot_release(s)
        pr.check(got, ref[n - 11:n - 10], f"marker at {place}, prompt")
        pr.check(dec, ref[n - 10:], f"marker at {place}, decoded")
    pr.close()


def test_matrix_memory_carries_the_first_token(ctx, tmp_path):
    """A model of matrix memories only, forget gates nearly open: what the first token was still decides the last logits 400 tokens later
    -- in one pass, in portions, and decoded."""
    cfg = P.make_config(40, 50, [P.mlstm_layer(2, 8, 10, None), P.mlstm_layer(1, 12, 6, 16)], eps=1e-5, residual_mult=0.5, side_dim=2)
    w = P.random_weights(cfg, 8)
    for l in ("l0.", "l1."):
        w[l + "mix.f.b"] = torch.full_like(w[l + "mix.f.b"], 9.0)
        w[l + "mix.f"] = w[l + "mix.f"] * 0.1
    pr = Pair(ctx, tmp_path, cfg, seed=8, f32=True, weights=w)
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
    """prefill() + next()/flush() (the engine's generation entry point; CUDA-graph decode when `graph`), 300 tokens: the windows (11 and
    30) pass over decoded tokens many times. The oracle reads the whole sequence once: every chosen token must be its best at that place
    within the rounding of the bf16 logits the sampler reads."""
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


def test_synthetic_checkpoint_of_a_preset_loads_and_decodes(ctx, tmp_path):
    """The benchmark's layer stack at a small width: the checkpoint writer's tensor names and shapes are the loader's."""
    cfg = synth.vakesun_preset(width=256, vocab=300, layers=5, ff=384, window=48, side_dim=16, memory_ff=False)
    path = synth.write_vakesun_model(cfg, tmp_path / "preset", seed=1)
    w = {k: torch.from_numpy(np.asarray(synth.st_bits_to_f32(np.asarray(v))).reshape(v.shape).copy()) for k, v in st.load(path / "model.safetensors")[0].items()}
    toks = tokens_for(cfg, 90, 3)
    ref, _, _ = P.forward(cfg, w, toks)
    with B.Engine(ctx, path, max_context_length=256, storage_f32=True) as eng:
        got = eng.forward_rows(toks[:80], [0, 47, 48, 49, 79])
        dec = np.concatenate([eng.forward_rows(toks[p:p + 1], [0]) for p in range(80, 90)])
    d = np.concatenate([got, dec]) - ref.numpy()[[0, 47, 48, 49, 79] + list(range(80, 90))]
    assert np.sqrt((d * d).mean(-1)).max() <= 2e-4 * float(ref.std())


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
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(step)]
    refs = {rid: P.forward(cfg, w, toks)[0].numpy() for rid, toks in reqs.items()}
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
        assert np.median(errs) < 6e-2, np.median(errs)
