// Dense (unquantised) linear: D (+)= scale * A . W^T, f32 activations, bf16 or f32 weights [n, k], f32 accumulation.
// Three kernels behind one entry point (uzu_dense_linear_encode):
//   rows kernel   (<= 8 rows per group): one warp per output feature, the weight row streamed once with 128-bit loads and multiplied
//                 with every activation row in f32 -- the decode step's weight pass, bound by the weight bytes;
//   tensor kernels (bf16 weights, >= 32 rows): 64 x 64 output tiles (128 x 128 with ldmatrix fragments from 96 rows on) on
//                 mma.sync.m16n8k16 (bf16 x bf16 -> f32), A rounded to bf16 while it is staged, double-buffered shared-memory tiles;
//   tile kernel   (everything else, and every f32-weight product of more than 8 rows): 64 x 64 tiles of f32 multiply-adds.
// All three share the operand addressing: z-batches (per-head weights: operand z starts z*stride further in A, W and D) and row groups
// (per-expert weights: compact rows [off[z], off[z+1]) use weight z, an optional map names the activation row a compact row reads).
#include <mma.h>

#include <type_traits>

#include "common.cuh"

namespace uzu {

// tcgen05 form of the plain bf16 product (dense_umma.cu)
bool dense_umma_applicable(const uzu_dense_linear_args& a);
void encode_dense_umma(uzu_command_buffer* cmd, const uzu_dense_linear_args& a);

struct DenseRows {
    uint32_t begin, count;
};

__device__ __forceinline__ DenseRows dense_rows(const uzu_dense_linear_args& a, uint32_t z) {
    if (a.group_offsets) {
        const uint32_t* off = reinterpret_cast<const uint32_t*>(a.group_offsets);
        const uint32_t b = off[z], e = off[z + 1];
        return {b, e - b};
    }
    return {0u, a.m};
}

template <typename TW>
__device__ __forceinline__ float w_to_f32(TW v);
template <>
__device__ __forceinline__ float w_to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float w_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float dense_a(const uzu_dense_linear_args& a, float x) {
    if (a.a_op == 1) return tanhf(x);
    if (a.a_op == 2) { const float r = fmaxf(x, 0.0f); return r * r; }
    return x;
}

// `row` is the compact row the value belongs to (the gate is indexed like D)
__device__ __forceinline__ void dense_store(const uzu_dense_linear_args& a, float* d, uint32_t z, uint32_t row, uint32_t col, float acc) {
    float v = acc * a.scale;
    if (a.row_scale) v *= reinterpret_cast<const float*>(a.row_scale)[row];
    if (a.gate) {
        float g = reinterpret_cast<const float*>(a.gate)[(size_t)row * a.gate_ld + (size_t)z * a.d_z_stride + col];
        if (a.gate_bias) g += reinterpret_cast<const float*>(a.gate_bias)[col];
        v *= 1.0f / (1.0f + expf(-g));
    }
    if (a.col_scale) v *= reinterpret_cast<const float*>(a.col_scale)[col];
    if (a.bias && z == 0) v += reinterpret_cast<const float*>(a.bias)[col];
    if (a.post_weight) {          // sandwich epilogue: the product's own Dynamic Tanh norm, the residual add, the next reader's norm
        float y = tanhf(a.post_alpha * v) * reinterpret_cast<const float*>(a.post_weight)[col];
        if (a.post_bias) y += reinterpret_cast<const float*>(a.post_bias)[col];
        const float x = fmaf(a.post_mult, y, *d);
        *d = x;
        if (a.next_out) {
            float n = tanhf(a.next_alpha * x);
            if (a.next_weight) n *= reinterpret_cast<const float*>(a.next_weight)[col];
            if (a.next_bias) n += reinterpret_cast<const float*>(a.next_bias)[col];
            reinterpret_cast<float*>(a.next_out)[(size_t)row * a.ldd + col] = n;
        }
        return;
    }
    if (a.token_table) {          // token-gate epilogue: gelu_tanh(product) * a table entry of the row's token
        const uint32_t tok = reinterpret_cast<const uint32_t*>(a.token_ids)[row];
        float e = 0.0f;
        if (tok < a.token_vocab) {
            const size_t at = (size_t)tok * a.token_table_stride + a.token_column + col;
            e = a.token_gate_dt == UZU_DT_F32 ? reinterpret_cast<const float*>(a.token_table)[at] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.token_table)[at]);
        }
        v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v))) * e;
    }
    if (a.accumulate) v += *d;
    *d = v;
}

// ---- rows kernel ------------------------------------------------------------------------------------------------------------------
constexpr int DL_MAX_ROWS = 8;

// KS warps share one output feature, each a contiguous slice of k; their partial sums meet in shared memory in slice order. Few output
// features with a long k (a down projection) would otherwise leave most of the memory system idle. PAIR: the warp streams a second
// weight row (`pair_rows` below the first) against the same activations and stores the clamped gated unit of the two sums.
template <int VEC, typename TW>
__device__ __forceinline__ void unpack_weights(const uint4& raw, float (&wf)[VEC]) {
    if constexpr (sizeof(TW) == 2) {
        const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            wf[2 * i] = __uint_as_float(w4[i] << 16);
            wf[2 * i + 1] = __uint_as_float(w4[i] & 0xffff0000u);
        }
    } else {
        wf[0] = __uint_as_float(raw.x); wf[1] = __uint_as_float(raw.y); wf[2] = __uint_as_float(raw.z); wf[3] = __uint_as_float(raw.w);
    }
}

__device__ __forceinline__ float clamped_glu_value(float g, float u, float limit, float alpha) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
}

constexpr uint32_t DL_STAGE_FLOATS = 8192;   // activation rows of a group are staged in shared memory when they fit (32 KB)

// RMAX = most activation rows of a group (1 for a plain decode step: one accumulator, no row pointers -> more CTAs per SM).
template <typename TW, int KS, bool PAIR, int RMAX>
__global__ void __launch_bounds__(256, RMAX == 1 ? 4 : 2) dense_rows_kernel(const uzu_dense_linear_args a) {
    __shared__ float part[PAIR ? 2 : 1][8][RMAX];
    __shared__ __align__(16) float a_s[DL_STAGE_FLOATS];
    const uint32_t z = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const uint32_t warp = threadIdx.x >> 5, slice = warp % KS;
    const uint32_t col = blockIdx.x * (8 / KS) + warp / KS;
    const bool col_ok = col < a.n;
    pdl_launch_dependents();
    const TW* w = reinterpret_cast<const TW*>(a.w) + (size_t)z * a.w_z_stride + (size_t)(col_ok ? col : 0) * a.k;
    const TW* w2 = w + (size_t)(PAIR ? a.pair_rows : 0) * a.k;
    constexpr int VEC = 16 / (int)sizeof(TW);            // weights per 128-bit load
    const bool vec_ok = (a.k % VEC == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0) && (a.lda % 4 == 0) && ((a.a & 15) == 0) &&
                        (a.a_z_stride % 4 == 0) && (((size_t)a.w_z_stride * sizeof(TW)) % 16 == 0) && (((size_t)a.k * sizeof(TW)) % 16 == 0) &&
                        (!PAIR || (((size_t)a.pair_rows * a.k * sizeof(TW)) % 16 == 0));
    const uint32_t sweep = vec_ok ? 32 * VEC : 32;       // k covered by one pass of the warp's lanes
    const uint32_t sweeps = (a.k + sweep - 1) / sweep, per = (sweeps + KS - 1) / KS;
    const uint32_t k_lo = min(a.k, slice * per * sweep), k_hi = min(a.k, (slice + 1) * per * sweep);
    // Weight loads of a lane run two batches deep: a batch is requested before the previous one is used. The first batch does not depend
    // on the previous kernel: with programmatic dependent launch it is in flight during that kernel's tail.
    constexpr uint32_t STEP = 32 * VEC, BATCH = PAIR ? 2 : 4;
    uint4 cur[BATCH], cur2[PAIR ? BATCH : 1];
    const uint32_t k_first = k_lo + (uint32_t)lane * VEC;
    auto request = [&](uint4 (&r)[BATCH], uint4 (&r2)[PAIR ? BATCH : 1], uint32_t kb) {
#pragma unroll
        for (uint32_t u = 0; u < BATCH; ++u) {
            const uint32_t k0 = kb + u * STEP;
            if (k0 < k_hi) {
                r[u] = ldg_stream_u4(w + k0);
                if constexpr (PAIR) r2[u] = ldg_stream_u4(w2 + k0);
            }
        }
    };
    if (vec_ok && col_ok) request(cur, cur2, k_first);
    pdl_wait();
    const DenseRows R = dense_rows(a, z);
    if (R.count == 0) return;                            // uniform over the CTA
    const uint32_t* map = reinterpret_cast<const uint32_t*>(a.rows_map);
    // the group's activation rows, with the A operation applied, go to shared memory once per CTA when they fit
    const bool staged = vec_ok && (size_t)R.count * a.k <= DL_STAGE_FLOATS;
    const float* arow[RMAX];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
        const uint32_t p = R.begin + ((uint32_t)r < R.count ? r : 0);
        arow[r] = reinterpret_cast<const float*>(a.a) + (size_t)z * a.a_z_stride + (size_t)(map ? map[p] : p) * a.lda;
    }
    if (staged) {
        const uint32_t k4 = a.k / 4;
        for (uint32_t i = threadIdx.x; i < R.count * k4; i += blockDim.x) {
            const uint32_t r = i / k4, c = i - r * k4;
            const uint32_t p = R.begin + r;
            const float* src = reinterpret_cast<const float*>(a.a) + (size_t)z * a.a_z_stride + (size_t)(map ? map[p] : p) * a.lda;
            float4 x = reinterpret_cast<const float4*>(src)[c];
            if (a.a_op) { x.x = dense_a(a, x.x); x.y = dense_a(a, x.y); x.z = dense_a(a, x.z); x.w = dense_a(a, x.w); }
            reinterpret_cast<float4*>(a_s)[i] = x;
        }
        __syncthreads();
    }
    float acc[RMAX], acc2[PAIR ? RMAX : 1];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) acc[r] = 0.0f;
#pragma unroll
    for (int r = 0; r < (PAIR ? RMAX : 1); ++r) acc2[r] = 0.0f;
    if (!col_ok) {
        // nothing to sum; the warp still meets the others at the barrier below
    } else if (vec_ok) {
        for (uint32_t kb = k_first; kb < k_hi; kb += BATCH * STEP) {
            uint4 nxt[BATCH], nxt2[PAIR ? BATCH : 1];
            if (kb + BATCH * STEP < k_hi) request(nxt, nxt2, kb + BATCH * STEP);
#pragma unroll
            for (uint32_t u = 0; u < BATCH; ++u) {
                const uint32_t k0 = kb + u * STEP;
                if (k0 >= k_hi) break;
                float wf[VEC], wf2[PAIR ? VEC : 1];
                unpack_weights<VEC, TW>(cur[u], wf);
                if constexpr (PAIR) unpack_weights<VEC, TW>(cur2[u], wf2);
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    if ((uint32_t)r < R.count) {
#pragma unroll
                        for (int i = 0; i < VEC; i += 4) {
                            float4 x;
                            if (staged) {
                                x = *reinterpret_cast<const float4*>(a_s + (size_t)r * a.k + k0 + i);
                            } else {
                                x = *reinterpret_cast<const float4*>(arow[r] + k0 + i);
                                if (a.a_op) { x.x = dense_a(a, x.x); x.y = dense_a(a, x.y); x.z = dense_a(a, x.z); x.w = dense_a(a, x.w); }
                            }
                            acc[r] = fmaf(x.x, wf[i], acc[r]);
                            acc[r] = fmaf(x.y, wf[i + 1], acc[r]);
                            acc[r] = fmaf(x.z, wf[i + 2], acc[r]);
                            acc[r] = fmaf(x.w, wf[i + 3], acc[r]);
                            if constexpr (PAIR) {
                                acc2[r] = fmaf(x.x, wf2[i], acc2[r]);
                                acc2[r] = fmaf(x.y, wf2[i + 1], acc2[r]);
                                acc2[r] = fmaf(x.z, wf2[i + 2], acc2[r]);
                                acc2[r] = fmaf(x.w, wf2[i + 3], acc2[r]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (uint32_t u = 0; u < BATCH; ++u) {
                cur[u] = nxt[u];
                if constexpr (PAIR) cur2[u] = nxt2[u];
            }
        }
    } else {
        for (uint32_t k0 = k_lo + lane; k0 < k_hi; k0 += 32) {
            const float wv = w_to_f32<TW>(w[k0]);
            const float wv2 = PAIR ? w_to_f32<TW>(w2[k0]) : 0.0f;
#pragma unroll
            for (int r = 0; r < RMAX; ++r)
                if ((uint32_t)r < R.count) {
                    const float x = dense_a(a, arow[r][k0]);
                    acc[r] = fmaf(x, wv, acc[r]);
                    if constexpr (PAIR) acc2[r] = fmaf(x, wv2, acc2[r]);
                }
        }
    }
    auto finish = [&](uint32_t r, float s, float s2) {
        float* d = reinterpret_cast<float*>(a.d) + (size_t)z * a.d_z_stride + (size_t)(R.begin + r) * a.ldd + col;
        if constexpr (PAIR) {
            if (a.row_scale) { const float rs = reinterpret_cast<const float*>(a.row_scale)[R.begin + r]; s *= rs; s2 *= rs; }
        }
        if constexpr (PAIR) *d = a.glu_kind == 1 ? s * (1.0f / (1.0f + expf(-s))) * s2 : clamped_glu_value(s, s2, a.glu_limit, a.glu_alpha);
        else dense_store(a, d, z, R.begin + r, col, s);
    };
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
        if ((uint32_t)r < R.count) {          // uniform over the warp
            const float s = warp_sum(acc[r]);
            float s2 = 0.0f;
            if constexpr (PAIR) s2 = warp_sum(acc2[r]);
            if (lane == 0) {
                if constexpr (KS == 1) {
                    if (col_ok) finish(r, s, s2);
                } else {
                    part[0][warp][r] = s;
                    if constexpr (PAIR) part[1][warp][r] = s2;
                }
            }
        }
    }
    if constexpr (KS > 1) {
        __syncthreads();
        if (slice == 0 && col_ok && (uint32_t)lane < R.count) {     // lane = activation row; slices added in order
            float s = 0.0f, s2 = 0.0f;
#pragma unroll
            for (int q = 0; q < KS; ++q) {
                s += part[0][warp + q][lane];
                if constexpr (PAIR) s2 += part[1][warp + q][lane];
            }
            finish(lane, s, s2);
        }
    }
}

// ---- tile kernel (f32 multiply-adds) ------------------------------------------------------------------------------------------------
constexpr int DT_BM = 64, DT_BN = 64, DT_BK = 16;

template <typename TW>
__global__ void __launch_bounds__(256) dense_tile_kernel(const uzu_dense_linear_args a) {
    __shared__ float As[DT_BK][DT_BM + 4];
    __shared__ float Ws[DT_BK][DT_BN + 4];
    const uint32_t z = blockIdx.z;
    const DenseRows R = dense_rows(a, z);
    const uint32_t m0 = blockIdx.y * DT_BM, n0 = blockIdx.x * DT_BN;
    if (m0 >= R.count) return;
    const uint32_t* map = reinterpret_cast<const uint32_t*>(a.rows_map);
    const float* A = reinterpret_cast<const float*>(a.a) + (size_t)z * a.a_z_stride;
    const TW* W = reinterpret_cast<const TW*>(a.w) + (size_t)z * a.w_z_stride;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    // staging: thread loads 4 consecutive k of one row (A) and one feature (W)
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const uint32_t pa = m0 + lr;
    const bool a_ok = pa < R.count;
    const float* a_src = A + (size_t)(a_ok ? (map ? map[R.begin + pa] : R.begin + pa) : 0) * a.lda;
    const bool w_ok = n0 + lr < a.n;
    const TW* w_src = W + (size_t)(w_ok ? n0 + lr : 0) * a.k;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (uint32_t k0 = 0; k0 < a.k; k0 += DT_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t k = k0 + lk + i;
            As[lk + i][lr] = (a_ok && k < a.k) ? dense_a(a, a_src[k]) : 0.0f;
            Ws[lk + i][lr] = (w_ok && k < a.k) ? w_to_f32<TW>(w_src[k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < DT_BK; ++k) {
            const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t p = m0 + ty * 4 + i;
        if (p >= R.count) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t col = n0 + tx * 4 + j;
            if (col >= a.n) continue;
            float* d = reinterpret_cast<float*>(a.d) + (size_t)z * a.d_z_stride + (size_t)(R.begin + p) * a.ldd + col;
            dense_store(a, d, z, R.begin + p, col, acc[i][j]);
        }
    }
}

// ---- tensor kernel (bf16 weights, mma.sync m16n8k16) --------------------------------------------------------------------------------
// 128 threads = 4 warps in a 2 x 2 grid, each warp a 32 x 32 part of the 64 x 64 tile = 2 x 4 MMA tiles. K blocks of 32, staged as bf16
// in shared memory with a row stride of 40 elements (80 bytes: the 8 rows of a fragment load fall into different banks).
constexpr int TC_BM = 64, TC_BN = 64, TC_BK = 32, TC_LD = 40;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(128) dense_tensor_kernel(const uzu_dense_linear_args a) {
    __shared__ __align__(16) __nv_bfloat16 As[2][TC_BM * TC_LD];
    __shared__ __align__(16) __nv_bfloat16 Ws[2][TC_BN * TC_LD];
    const uint32_t z = blockIdx.z;
    const DenseRows R = dense_rows(a, z);
    const uint32_t m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * TC_BN;
    if (m0 >= R.count) return;
    const uint32_t* map = reinterpret_cast<const uint32_t*>(a.rows_map);
    const float* A = reinterpret_cast<const float*>(a.a) + (size_t)z * a.a_z_stride;
    const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(a.w) + (size_t)z * a.w_z_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    // staging: a thread owns half a row (16 k) of the A tile and of the W tile
    const int sr = tid >> 1, sk = (tid & 1) * 16;
    const uint32_t pa = m0 + sr;
    const bool a_ok = pa < R.count;
    const float* a_src = A + (size_t)(a_ok ? (map ? map[R.begin + pa] : R.begin + pa) : 0) * a.lda;
    const bool w_ok = n0 + sr < a.n;
    const __nv_bfloat16* w_src = W + (size_t)(w_ok ? n0 + sr : 0) * a.k;
    const bool a_vec = (a.lda % 4 == 0) && ((a.a & 15) == 0) && (a.a_z_stride % 4 == 0) && (a.k % 4 == 0);
    const bool w_vec = (a.k % 8 == 0) && ((a.w & 15) == 0) && (a.w_z_stride % 8 == 0);
    float ra[16];
    __align__(16) __nv_bfloat16 rw[16];
    auto fetch = [&](uint32_t k0) {
        const uint32_t kb = k0 + sk;
        if (a_ok && a_vec && kb + 16 <= a.k) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = *reinterpret_cast<const float4*>(a_src + kb + 4 * i);
                ra[4 * i] = v.x; ra[4 * i + 1] = v.y; ra[4 * i + 2] = v.z; ra[4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) ra[i] = (a_ok && kb + i < a.k) ? a_src[kb + i] : 0.0f;
        }
        if (w_ok && w_vec && kb + 16 <= a.k) {
            *reinterpret_cast<uint4*>(&rw[0]) = *reinterpret_cast<const uint4*>(w_src + kb);
            *reinterpret_cast<uint4*>(&rw[8]) = *reinterpret_cast<const uint4*>(w_src + kb + 8);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) rw[i] = (w_ok && kb + i < a.k) ? w_src[kb + i] : __float2bfloat16_rn(0.0f);
        }
    };
    auto stash = [&](int buf) {
        if (a.a_op) {
#pragma unroll
            for (int i = 0; i < 16; ++i) ra[i] = dense_a(a, ra[i]);
        }
        __nv_bfloat16* as = &As[buf][sr * TC_LD + sk];
        __nv_bfloat16* ws = &Ws[buf][sr * TC_LD + sk];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            *reinterpret_cast<__nv_bfloat162*>(as + i) = __floats2bfloat162_rn(ra[i], ra[i + 1]);
            *reinterpret_cast<__nv_bfloat162*>(ws + i) = __halves2bfloat162(rw[i], rw[i + 1]);
        }
    };
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.0f;
    const uint32_t nk = (a.k + TC_BK - 1) / TC_BK;
    fetch(0);
    stash(0);
    __syncthreads();
    const int g = lane >> 2, t4 = lane & 3;
    for (uint32_t kb = 0; kb < nk; ++kb) {
        const int cur = kb & 1;
        if (kb + 1 < nk) fetch((kb + 1) * TC_BK);
#pragma unroll
        for (int ks = 0; ks < TC_BK; ks += 16) {
            uint32_t af[2][4], bf[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const __nv_bfloat16* base = &As[cur][(wm + i * 16 + g) * TC_LD + ks + t4 * 2];
                af[i][0] = *reinterpret_cast<const uint32_t*>(base);
                af[i][1] = *reinterpret_cast<const uint32_t*>(base + 8 * TC_LD);
                af[i][2] = *reinterpret_cast<const uint32_t*>(base + 8);
                af[i][3] = *reinterpret_cast<const uint32_t*>(base + 8 * TC_LD + 8);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat16* base = &Ws[cur][(wn + j * 8 + g) * TC_LD + ks + t4 * 2];
                bf[j][0] = *reinterpret_cast<const uint32_t*>(base);
                bf[j][1] = *reinterpret_cast<const uint32_t*>(base + 8);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], af[i], bf[j]);
        }
        if (kb + 1 < nk) stash(cur ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t p = m0 + wm + i * 16 + g + (q >> 1) * 8;
                const uint32_t col = n0 + wn + j * 8 + t4 * 2 + (q & 1);
                if (p < R.count && col < a.n) {
                    float* d = reinterpret_cast<float*>(a.d) + (size_t)z * a.d_z_stride + (size_t)(R.begin + p) * a.ldd + col;
                    dense_store(a, d, z, R.begin + p, col, acc[i][j][q]);
                }
            }
}

// ---- tensor kernel for long passes (bf16 weights, >= 96 rows): 128 x 128 tiles, 8 warps in a 2 x 4 grid, each a 64 x 32 part = 4 x 4
// MMA tiles; fragments come from shared memory with ldmatrix (6 loads per 16 MMAs), same staging and double buffering as above.
constexpr int T8_BM = 128, T8_BN = 128;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__global__ void __launch_bounds__(256) dense_tensor128_kernel(const uzu_dense_linear_args a) {
    __shared__ __align__(16) __nv_bfloat16 As[2][T8_BM * TC_LD];
    __shared__ __align__(16) __nv_bfloat16 Ws[2][T8_BN * TC_LD];
    const uint32_t z = blockIdx.z;
    const DenseRows R = dense_rows(a, z);
    const uint32_t m0 = blockIdx.y * T8_BM, n0 = blockIdx.x * T8_BN;
    if (m0 >= R.count) return;
    const uint32_t* map = reinterpret_cast<const uint32_t*>(a.rows_map);
    const float* A = reinterpret_cast<const float*>(a.a) + (size_t)z * a.a_z_stride;
    const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(a.w) + (size_t)z * a.w_z_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
    // staging: a thread owns half a row (16 k) of the A tile and of the W tile
    const int sr = tid >> 1, sk = (tid & 1) * 16;
    const uint32_t pa = m0 + sr;
    const bool a_ok = pa < R.count;
    const float* a_src = A + (size_t)(a_ok ? (map ? map[R.begin + pa] : R.begin + pa) : 0) * a.lda;
    const bool w_ok = n0 + sr < a.n;
    const __nv_bfloat16* w_src = W + (size_t)(w_ok ? n0 + sr : 0) * a.k;
    const bool a_vec = (a.lda % 4 == 0) && ((a.a & 15) == 0) && (a.a_z_stride % 4 == 0) && (a.k % 4 == 0);
    const bool w_vec = (a.k % 8 == 0) && ((a.w & 15) == 0) && (a.w_z_stride % 8 == 0);
    float ra[16];
    __align__(16) __nv_bfloat16 rw[16];
    auto fetch = [&](uint32_t k0) {
        const uint32_t kb = k0 + sk;
        if (a_ok && a_vec && kb + 16 <= a.k) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = *reinterpret_cast<const float4*>(a_src + kb + 4 * i);
                ra[4 * i] = v.x; ra[4 * i + 1] = v.y; ra[4 * i + 2] = v.z; ra[4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) ra[i] = (a_ok && kb + i < a.k) ? a_src[kb + i] : 0.0f;
        }
        if (w_ok && w_vec && kb + 16 <= a.k) {
            *reinterpret_cast<uint4*>(&rw[0]) = *reinterpret_cast<const uint4*>(w_src + kb);
            *reinterpret_cast<uint4*>(&rw[8]) = *reinterpret_cast<const uint4*>(w_src + kb + 8);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) rw[i] = (w_ok && kb + i < a.k) ? w_src[kb + i] : __float2bfloat16_rn(0.0f);
        }
    };
    auto stash = [&](int buf) {
        if (a.a_op) {
#pragma unroll
            for (int i = 0; i < 16; ++i) ra[i] = dense_a(a, ra[i]);
        }
        // rows are 80 bytes apart and a thread's half row starts at byte 0 or 32: 16-byte stores
        uint32_t pa2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(ra[2 * i], ra[2 * i + 1]);
            pa2[i] = *reinterpret_cast<const uint32_t*>(&v);
        }
        uint4* as = reinterpret_cast<uint4*>(&As[buf][sr * TC_LD + sk]);
        uint4* ws = reinterpret_cast<uint4*>(&Ws[buf][sr * TC_LD + sk]);
        as[0] = make_uint4(pa2[0], pa2[1], pa2[2], pa2[3]);
        as[1] = make_uint4(pa2[4], pa2[5], pa2[6], pa2[7]);
        ws[0] = *reinterpret_cast<const uint4*>(&rw[0]);
        ws[1] = *reinterpret_cast<const uint4*>(&rw[8]);
    };
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.0f;
    const uint32_t nk = (a.k + TC_BK - 1) / TC_BK;
    fetch(0);
    stash(0);
    __syncthreads();
    for (uint32_t kb = 0; kb < nk; ++kb) {
        const int cur = kb & 1;
        if (kb + 1 < nk) fetch((kb + 1) * TC_BK);
#pragma unroll
        for (int ks = 0; ks < TC_BK; ks += 16) {
            uint32_t af[4][4], bf[2][4];
            // A: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15) = the MMA's a0..a3
#pragma unroll
            for (int i = 0; i < 4; ++i) ldmatrix_x4(af[i], &As[cur][(wm + i * 16 + (lane & 15)) * TC_LD + ks + (lane >> 4) * 8]);
            // W: two n8 tiles per load: (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15) = b0, b1 of tile 0, b0, b1 of tile 1
#pragma unroll
            for (int j = 0; j < 2; ++j)
                ldmatrix_x4(bf[j], &Ws[cur][(wn + j * 16 + (lane & 7) + ((lane >> 4) << 3)) * TC_LD + ks + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t b2[2] = {bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]};
                    mma_bf16_16816(acc[i][j], af[i], b2);
                }
        }
        if (kb + 1 < nk) stash(cur ^ 1);
        __syncthreads();
    }
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t p = m0 + wm + i * 16 + g + (q >> 1) * 8;
                const uint32_t col = n0 + wn + j * 8 + t4 * 2 + (q & 1);
                if (p < R.count && col < a.n) {
                    float* d = reinterpret_cast<float*>(a.d) + (size_t)z * a.d_z_stride + (size_t)(R.begin + p) * a.ldd + col;
                    dense_store(a, d, z, R.begin + p, col, acc[i][j][q]);
                }
            }
}

}  // namespace uzu

extern "C" void uzu_dense_linear_encode(uzu_command_buffer* cmd, const uzu_dense_linear_args* args) {
    using namespace uzu;
    if (!encodable(cmd, "dense_linear")) return;
    uzu_dense_linear_args a = *args;
    if (!a.a || !a.w || !a.d || (a.weights_dt != UZU_DT_BF16 && a.weights_dt != UZU_DT_F32) || a.batch == 0 || (a.rows_map && !a.group_offsets && a.batch != 1)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "dense_linear: null operand / bad dtype / bad batch");
        return;
    }
    if (a.a_op > 2 || a.glu_kind > 1 || (a.gate_bias && !a.gate) || (a.pair_rows && (a.gate || a.bias || a.accumulate || a.col_scale))) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "dense_linear: unknown A operation, or a paired epilogue combined with gate / bias / accumulate");
        return;
    }
    if ((a.post_weight && (a.accumulate || a.batch != 1 || a.pair_rows || a.token_table)) ||
        (a.token_table && (!a.token_ids || a.pair_rows || a.batch != 1 || (a.token_gate_dt != UZU_DT_BF16 && a.token_gate_dt != UZU_DT_F32) ||
                           a.token_column + a.n > a.token_table_stride))) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "dense_linear: the sandwich / token-gate epilogues take one plain product (no accumulate, no pairs, no batch)");
        return;
    }
    if (a.m == 0 || a.n == 0) return;
    if (a.a_bf16) {      // A rows that are bf16 already (a cache's rows): the tensor-memory form reads them as they are
        const bool dense_rows = a.lda == 0 || a.lda == a.k;
        a.lda = a.k;
        if (!dense_rows || a.a_op || a.post_weight || a.token_table || !dense_umma_applicable(a)) {
            cmd->record_error(UZU_ERROR_UNSUPPORTED, "dense_linear: bf16 activations need the tcgen05 form (bf16 weights, dense rows, a workspace pointer, m >= 128, k a multiple of 64, n >= 64, no A operation)");
            return;
        }
        encode_dense_umma(cmd, a);
        return;
    }
    if (a.lda == 0) a.lda = a.k;
    if (a.ldd == 0) a.ldd = a.n;
    const bool bf16 = a.weights_dt == UZU_DT_BF16;
    static const bool no_tensor = getenv("UZU_DENSE_NO_TENSOR") != nullptr;
    if (a.m <= DL_MAX_ROWS) {
        // warps per output feature: enough warps in flight to cover the memory latency when there are few features and k is long
        const uint32_t sweep = bf16 ? 256 : 128;
        const uint64_t features = (uint64_t)a.n * a.batch;
        const int ks = (features >= 4096 || a.k < 2 * sweep) ? 1 : (features >= 2048 || a.k < 4 * sweep) ? 2 : 4;
        dim3 grid((a.n * ks + 7) / 8, a.batch);
        auto go = [&](auto kernel) { launch(cmd, "dense_rows_kernel", kernel, grid, dim3(256), 0, a); };
        auto pick = [&](auto tw, auto ks_c, auto pair_c) {
            using TW = decltype(tw);
            constexpr int KSv = decltype(ks_c)::value;
            constexpr bool PAIRv = decltype(pair_c)::value;
            if (a.m == 1) go(dense_rows_kernel<TW, KSv, PAIRv, 1>);
            else go(dense_rows_kernel<TW, KSv, PAIRv, DL_MAX_ROWS>);
        };
        auto by_pair = [&](auto tw, auto ks_c) {
            if (a.pair_rows) pick(tw, ks_c, std::true_type{});
            else pick(tw, ks_c, std::false_type{});
        };
        auto by_ks = [&](auto tw) {
            if (ks == 1) by_pair(tw, std::integral_constant<int, 1>{});
            else if (ks == 2) by_pair(tw, std::integral_constant<int, 2>{});
            else by_pair(tw, std::integral_constant<int, 4>{});
        };
        if (bf16) by_ks(__nv_bfloat16{});
        else by_ks(float{});
        return;
    }
    if (a.pair_rows) {
        cmd->record_error(UZU_ERROR_UNSUPPORTED, "dense_linear: the paired gated-unit epilogue covers passes of at most 8 rows");
        return;
    }
    if (!a.post_weight && !a.token_table && dense_umma_applicable(a)) {
        encode_dense_umma(cmd, a);
        return;
    }
    static const bool no_tensor128 = getenv("UZU_DENSE_NO_TENSOR128") != nullptr;     // A/B runs
    if (bf16 && a.m >= 96 && !no_tensor && !no_tensor128) {
        dim3 grid((a.n + T8_BN - 1) / T8_BN, (a.m + T8_BM - 1) / T8_BM, a.batch);
        dense_tensor128_kernel<<<grid, 256, 0, cmd->ctx->stream>>>(a);
        after_launch(cmd, "dense_tensor128_kernel");
        return;
    }
    if (bf16 && a.m >= 32 && !no_tensor) {
        dim3 grid((a.n + TC_BN - 1) / TC_BN, (a.m + TC_BM - 1) / TC_BM, a.batch);
        dense_tensor_kernel<<<grid, 128, 0, cmd->ctx->stream>>>(a);
        after_launch(cmd, "dense_tensor_kernel");
        return;
    }
    dim3 grid((a.n + DT_BN - 1) / DT_BN, (a.m + DT_BM - 1) / DT_BM, a.batch);
    if (bf16) dense_tile_kernel<__nv_bfloat16><<<grid, 256, 0, cmd->ctx->stream>>>(a);
    else dense_tile_kernel<float><<<grid, 256, 0, cmd->ctx->stream>>>(a);
    after_launch(cmd, "dense_tile_kernel");
}
