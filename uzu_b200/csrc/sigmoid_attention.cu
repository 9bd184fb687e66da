// Sigmoid attention: every visible key gets the weight sigmoid(score) on its own -- no softmax, no normalisation over keys, no rotation.
// Positions enter through a per-head distance bias r1 * ln(1 + r2 * (i - j)) taken off the score and through a query temperature
// 1 + coef * ln(floor((p + 1) / every) + 1); a per-head bias is added to the score. Keys and queries are RMS-normed over the whole
// projection (all heads at once) before they are split into heads. Grouped key / value heads; key and value sizes may differ.
//   prepare: per token the normed, temperature-scaled query row (f32) and, for a layer that owns its cache, the normed key row and the
//            value row at the token's position (a layer that reads another layer's cache writes nothing);
//   attend:  one CTA per (query token, head, split of the keys, in tiles of 16): a warp per key, lanes across the head's channels (coalesced rows),
//            four keys of a warp in flight; because the weights are not normalised the partial results of the splits simply add: the
//            last split to finish (a ticket per query and head) adds them in split order, so no second launch and no dependence on
//            the order of arrival;
//   attend, tensor pipe (sigmoid_attention_mma_kernel): bf16 caches and passes of >= 64 rows (described at the kernel).
// The cache holds bf16 or f32 rows; scores, weights and sums are f32.
#include "common.cuh"

namespace uzu {

namespace {

template <typename T>
__device__ __forceinline__ void sa_store(T* p, float v);
template <>
__device__ __forceinline__ void sa_store<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void sa_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// a 4-byte word of a cache row: EPW = 1 element (f32, or one bf16 of an odd-sized row) or 2 bf16 elements
template <typename T, int EPW>
__device__ __forceinline__ void sa_load(const T* p, float (&x)[EPW]) {
    if constexpr (sizeof(T) == 4) {
        x[0] = *p;
    } else if constexpr (EPW == 1) {
        x[0] = __bfloat162float(*p);
    } else {
        const uint32_t u = *reinterpret_cast<const uint32_t*>(p);
        x[0] = __uint_as_float(u << 16);
        x[1] = __uint_as_float(u & 0xffff0000u);
    }
}

__device__ __forceinline__ float sa_temperature(uint32_t pos, uint32_t every, float coef) {
    return every ? 1.0f + coef * logf((float)((pos + 1) / every + 1)) : 1.0f;
}

}  // namespace

// grid (rows, 3): unit 0 the query row, unit 1 the key row, unit 2 the value row
template <typename T>
__global__ void __launch_bounds__(256) sigmoid_attention_prepare_kernel(const uzu_sigmoid_attention_prepare_args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[32];
    const uint32_t t = blockIdx.x, unit = blockIdx.y;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t pos = prefix + t;
    if (unit == 0) {
        if (!a.q) return;
        const float* src = reinterpret_cast<const float*>(a.q) + (size_t)t * a.q_stride;
        const float* sc = reinterpret_cast<const float*>(a.q_scales);
        float* out = reinterpret_cast<float*>(a.query) + (size_t)t * a.q_n;
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x; i < a.q_n; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.q_n + a.epsilon);
        const float temp = sa_temperature(pos, a.temp_every, a.temp_coef);
        for (uint32_t i = threadIdx.x; i < a.q_n; i += blockDim.x) out[i] = src[i] * inv * (sc ? sc[i] : 1.0f) * temp;
    } else if (unit == 1) {
        if (!a.k) return;
        const float* src = reinterpret_cast<const float*>(a.k) + (size_t)t * a.k_stride;
        const float* sc = reinterpret_cast<const float*>(a.k_scales);
        T* out = reinterpret_cast<T*>(a.keys) + (size_t)pos * a.k_n;
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x; i < a.k_n; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.k_n + a.epsilon);
        for (uint32_t i = threadIdx.x; i < a.k_n; i += blockDim.x) sa_store<T>(out + i, src[i] * inv * (sc ? sc[i] : 1.0f));
    } else {
        if (!a.v) return;
        const float* src = reinterpret_cast<const float*>(a.v) + (size_t)t * a.v_stride;
        T* out = reinterpret_cast<T*>(a.values) + (size_t)pos * a.v_n;
        for (uint32_t i = threadIdx.x; i < a.v_n; i += blockDim.x) sa_store<T>(out + i, src[i]);
    }
}

constexpr int SA_WARPS = 4, SA_TILE = 16, SA_UNROLL = 4;

// WPL = words of a head's key / value row per lane (the larger of the two)
template <typename T, int EPW, int WPL>
__global__ void __launch_bounds__(SA_WARPS * 32) sigmoid_attention_kernel(const uzu_sigmoid_attention_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sa_part[];          // [SA_WARPS][vdim]
    __shared__ uint32_t is_last;
    const uint32_t t = blockIdx.x, h = blockIdx.y, split = blockIdx.z, splits = gridDim.z;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t p = prefix + t, keys = p + 1;                 // causal: positions 0 .. own
    const uint32_t tiles = (keys + SA_TILE - 1) / SA_TILE, per = (tiles + splits - 1) / splits;
    const uint32_t j_begin = min(keys, split * per * SA_TILE), j_end = min(keys, (split + 1) * per * SA_TILE);
    const uint32_t g = h / (a.heads / a.kv_heads);
    const uint32_t dwords = (a.dim + EPW - 1) / EPW, vwords = (a.vdim + EPW - 1) / EPW;
    const float r1 = a.dist_r1 ? reinterpret_cast<const float*>(a.dist_r1)[h] : 0.0f;
    const float r2 = a.dist_r2 ? reinterpret_cast<const float*>(a.dist_r2)[h] : 0.0f;
    const float pb = a.head_bias ? reinterpret_cast<const float*>(a.head_bias)[h] : 0.0f;
    float q[WPL][EPW], acc[WPL][EPW];
    {
        const float* qrow = reinterpret_cast<const float*>(a.query) + ((size_t)t * a.heads + h) * a.dim;
#pragma unroll
        for (int i = 0; i < WPL; ++i) {
            const uint32_t w = lane + 32u * i;
#pragma unroll
            for (int e = 0; e < EPW; ++e) {
                q[i][e] = (w < dwords && w * EPW + e < a.dim) ? qrow[w * EPW + e] * a.scale : 0.0f;
                acc[i][e] = 0.0f;
            }
        }
    }
    const T* kbase = reinterpret_cast<const T*>(a.keys) + (size_t)g * a.dim;
    const T* vbase = reinterpret_cast<const T*>(a.values) + (size_t)g * a.vdim;
    const size_t kstride = (size_t)a.kv_heads * a.dim, vstride = (size_t)a.kv_heads * a.vdim;
    constexpr bool EARLY_V = WPL <= 2;          // small heads: the value words are requested with the key words, before the scores exist
    for (uint32_t j0 = j_begin + warp * SA_UNROLL; j0 < j_end; j0 += SA_WARPS * SA_UNROLL) {
        float s[SA_UNROLL];
        float vx[EARLY_V ? SA_UNROLL : 1][WPL][EPW];
#pragma unroll
        for (int u = 0; u < SA_UNROLL; ++u) {
            const uint32_t j = j0 + u;
            s[u] = 0.0f;
            if (j < j_end) {
                const T* krow = kbase + j * kstride;
                float kx[WPL][EPW];
#pragma unroll
                for (int i = 0; i < WPL; ++i) {
                    const uint32_t w = lane + 32u * i;
                    if (w < dwords) sa_load<T, EPW>(krow + (size_t)w * EPW, kx[i]);
                }
                if constexpr (EARLY_V) {
                    const T* vrow = vbase + j * vstride;
#pragma unroll
                    for (int i = 0; i < WPL; ++i) {
                        const uint32_t w = lane + 32u * i;
                        if (w < vwords) sa_load<T, EPW>(vrow + (size_t)w * EPW, vx[u][i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < WPL; ++i) {
                    const uint32_t w = lane + 32u * i;
                    if (w < dwords) {
#pragma unroll
                        for (int e = 0; e < EPW; ++e) s[u] = fmaf(q[i][e], kx[i][e], s[u]);
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < SA_UNROLL; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
#pragma unroll
        for (int u = 0; u < SA_UNROLL; ++u) {
            const uint32_t j = j0 + u;
            if (j < j_end) {
                const float score = s[u] - r1 * log1pf(r2 * (float)(p - j)) + pb;
                const float wgt = 1.0f / (1.0f + expf(-score));
                const T* vrow = vbase + j * vstride;
#pragma unroll
                for (int i = 0; i < WPL; ++i) {
                    const uint32_t w = lane + 32u * i;
                    if (w < vwords) {
                        float x[EPW];
                        if constexpr (EARLY_V) {
#pragma unroll
                            for (int e = 0; e < EPW; ++e) x[e] = vx[u][i][e];
                        } else {
                            sa_load<T, EPW>(vrow + (size_t)w * EPW, x);
                        }
#pragma unroll
                        for (int e = 0; e < EPW; ++e) acc[i][e] = fmaf(wgt, x[e], acc[i][e]);
                    }
                }
            }
        }
    }
    // the warps' sums meet in warp order
#pragma unroll
    for (int i = 0; i < WPL; ++i) {
        const uint32_t w = lane + 32u * i;
#pragma unroll
        for (int e = 0; e < EPW; ++e)
            if (w < vwords && w * EPW + e < a.vdim) sa_part[warp * a.vdim + w * EPW + e] = acc[i][e];
    }
    __syncthreads();
    float* out = reinterpret_cast<float*>(a.out) + ((size_t)t * a.heads + h) * a.vdim;
    float* mine = splits > 1 ? reinterpret_cast<float*>(a.partials) + (((size_t)t * a.heads + h) * splits + split) * a.vdim : out;
    for (uint32_t c = tid; c < a.vdim; c += blockDim.x) {
        float v = 0.0f;
#pragma unroll
        for (int wq = 0; wq < SA_WARPS; ++wq) v += sa_part[wq * a.vdim + c];
        mine[c] = v;
    }
    if (splits == 1) return;
    __threadfence();
    __syncthreads();
    uint32_t* ticket = reinterpret_cast<uint32_t*>(a.tickets) + (size_t)t * a.heads + h;
    if (tid == 0) is_last = atomicAdd(ticket, 1u) == splits - 1 ? 1u : 0u;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* parts = reinterpret_cast<const float*>(a.partials) + ((size_t)t * a.heads + h) * splits * a.vdim;
    for (uint32_t c = tid; c < a.vdim; c += blockDim.x) {
        float v = 0.0f;
        uint32_t sp = 0;
        for (; sp + 8 <= splits; sp += 8) {        // eight loads in flight, added in split order
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = __ldcg(parts + (size_t)(sp + u) * a.vdim + c);
#pragma unroll
            for (int u = 0; u < 8; ++u) v += x[u];
        }
        for (; sp < splits; ++sp) v += __ldcg(parts + (size_t)sp * a.vdim + c);
        out[c] = v;
    }
    if (tid == 0) *ticket = 0;
}

template <typename T, int EPW>
static void launch_sigmoid_attention(uzu_command_buffer* cmd, const uzu_sigmoid_attention_args& a, uint32_t splits) {
    const uint32_t words = (std::max(a.dim, a.vdim) + EPW - 1) / EPW, wpl = (words + 31) / 32;
    const dim3 grid(a.rows, a.heads, splits), block(SA_WARPS * 32);
    const size_t smem = (size_t)SA_WARPS * a.vdim * sizeof(float);
    if (wpl <= 1) launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 1>, grid, block, smem, a);
    else if (wpl <= 2) launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 2>, grid, block, smem, a);
    else if (wpl <= 4) launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 4>, grid, block, smem, a);
    else if (wpl <= 8) launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 8>, grid, block, smem, a);
    else launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 16>, grid, block, smem, a);
}

bool encode_sigmoid_attention_mma(uzu_command_buffer* cmd, const uzu_sigmoid_attention_args& a);

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_sigmoid_attention_prepare_encode(uzu_command_buffer* cmd, const uzu_sigmoid_attention_prepare_args* a) {
    if (!encodable(cmd, "sigmoid_attention_prepare")) return;
    if ((a->cache_dt != UZU_DT_BF16 && a->cache_dt != UZU_DT_F32) || (a->q && !a->query) || (a->k && !a->keys) || (a->v && !a->values)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "sigmoid_attention_prepare: bad cache type or a projection without its destination");
        return;
    }
    if (a->rows == 0) return;
    if (a->cache_dt == UZU_DT_BF16)
        launch(cmd, "sigmoid_attention_prepare_kernel", sigmoid_attention_prepare_kernel<__nv_bfloat16>, dim3(a->rows, 3), dim3(256), 0, *a);
    else
        launch(cmd, "sigmoid_attention_prepare_kernel", sigmoid_attention_prepare_kernel<float>, dim3(a->rows, 3), dim3(256), 0, *a);
}

void uzu_sigmoid_attention_encode(uzu_command_buffer* cmd, const uzu_sigmoid_attention_args* args) {
    if (!encodable(cmd, "sigmoid_attention")) return;
    uzu_sigmoid_attention_args a = *args;
    if (!a.query || !a.keys || !a.values || !a.out || (a.cache_dt != UZU_DT_BF16 && a.cache_dt != UZU_DT_F32) || a.heads == 0 || a.kv_heads == 0 ||
        a.heads % a.kv_heads != 0 || a.dim == 0 || a.vdim == 0 || a.dim > 512 || a.vdim > 512) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "sigmoid_attention: null operand, bad cache type, head counts that do not divide, or a head size outside 1..512");
        return;
    }
    if (a.rows == 0) return;
    uint32_t splits = std::max(1u, a.splits);
    if (splits > 1 && (!a.partials || !a.tickets)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "sigmoid_attention: key splits need the partial-sum and ticket scratch");
        return;
    }
    if (splits == 1 && encode_sigmoid_attention_mma(cmd, a)) return;
    if (a.cache_dt == UZU_DT_F32) {
        launch_sigmoid_attention<float, 1>(cmd, a, splits);
    } else if (a.dim % 2 == 0 && a.vdim % 2 == 0 && (a.keys & 3) == 0 && (a.values & 3) == 0) {
        launch_sigmoid_attention<__nv_bfloat16, 2>(cmd, a, splits);
    } else {
        launch_sigmoid_attention<__nv_bfloat16, 1>(cmd, a, splits);
    }
}

}  // extern "C"

// ---- tensor pipe (bf16 caches, passes of >= 64 rows) ----------------------------------------------------------------------------------
// One CTA = 64 query rows of one head (4 warps x 16 rows), key tiles of 64 from position 0 up to the CTA's last row; the next tile's
// keys and values arrive by cp.async while the current one is used. mma.sync.m16n8k16 (bf16 x bf16 -> f32):
//   S = (q * scale) . K^T     with q = q_hi + q_lo, two bf16 numbers per f32 query entry (two MMAs per tile of S);
//   w = sigmoid(S - r1 ln(1 + r2 (i - j)) + pb), 0 for j > i, in f32 on the accumulator fragment;
//   O += w . V                with w = w_hi + w_lo again, the accumulator fragment of S re-used as the A fragment (two adjacent
//                             8-key tiles form one 16-key step), V fragments by ldmatrix.trans from the row-major tile.
// The split keeps the error of the query and of the weights below 2^-16 relative, so only the cache's own bf16 rounding remains.
// With chunk_tiles the key tiles of a row tile are cut into chunks of that many, one CTA each: late row tiles of a long prompt would
// otherwise walk many times the keys of early ones while every CTA of the launch is resident from the start.
namespace uzu {

namespace {

constexpr int SM_BM = 64, SM_BN = 64, SM_PAD = 8;

__device__ __forceinline__ void sm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void sm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void sm_cp_async16(void* smem_ptr, const void* gmem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(gmem_ptr) : "memory");
}

// x = hi + lo with both parts bf16; a pair of values packed for an MMA fragment
__device__ __forceinline__ void sm_split_pair(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
    const __nv_bfloat162 h = __halves2bfloat162(h0, h1);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x0 - __bfloat162float(h0), x1 - __bfloat162float(h1));
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

}  // namespace

// DK = most 16-channel steps of a key row (dim / 16 rounded up to 4 or 8), DV = most 16-column blocks of a value row
template <int DK, int DV>
__global__ void __launch_bounds__(128) sigmoid_attention_mma_kernel(const uzu_sigmoid_attention_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char sm_raw[];
    const uint32_t dim = a.dim, vdim = a.vdim, ldk = dim + SM_PAD, ldv = vdim + SM_PAD, dk = dim / 16, dv = vdim / 16;
    __nv_bfloat16* q_hi = reinterpret_cast<__nv_bfloat16*>(sm_raw);      // [64][ldk]
    __nv_bfloat16* q_lo = q_hi + SM_BM * ldk;
    __nv_bfloat16* k_s = q_lo + SM_BM * ldk;                             // [2][64][ldk]
    __nv_bfloat16* v_s = k_s + 2 * SM_BN * ldk;                          // [2][64][ldv]
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const uint32_t h = blockIdx.y, kvh = h / (a.heads / a.kv_heads);
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    // blockIdx.x counts (row tile, chunk of its key tiles) pairs, the row tiles with the most keys first
    const uint32_t chunk_tiles = a.chunk_tiles ? a.chunk_tiles : 0xFFFFu;
    uint32_t mt = (a.rows + SM_BM - 1) / SM_BM, chunk = blockIdx.x, nchunks = 1;
    while (mt > 0) {
        --mt;
        const uint32_t nt = (prefix + min(a.rows, (mt + 1) * SM_BM) + SM_BN - 1) / SM_BN;
        nchunks = (nt + chunk_tiles - 1) / chunk_tiles;
        if (chunk < nchunks) break;
        chunk -= nchunks;
    }
    const uint32_t m0 = mt * SM_BM;
    const uint32_t rows_here = min((uint32_t)SM_BM, a.rows - m0);
    const uint32_t nkeys = prefix + m0 + rows_here, ntiles_all = (nkeys + SM_BN - 1) / SM_BN;
    const uint32_t t_begin = min(ntiles_all, chunk * chunk_tiles), ntiles = min(ntiles_all, t_begin + chunk_tiles);
    // scores are kept in units of ln 2: sigmoid(s) = 1 / (1 + 2^(-s log2 e)), and r1 ln(x) log2 e = r1 log2(x)
    constexpr float kLog2e = 1.4426950408889634f;
    const float qscale = a.scale * kLog2e;
    const float r1 = a.dist_r1 ? reinterpret_cast<const float*>(a.dist_r1)[h] : 0.0f;
    const float r2 = a.dist_r2 ? reinterpret_cast<const float*>(a.dist_r2)[h] : 0.0f;
    const float pb = (a.head_bias ? reinterpret_cast<const float*>(a.head_bias)[h] : 0.0f) * kLog2e;
    const __nv_bfloat16* keys = reinterpret_cast<const __nv_bfloat16*>(a.keys) + (size_t)kvh * dim;
    const __nv_bfloat16* values = reinterpret_cast<const __nv_bfloat16*>(a.values) + (size_t)kvh * vdim;
    const size_t kstride = (size_t)a.kv_heads * dim, vstride = (size_t)a.kv_heads * vdim;
    // a thread's 16-byte pieces of a tile: piece tid, tid + 128, ... of rows x (row size / 8); row and column advance without divisions
    const uint32_t kc = dim / 8, vc = vdim / 8;
    const uint32_t k_r0 = tid / kc, k_c0 = tid % kc, k_dr = 128 / kc, k_dc = 128 % kc;
    const uint32_t v_r0 = tid / vc, v_c0 = tid % vc, v_dr = 128 / vc, v_dc = 128 % vc;
    auto load_rows = [&](__nv_bfloat16* dst_tile, uint32_t ld, const __nv_bfloat16* src, size_t stride, uint32_t j0, uint32_t r, uint32_t c, uint32_t dr,
                         uint32_t dc, uint32_t pieces_per_row) {
        while (r < SM_BN) {
            __nv_bfloat16* dst = dst_tile + r * ld + c * 8;
            if (j0 + r < nkeys) sm_cp_async16(dst, src + (size_t)(j0 + r) * stride + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            r += dr; c += dc;
            if (c >= pieces_per_row) { c -= pieces_per_row; ++r; }
        }
    };
    auto load_tile = [&](uint32_t t, uint32_t buf) {      // rows past the last key are zero: cache pages beyond the context may not exist
        const uint32_t j0 = t * SM_BN;
        load_rows(k_s + buf * SM_BN * ldk, ldk, keys, kstride, j0, k_r0, k_c0, k_dr, k_dc, kc);
        load_rows(v_s + buf * SM_BN * ldv, ldv, values, vstride, j0, v_r0, v_c0, v_dr, v_dc, vc);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float o[2 * DV][4];
#pragma unroll
    for (int n = 0; n < 2 * DV; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[n][c] = 0.0f;
    const uint32_t row_lo = warp * 16 + g;                     // this thread's rows of the tile: row_lo and row_lo + 8
    const uint32_t i_lo = prefix + m0 + row_lo, i_warp_last = prefix + m0 + warp * 16 + 15;
    load_tile(t_begin, t_begin & 1);
    {   // the query tile, scaled, as hi + lo; sixteen loads of a thread in flight, behind the first tile's requests
        const float* q = reinterpret_cast<const float*>(a.query) + (size_t)m0 * a.heads * dim + (size_t)h * dim;
        const uint32_t pairs = dim / 2, total = SM_BM * pairs;
        for (uint32_t i0 = tid; i0 < total; i0 += 16 * blockDim.x) {
            float2 x[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const uint32_t i = i0 + u * blockDim.x, r = i / pairs, c = (i - r * pairs) * 2;
                x[u] = make_float2(0.0f, 0.0f);
                if (i < total && r < rows_here) x[u] = *reinterpret_cast<const float2*>(q + (size_t)r * a.heads * dim + c);
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const uint32_t i = i0 + u * blockDim.x, r = i / pairs, c = (i - r * pairs) * 2;
                if (i < total) {
                    uint32_t hi, lo;
                    sm_split_pair(x[u].x * qscale, x[u].y * qscale, hi, lo);
                    *reinterpret_cast<uint32_t*>(q_hi + r * ldk + c) = hi;
                    *reinterpret_cast<uint32_t*>(q_lo + r * ldk + c) = lo;
                }
            }
        }
    }
    for (uint32_t t = t_begin; t < ntiles; ++t) {
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();                                       // tile t is in place, tile t - 1 is used up
        if (t + 1 < ntiles) load_tile(t + 1, (t + 1) & 1);
        const uint32_t j0 = t * SM_BN;
        if (j0 > i_warp_last) continue;                        // nothing of this tile is visible to the warp's rows
        const __nv_bfloat16* kt = k_s + (t & 1) * SM_BN * ldk;
        const __nv_bfloat16* vt = v_s + (t & 1) * SM_BN * ldv;
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[n][c] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < DK; ++kk) {
            if ((uint32_t)kk < dk) {
                uint32_t ah[4], al[4];
                const uint32_t off = row_lo * ldk + kk * 16 + t4 * 2;
                ah[0] = *reinterpret_cast<const uint32_t*>(q_hi + off);
                ah[1] = *reinterpret_cast<const uint32_t*>(q_hi + off + 8 * ldk);
                ah[2] = *reinterpret_cast<const uint32_t*>(q_hi + off + 8);
                ah[3] = *reinterpret_cast<const uint32_t*>(q_hi + off + 8 * ldk + 8);
                al[0] = *reinterpret_cast<const uint32_t*>(q_lo + off);
                al[1] = *reinterpret_cast<const uint32_t*>(q_lo + off + 8 * ldk);
                al[2] = *reinterpret_cast<const uint32_t*>(q_lo + off + 8);
                al[3] = *reinterpret_cast<const uint32_t*>(q_lo + off + 8 * ldk + 8);
                uint32_t kb0[8], kb1[8];
#pragma unroll
                for (int n = 0; n < 8; ++n) {
                    const __nv_bfloat16* kb = kt + (n * 8 + g) * ldk + kk * 16 + t4 * 2;
                    kb0[n] = *reinterpret_cast<const uint32_t*>(kb);
                    kb1[n] = *reinterpret_cast<const uint32_t*>(kb + 8);
                }
                // the hi and the lo product of a tile use the same accumulator: eight other MMAs lie between them
#pragma unroll
                for (int n = 0; n < 8; ++n) sm_mma(s[n], ah, kb0[n], kb1[n]);
#pragma unroll
                for (int n = 0; n < 8; ++n) sm_mma(s[n], al, kb0[n], kb1[n]);
            }
        }
        // weights on the fragment: element c of tile n is row row_lo + 8 * (c >> 1), key j0 + n * 8 + t4 * 2 + (c & 1); its distance
        // i - j is the thread's base distance plus a constant. Only tiles that reach the diagonal need the mask.
        const float d0 = (float)((int)i_lo - (int)j0 - (int)(t4 * 2));
        const bool diagonal = j0 + SM_BN - 1 > prefix + m0 + warp * 16;
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float d = d0 + (float)(8 * (c >> 1) - n * 8 - (c & 1));
                const float score = s[n][c] - r1 * __log2f(fmaf(r2, fmaxf(d, 0.0f), 1.0f)) + pb;
                float w = __fdividef(1.0f, 1.0f + exp2f(-score));
                if (diagonal && d < 0.0f) w = 0.0f;
                s[n][c] = w;
            }
#pragma unroll
        for (int kk = 0; kk < SM_BN / 16; ++kk) {
            uint32_t ph[4], pl[4];
            sm_split_pair(s[2 * kk][0], s[2 * kk][1], ph[0], pl[0]);
            sm_split_pair(s[2 * kk][2], s[2 * kk][3], ph[1], pl[1]);
            sm_split_pair(s[2 * kk + 1][0], s[2 * kk + 1][1], ph[2], pl[2]);
            sm_split_pair(s[2 * kk + 1][2], s[2 * kk + 1][3], ph[3], pl[3]);
#pragma unroll
            for (int n = 0; n < DV; n += 2) {      // two 16-column blocks at a time: four independent accumulators between hi and lo
                if ((uint32_t)n < dv) {
                    const bool two = (uint32_t)n + 1 < dv;
                    uint32_t b[4], c[4] = {0, 0, 0, 0};
                    const __nv_bfloat16* vb = vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + (lane >> 4) * 8;
                    sm_ldmatrix_x4_trans(b, vb + n * 16);
                    if (two) sm_ldmatrix_x4_trans(c, vb + (n + 1) * 16);
                    sm_mma(o[2 * n], ph, b[0], b[1]);
                    sm_mma(o[2 * n + 1], ph, b[2], b[3]);
                    if (two) {
                        sm_mma(o[2 * n + 2], ph, c[0], c[1]);
                        sm_mma(o[2 * n + 3], ph, c[2], c[3]);
                    }
                    sm_mma(o[2 * n], pl, b[0], b[1]);
                    sm_mma(o[2 * n + 1], pl, b[2], b[3]);
                    if (two) {
                        sm_mma(o[2 * n + 2], pl, c[0], c[1]);
                        sm_mma(o[2 * n + 3], pl, c[2], c[3]);
                    }
                }
            }
        }
    }
    // one chunk: straight to the output. Several: every chunk leaves its partial tile in `partials` [chunk][row][heads * vdim]; weights are
    // not normalised, so the partial tiles simply add, and the last chunk to finish adds them in chunk order.
    const size_t row_stride = (size_t)a.heads * vdim;
    float* out = reinterpret_cast<float*>(a.out) + (size_t)m0 * row_stride + (size_t)h * vdim;
    float* mine = nchunks > 1 ? reinterpret_cast<float*>(a.partials) + ((size_t)chunk * a.rows + m0) * row_stride + (size_t)h * vdim : out;
#pragma unroll
    for (int n = 0; n < 2 * DV; ++n) {
        if ((uint32_t)n < 2 * dv) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint32_t r = row_lo + 8 * half;
                if (r < rows_here) *reinterpret_cast<float2*>(mine + (size_t)r * row_stride + n * 8 + t4 * 2) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
            }
        }
    }
    if (nchunks == 1) return;
    __shared__ uint32_t is_last;
    __threadfence();
    __syncthreads();
    uint32_t* ticket = reinterpret_cast<uint32_t*>(a.tickets) + (size_t)mt * a.heads + h;
    if (tid == 0) is_last = atomicAdd(ticket, 1u) == nchunks - 1 ? 1u : 0u;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* parts = reinterpret_cast<const float*>(a.partials) + (size_t)m0 * row_stride + (size_t)h * vdim;
    const uint32_t quads = vdim / 4;
    for (uint32_t i = tid; i < rows_here * quads; i += blockDim.x) {
        const uint32_t r = i / quads, c = (i - r * quads) * 4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t c0 = 0; c0 < nchunks; c0 += 4) {          // four chunks' loads in flight, added in chunk order
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                x[u] = c0 + u < nchunks ? __ldcg(reinterpret_cast<const float4*>(parts + ((size_t)(c0 + u) * a.rows + r) * row_stride + c)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int u = 0; u < 4; ++u) { v.x += x[u].x; v.y += x[u].y; v.z += x[u].z; v.w += x[u].w; }
        }
        *reinterpret_cast<float4*>(out + (size_t)r * row_stride + c) = v;
    }
    if (tid == 0) *ticket = 0;
}

template <int DK, int DV>
static void launch_sigmoid_attention_mma(uzu_command_buffer* cmd, const uzu_sigmoid_attention_args& a) {
    const size_t smem = ((size_t)4 * SM_BM * (a.dim + SM_PAD) + (size_t)2 * SM_BN * (a.vdim + SM_PAD)) * sizeof(__nv_bfloat16);
    // the opt-in is made once per instance and device: for the largest head sizes the instance serves
    constexpr size_t smem_most = ((size_t)4 * SM_BM * (DK * 16 + SM_PAD) + (size_t)2 * SM_BN * (DV * 16 + SM_PAD)) * sizeof(__nv_bfloat16);
    static std::atomic<uint64_t> opt_in{0};
    opt_in_dynamic_smem(cmd, sigmoid_attention_mma_kernel<DK, DV>, (int)smem_most, opt_in);
    uint32_t ctas = 0;                           // (row tile, chunk) pairs
    for (uint32_t mt = 0; mt < (a.rows + SM_BM - 1) / SM_BM; ++mt) {
        const uint32_t nt = (a.prefix + std::min(a.rows, (mt + 1) * SM_BM) + SM_BN - 1) / SM_BN;
        ctas += a.chunk_tiles ? (nt + a.chunk_tiles - 1) / a.chunk_tiles : 1;
    }
    launch(cmd, "sigmoid_attention_mma_kernel", sigmoid_attention_mma_kernel<DK, DV>, dim3(ctas, a.heads), dim3(128), smem, a);
}

// Shapes the tensor-pipe kernel takes: bf16 caches, passes of >= 64 rows, key and value sizes multiples of 16 up to 128, 16-byte aligned
// caches and an 8-byte aligned query / output. Everything else (and every f32 cache) runs the plain kernel.
bool encode_sigmoid_attention_mma(uzu_command_buffer* cmd, const uzu_sigmoid_attention_args& a) {
    static const bool off = getenv("UZU_SIGMOID_NO_MMA") != nullptr;       // A/B runs
    if (off || a.cache_dt != UZU_DT_BF16 || a.rows < SM_BM || a.dim % 16 || a.vdim % 16 || a.dim > 128 || a.vdim > 128) return false;
    if ((a.keys & 15) || (a.values & 15) || (a.query & 7) || (a.out & 15) || a.dynamic_position) return false;
    if (a.chunk_tiles && (!a.partials || !a.tickets || (a.partials & 15))) return false;
    const bool k8 = a.dim > 64, v8 = a.vdim > 64;
    if (k8 && v8) launch_sigmoid_attention_mma<8, 8>(cmd, a);
    else if (k8) launch_sigmoid_attention_mma<8, 4>(cmd, a);
    else if (v8) launch_sigmoid_attention_mma<4, 8>(cmd, a);
    else launch_sigmoid_attention_mma<4, 4>(cmd, a);
    return true;
}

}  // namespace uzu
