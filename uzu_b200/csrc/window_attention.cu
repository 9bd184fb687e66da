// Windowed softmax attention with kept first tokens, rotated keys AND rotated values.
//   visibility:  key j is seen from position p when j <= p and (p - j < window or j < keep_first); kept tokens keep their true positions
//   score:       s = scale * temp[h] * q . k, then softcap * tanh(s / softcap); ordinary softmax over the visible keys
//   rotation:    q and k turn by their position over the first 2 * rot_pairs channels (pairs (2i, 2i+1), or (i, i + rot_pairs) with
//                rot_halves); the value of position j turns
//                by j over 2 * v_pairs channels with its own frequencies and is cached so; a head's weighted sum at position p is turned
//                back by -p. (The sum then holds every value turned by j - p, a relative position, without a second pass over the cache.)
//   prepare:     per token and head the RMS norm over the head's channels (one weight row shared by the heads), the rotation, the f32
//                query row and the cache rows (keys and values of the token's position);
//   attend:      one CTA per (query token, head, split of the visible keys): a warp per key with the lanes across the head's channels,
//                four keys of a warp in flight, a running (max, sum, weighted sum) per warp; warps meet in shared memory in warp order,
//                splits in a scratch: the last split to finish (a ticket per query and head) merges them in split order;
//   attend, tensor pipe (window_attention_mma_kernel): bf16 caches and passes of >= 64 rows (described at the kernel).
// The cache holds bf16 or f32 rows; scores, weights and sums are f32. Only the visible keys are read: a long context costs a decode
// step window + keep_first keys.
#include <type_traits>

#include "common.cuh"

namespace uzu {

namespace {

template <typename T>
__device__ __forceinline__ void wa_store(T* p, float v);
template <>
__device__ __forceinline__ void wa_store<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void wa_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// a 4-byte word of a cache row: EPW = 1 element (f32, or one bf16 of an odd-sized row) or 2 bf16 elements
template <typename T, int EPW>
__device__ __forceinline__ void wa_load(const T* p, float (&x)[EPW]) {
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

// one warp: out[0:n] = rotate(src * inv * scales) over the first `pairs` pairs, the rest copied
template <typename TO>
__device__ __forceinline__ void wa_rotate_row(const float* src, float inv, const float* scales, TO* out, uint32_t n, uint32_t pairs,
                                              const float* cosines, const float* sines, uint32_t lane) {
    for (uint32_t i = lane; 2 * i < n; i += 32) {
        const uint32_t c0 = 2 * i, c1 = c0 + 1;
        const float x0 = src[c0] * inv * (scales ? scales[c0] : 1.0f);
        const float x1 = c1 < n ? src[c1] * inv * (scales ? scales[c1] : 1.0f) : 0.0f;
        if (i < pairs) {
            const float c = cosines[i], s = sines[i];
            wa_store<TO>(out + c0, x0 * c - x1 * s);
            wa_store<TO>(out + c1, x1 * c + x0 * s);
        } else {
            wa_store<TO>(out + c0, x0);
            if (c1 < n) wa_store<TO>(out + c1, x1);
        }
    }
}

// the same with the pairs laid out as two halves: channel i turns with channel i + pairs (i < pairs), channels from 2 * pairs on are copied
template <typename TO>
__device__ __forceinline__ void wa_rotate_row_halves(const float* src, float inv, const float* scales, TO* out, uint32_t n, uint32_t pairs,
                                                     const float* cosines, const float* sines, uint32_t lane) {
    for (uint32_t i = lane; i < pairs; i += 32) {
        const uint32_t c0 = i, c1 = i + pairs;
        const float x0 = src[c0] * inv * (scales ? scales[c0] : 1.0f);
        const float x1 = src[c1] * inv * (scales ? scales[c1] : 1.0f);
        const float c = cosines[i], s = sines[i];
        wa_store<TO>(out + c0, x0 * c - x1 * s);
        wa_store<TO>(out + c1, x1 * c + x0 * s);
    }
    for (uint32_t i = 2 * pairs + lane; i < n; i += 32) wa_store<TO>(out + i, src[i] * inv * (scales ? scales[i] : 1.0f));
}

__device__ __forceinline__ float wa_head_inv_rms(const float* src, uint32_t n, float eps, uint32_t lane) {
    float ss = 0.0f;
    for (uint32_t i = lane; i < n; i += 32) ss = fmaf(src[i], src[i], ss);
    return 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
}

// the visible keys of position p, as one index range [0, total): first the kept tokens that the window no longer covers, then the window
struct Visible {
    uint32_t first, lo, total;
    __device__ __forceinline__ uint32_t key(uint32_t idx) const { return idx < first ? idx : lo + (idx - first); }
};

__device__ __forceinline__ Visible wa_visible(uint32_t p, uint32_t window, uint32_t keep_first) {
    Visible v;
    v.lo = (window && p + 1 > window) ? p + 1 - window : 0u;
    v.first = min(keep_first, v.lo);
    v.total = v.first + (p + 1 - v.lo);
    return v;
}

}  // namespace

// a warp per (token, unit): units [0, heads) queries, [heads, heads + kv_heads) keys, then values
template <typename T>
__global__ void __launch_bounds__(128) window_attention_prepare_kernel(const uzu_window_attention_prepare_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t units = a.heads + 2 * a.kv_heads;
    const uint32_t item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= a.rows * units) return;
    const uint32_t t = item / units, unit = item % units;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t pos = prefix + t;
    const float* cs = a.rot_pairs ? reinterpret_cast<const float*>(a.cosines) + (size_t)pos * a.rot_pairs : nullptr;
    const float* sn = a.rot_pairs ? reinterpret_cast<const float*>(a.sines) + (size_t)pos * a.rot_pairs : nullptr;
    if (unit < a.heads) {
        const float* src = reinterpret_cast<const float*>(a.q) + (size_t)t * a.q_stride + (size_t)unit * a.dim;
        const float* sc = reinterpret_cast<const float*>(a.q_scales);
        const float inv = sc ? wa_head_inv_rms(src, a.dim, a.epsilon, lane) : 1.0f;
        float* dst = reinterpret_cast<float*>(a.query) + ((size_t)t * a.heads + unit) * a.dim;
        if (a.rot_halves) wa_rotate_row_halves<float>(src, inv, sc, dst, a.dim, a.rot_pairs, cs, sn, lane);
        else wa_rotate_row<float>(src, inv, sc, dst, a.dim, a.rot_pairs, cs, sn, lane);
    } else if (unit < a.heads + a.kv_heads) {
        const uint32_t g = unit - a.heads;
        const float* src = reinterpret_cast<const float*>(a.k) + (size_t)t * a.k_stride + (size_t)g * a.dim;
        const float* sc = reinterpret_cast<const float*>(a.k_scales);
        const float inv = sc ? wa_head_inv_rms(src, a.dim, a.epsilon, lane) : 1.0f;
        T* dst = reinterpret_cast<T*>(a.keys) + ((size_t)pos * a.kv_heads + g) * a.dim;
        if (a.rot_halves) wa_rotate_row_halves<T>(src, inv, sc, dst, a.dim, a.rot_pairs, cs, sn, lane);
        else wa_rotate_row<T>(src, inv, sc, dst, a.dim, a.rot_pairs, cs, sn, lane);
    } else {
        const uint32_t g = unit - a.heads - a.kv_heads;
        const float* src = reinterpret_cast<const float*>(a.v) + (size_t)t * a.v_stride + (size_t)g * a.vdim;
        const float* vc = a.v_pairs ? reinterpret_cast<const float*>(a.v_cosines) + (size_t)pos * a.v_pairs : nullptr;
        const float* vs = a.v_pairs ? reinterpret_cast<const float*>(a.v_sines) + (size_t)pos * a.v_pairs : nullptr;
        wa_rotate_row<T>(src, 1.0f, nullptr, reinterpret_cast<T*>(a.values) + ((size_t)pos * a.kv_heads + g) * a.vdim, a.vdim, a.v_pairs, vc, vs, lane);
    }
}

constexpr int WA_WARPS = 4, WA_TILE = 16, WA_UNROLL = 4, WA_MAX_SPLITS = 128;

// WPL = words of a head's key / value row per lane (the larger of the two)
template <typename T, int EPW, int WPL>
__global__ void __launch_bounds__(WA_WARPS * 32) window_attention_kernel(const uzu_window_attention_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float wa_smem[];          // [WA_WARPS][vdim] partial sums, then [vdim] the head's result
    __shared__ float warp_m[WA_WARPS], warp_l[WA_WARPS];
    __shared__ uint32_t is_last;
    __shared__ float split_f[WA_MAX_SPLITS], split_l[WA_MAX_SPLITS];
    const uint32_t t = blockIdx.x, h = blockIdx.y, split = blockIdx.z, splits = gridDim.z;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t p = prefix + t;
    const Visible vis = wa_visible(p, a.window, a.keep_first);
    const uint32_t tiles = (vis.total + WA_TILE - 1) / WA_TILE, per = (tiles + splits - 1) / splits;
    const uint32_t i_begin = min(vis.total, split * per * WA_TILE), i_end = min(vis.total, (split + 1) * per * WA_TILE);
    const uint32_t g = h / (a.heads / a.kv_heads);
    const uint32_t dwords = (a.dim + EPW - 1) / EPW, vwords = (a.vdim + EPW - 1) / EPW;
    const float qscale = a.scale * (a.head_temp ? reinterpret_cast<const float*>(a.head_temp)[h] : 1.0f);
    const float cap = a.softcap, inv_cap = a.softcap > 0.0f ? 1.0f / a.softcap : 0.0f;
    float q[WPL][EPW], acc[WPL][EPW];
    {
        const float* qrow = reinterpret_cast<const float*>(a.query) + ((size_t)t * a.heads + h) * a.dim;
#pragma unroll
        for (int i = 0; i < WPL; ++i) {
            const uint32_t w = lane + 32u * i;
#pragma unroll
            for (int e = 0; e < EPW; ++e) {
                q[i][e] = (w < dwords && w * EPW + e < a.dim) ? qrow[w * EPW + e] * qscale : 0.0f;
                acc[i][e] = 0.0f;
            }
        }
    }
    const T* kbase = reinterpret_cast<const T*>(a.keys) + (size_t)g * a.dim;
    const T* vbase = reinterpret_cast<const T*>(a.values) + (size_t)g * a.vdim;
    const size_t kstride = (size_t)a.kv_heads * a.dim, vstride = (size_t)a.kv_heads * a.vdim;
    float run_m = -INFINITY, run_l = 0.0f;
    for (uint32_t i0 = i_begin + warp * WA_UNROLL; i0 < i_end; i0 += WA_WARPS * WA_UNROLL) {
        float s[WA_UNROLL];
        uint32_t key[WA_UNROLL];
#pragma unroll
        for (int u = 0; u < WA_UNROLL; ++u) {
            s[u] = 0.0f;
            key[u] = vis.key(min(i0 + u, i_end - 1));
            if (i0 + u < i_end) {
                const T* krow = kbase + key[u] * kstride;
#pragma unroll
                for (int i = 0; i < WPL; ++i) {
                    const uint32_t w = lane + 32u * i;
                    if (w < dwords) {
                        float kx[EPW];
                        wa_load<T, EPW>(krow + (size_t)w * EPW, kx);
#pragma unroll
                        for (int e = 0; e < EPW; ++e) s[u] = fmaf(q[i][e], kx[e], s[u]);
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < WA_UNROLL; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
        float batch_m = -INFINITY;
#pragma unroll
        for (int u = 0; u < WA_UNROLL; ++u) {
            if (cap > 0.0f) s[u] = cap * tanhf(s[u] * inv_cap);
            if (i0 + u >= i_end) s[u] = -INFINITY;
            batch_m = fmaxf(batch_m, s[u]);
        }
        const float new_m = fmaxf(run_m, batch_m);          // finite: the first key of the batch exists
        const float keep = expf(run_m - new_m);             // 0 at the first batch (run_m = -inf)
        run_m = new_m;
        run_l *= keep;
#pragma unroll
        for (int i = 0; i < WPL; ++i)
#pragma unroll
            for (int e = 0; e < EPW; ++e) acc[i][e] *= keep;
#pragma unroll
        for (int u = 0; u < WA_UNROLL; ++u) {
            if (i0 + u < i_end) {
                const float wgt = expf(s[u] - new_m);
                run_l += wgt;
                const T* vrow = vbase + key[u] * vstride;
#pragma unroll
                for (int i = 0; i < WPL; ++i) {
                    const uint32_t w = lane + 32u * i;
                    if (w < vwords) {
                        float x[EPW];
                        wa_load<T, EPW>(vrow + (size_t)w * EPW, x);
#pragma unroll
                        for (int e = 0; e < EPW; ++e) acc[i][e] = fmaf(wgt, x[e], acc[i][e]);
                    }
                }
            }
        }
    }
    // the warps' states meet in warp order
#pragma unroll
    for (int i = 0; i < WPL; ++i) {
        const uint32_t w = lane + 32u * i;
#pragma unroll
        for (int e = 0; e < EPW; ++e)
            if (w < vwords && w * EPW + e < a.vdim) wa_smem[warp * a.vdim + w * EPW + e] = acc[i][e];
    }
    if (lane == 0) { warp_m[warp] = run_m; warp_l[warp] = run_l; }
    __syncthreads();
    float cta_m = -INFINITY;
#pragma unroll
    for (int wq = 0; wq < WA_WARPS; ++wq) cta_m = fmaxf(cta_m, warp_m[wq]);
    float cta_l = 0.0f, wf[WA_WARPS];
#pragma unroll
    for (int wq = 0; wq < WA_WARPS; ++wq) {
        wf[wq] = warp_m[wq] == -INFINITY ? 0.0f : expf(warp_m[wq] - cta_m);
        cta_l = fmaf(warp_l[wq], wf[wq], cta_l);
    }
    float* result = wa_smem + WA_WARPS * a.vdim;     // [vdim]
    // a sink adds exp(sink - max) to the denominator; a head gate multiplies the head's result by its sigmoid
    const float sink = a.sinks ? reinterpret_cast<const float*>(a.sinks)[h] : -INFINITY;
    const float gate = a.head_gate ? 1.0f / (1.0f + expf(-reinterpret_cast<const float*>(a.head_gate)[(size_t)t * a.head_gate_stride + h])) : 1.0f;
    if (splits == 1) {
        const float norm = gate / (a.sinks ? cta_l + expf(sink - cta_m) : cta_l);
        for (uint32_t c = tid; c < a.vdim; c += blockDim.x) {
            float v = 0.0f;
#pragma unroll
            for (int wq = 0; wq < WA_WARPS; ++wq) v = fmaf(wa_smem[wq * a.vdim + c], wf[wq], v);
            result[c] = v * norm;
        }
    } else {
        const uint32_t pw = a.vdim + 2;
        float* mine = reinterpret_cast<float*>(a.partials) + (((size_t)t * a.heads + h) * splits + split) * pw;
        for (uint32_t c = tid; c < a.vdim; c += blockDim.x) {
            float v = 0.0f;
#pragma unroll
            for (int wq = 0; wq < WA_WARPS; ++wq) v = fmaf(wa_smem[wq * a.vdim + c], wf[wq], v);
            mine[2 + c] = v;
        }
        if (tid == 0) { mine[0] = cta_m; mine[1] = cta_l; }
        __threadfence();
        __syncthreads();
        uint32_t* ticket = reinterpret_cast<uint32_t*>(a.tickets) + (size_t)t * a.heads + h;
        if (tid == 0) is_last = atomicAdd(ticket, 1u) == splits - 1 ? 1u : 0u;
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        const float* parts = reinterpret_cast<const float*>(a.partials) + ((size_t)t * a.heads + h) * splits * pw;
        for (uint32_t sp = tid; sp < splits; sp += blockDim.x) {
            split_f[sp] = __ldcg(parts + (size_t)sp * pw);
            split_l[sp] = __ldcg(parts + (size_t)sp * pw + 1);
        }
        __syncthreads();
        float all_m = -INFINITY;
        for (uint32_t sp = 0; sp < splits; ++sp) all_m = fmaxf(all_m, split_f[sp]);
        __syncthreads();
        for (uint32_t sp = tid; sp < splits; sp += blockDim.x) split_f[sp] = split_f[sp] == -INFINITY ? 0.0f : expf(split_f[sp] - all_m);
        __syncthreads();
        float all_l = 0.0f;
        for (uint32_t sp = 0; sp < splits; ++sp) all_l = fmaf(split_l[sp], split_f[sp], all_l);      // in split order
        if (a.sinks) all_l += expf(sink - all_m);
        all_l /= gate;
        for (uint32_t c = tid; c < a.vdim; c += blockDim.x) {
            float v = 0.0f;
            uint32_t sp = 0;
            for (; sp + 8 <= splits; sp += 8) {        // eight loads in flight, added in split order
                float x[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) x[u] = __ldcg(parts + (size_t)(sp + u) * pw + 2 + c);
#pragma unroll
                for (int u = 0; u < 8; ++u) v = fmaf(x[u], split_f[sp + u], v);
            }
            for (; sp < splits; ++sp) v = fmaf(__ldcg(parts + (size_t)sp * pw + 2 + c), split_f[sp], v);
            result[c] = v / all_l;
        }
        if (tid == 0) *ticket = 0;
    }
    __syncthreads();
    // the head's sum turns back by its own position
    float* out = reinterpret_cast<float*>(a.out) + ((size_t)t * a.heads + h) * a.vdim;
    const float* vc = a.v_pairs ? reinterpret_cast<const float*>(a.v_cosines) + (size_t)p * a.v_pairs : nullptr;
    const float* vs = a.v_pairs ? reinterpret_cast<const float*>(a.v_sines) + (size_t)p * a.v_pairs : nullptr;
    for (uint32_t i = tid; 2 * i < a.vdim; i += blockDim.x) {
        const uint32_t c0 = 2 * i, c1 = c0 + 1;
        const float x0 = result[c0], x1 = c1 < a.vdim ? result[c1] : 0.0f;
        if (i < a.v_pairs) {
            const float c = vc[i], s = vs[i];
            out[c0] = x0 * c + x1 * s;
            out[c1] = x1 * c - x0 * s;
        } else {
            out[c0] = x0;
            if (c1 < a.vdim) out[c1] = x1;
        }
    }
}

bool encode_window_attention_mma(uzu_command_buffer* cmd, const uzu_window_attention_args& a);     // window_attention_mma.cu

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_window_attention_prepare_encode(uzu_command_buffer* cmd, const uzu_window_attention_prepare_args* a) {
    if (!encodable(cmd, "window_attention_prepare")) return;
    if (!a->q || !a->k || !a->v || !a->query || !a->keys || !a->values || a->heads == 0 || a->kv_heads == 0 || a->dim == 0 || a->vdim == 0 ||
        (a->cache_dt != UZU_DT_BF16 && a->cache_dt != UZU_DT_F32) || 2 * a->rot_pairs > a->dim || 2 * a->v_pairs > a->vdim ||
        (a->rot_pairs && (!a->cosines || !a->sines)) || (a->v_pairs && (!a->v_cosines || !a->v_sines))) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "window_attention_prepare: null operand, bad cache type, or more rotated pairs than channels");
        return;
    }
    if (a->rows == 0) return;
    uzu_window_attention_prepare_args b = *a;
    if (!b.q_stride) b.q_stride = b.heads * b.dim;
    if (!b.k_stride) b.k_stride = b.kv_heads * b.dim;
    if (!b.v_stride) b.v_stride = b.kv_heads * b.vdim;
    const uint32_t items = b.rows * (b.heads + 2 * b.kv_heads);
    if (b.cache_dt == UZU_DT_F32)
        launch(cmd, "window_attention_prepare_kernel", window_attention_prepare_kernel<float>, dim3((items + 3) / 4), dim3(128), 0, b);
    else
        launch(cmd, "window_attention_prepare_kernel", window_attention_prepare_kernel<__nv_bfloat16>, dim3((items + 3) / 4), dim3(128), 0, b);
}

void uzu_window_attention_encode(uzu_command_buffer* cmd, const uzu_window_attention_args* a) {
    if (!encodable(cmd, "window_attention")) return;
    if (!a->query || !a->keys || !a->values || !a->out || a->heads == 0 || a->kv_heads == 0 || a->heads % a->kv_heads || a->dim == 0 || a->vdim == 0 ||
        a->dim > 512 || a->vdim > 512 || (a->cache_dt != UZU_DT_BF16 && a->cache_dt != UZU_DT_F32) || 2 * a->v_pairs > a->vdim ||
        (a->v_pairs && (!a->v_cosines || !a->v_sines))) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "window_attention: null operand, kv_heads not dividing heads, head size outside 1..512, or bad cache type");
        return;
    }
    if (a->rows == 0) return;
    uint32_t splits = std::min<uint32_t>(a->splits ? a->splits : 1, WA_MAX_SPLITS);
    if (splits > 1 && (!a->partials || !a->tickets)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "window_attention: key splits need the partials and tickets scratch");
        return;
    }
    if (splits == 1 && encode_window_attention_mma(cmd, *a)) return;
    const bool f32 = a->cache_dt == UZU_DT_F32;
    // bf16 rows of even head sizes are read two elements per word
    const bool pairs = !f32 && a->dim % 2 == 0 && a->vdim % 2 == 0;
    const uint32_t epw = pairs ? 2 : 1;
    const uint32_t words = (std::max(a->dim, a->vdim) + epw - 1) / epw;
    const uint32_t wpl = (words + 31) / 32;
    const dim3 grid(a->rows, a->heads, splits), block(WA_WARPS * 32);
    const size_t smem = (size_t)(WA_WARPS + 1) * a->vdim * sizeof(float);
    auto go = [&](auto kernel) { launch(cmd, "window_attention_kernel", kernel, grid, block, smem, *a); };
    auto by_wpl = [&](auto tw, auto epw_c) {
        using T = decltype(tw);
        constexpr int E = decltype(epw_c)::value;
        switch (wpl) {
            case 1: go(window_attention_kernel<T, E, 1>); break;
            case 2: go(window_attention_kernel<T, E, 2>); break;
            case 3: case 4: go(window_attention_kernel<T, E, 4>); break;
            case 5: case 6: case 7: case 8: go(window_attention_kernel<T, E, 8>); break;
            default: go(window_attention_kernel<T, E, 16>); break;
        }
    };
    if (f32) by_wpl(float{}, std::integral_constant<int, 1>{});
    else if (pairs) by_wpl(__nv_bfloat16{}, std::integral_constant<int, 2>{});
    else by_wpl(__nv_bfloat16{}, std::integral_constant<int, 1>{});
}

}  // extern "C"
