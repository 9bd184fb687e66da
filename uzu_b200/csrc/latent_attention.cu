// Latent attention: every head scores against ONE cached row per token, [normed latent c (rank) | rotated shared key part (rot_dim)],
// and sums the latent part of the rows; the per-head key / value up-projections are folded into the query (absorbed key projection)
// and applied after the weighted sum (value projection), both as z-batched dense linears outside these kernels.
//   prepare: per token the cache row (RMS norm of the latent, interleaved-pair rotation of the shared key part) and the rotated part of
//            every head's query;
//   attend:  one CTA per (query token, group of 8 heads, split of the keys): a tile of 32 cache rows is staged once in shared memory as
//            f32 and used by all heads of the group (warp = head, lane = key for the scores, lane = latent channel for the weighted
//            sum); running maximum / normaliser / accumulator in f32 registers (online softmax), causal bound = the query's own
//            position. A pass of few query rows (decode) splits the keys over many CTAs and a second kernel merges the partial
//            softmax states; a prompt's rows fill the GPU by themselves and write their output directly. Options: a sliding window
//            (only the last `window` positions are visible), a sink per head (one more term exp(sink) in the denominator, with no
//            key and no value), a gate per head (the head's sum times sigmoid(gate)).
// The cache holds bf16 or f32 rows; scores, weights and sums are f32.
#include "common.cuh"

namespace uzu {

template <typename T>
__device__ __forceinline__ void cache_store(T* p, float v);
template <>
__device__ __forceinline__ void cache_store<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void cache_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float cache_load(const float* p) { return *p; }
__device__ __forceinline__ float cache_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const uzu_latent_prepare_args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[32];
    const uint32_t t = blockIdx.x, unit = blockIdx.y;        // unit 0: the cache row; unit 1 + h: the rotated part of head h's query; the last unit: the query latent's norm
    if (a.q_latent && unit == gridDim.y - 1) {
        const float* x = reinterpret_cast<const float*>(a.q_latent) + (size_t)t * a.q_latent_stride;
        float* out = reinterpret_cast<float*>(a.q_latent_out) + (size_t)t * a.q_rank;
        const float* sc = reinterpret_cast<const float*>(a.q_latent_scales);
        constexpr int KEEP = 8;        // the row's elements and weights are requested at once and stay in registers between the sum and the scaling
        float v[KEEP], w[KEEP];
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            v[j] = i < a.q_rank ? x[i] : 0.0f;
            w[j] = (i < a.q_rank && sc) ? sc[i] : 1.0f;
        }
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < KEEP; ++j) ss = fmaf(v[j], v[j], ss);
        for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < a.q_rank; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.q_rank + a.epsilon);
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            if (i < a.q_rank) out[i] = v[j] * inv * w[j];
        }
        for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < a.q_rank; i += blockDim.x) out[i] = x[i] * inv * (sc ? sc[i] : 1.0f);
        return;
    }
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t pos = prefix + t;
    const uint32_t width = a.rank + a.rot_dim;
    const float* cosr = reinterpret_cast<const float*>(a.cosines) + (size_t)pos * a.rot_pairs;
    const float* sinr = reinterpret_cast<const float*>(a.sines) + (size_t)pos * a.rot_pairs;
    if (unit == 0) {
        if (!a.kv) return;
        const float* kv = reinterpret_cast<const float*>(a.kv) + (size_t)t * a.kv_stride;
        T* row = reinterpret_cast<T*>(a.cache) + (size_t)pos * width;
        const float* sc = reinterpret_cast<const float*>(a.latent_scales);
        float v[4], w[4];              // rank <= 512 = 4 x 128 threads: the latent and its weights are requested at once
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            v[j] = i < a.rank ? kv[i] : 0.0f;
            w[j] = (i < a.rank && sc) ? sc[i] : 1.0f;
        }
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) ss = fmaf(v[j], v[j], ss);
        for (uint32_t i = threadIdx.x + 4 * blockDim.x; i < a.rank; i += blockDim.x) ss = fmaf(kv[i], kv[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.rank + a.epsilon);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            if (i < a.rank) cache_store<T>(row + i, v[j] * inv * w[j]);
        }
        for (uint32_t i = threadIdx.x + 4 * blockDim.x; i < a.rank; i += blockDim.x) cache_store<T>(row + i, kv[i] * inv * (sc ? sc[i] : 1.0f));
        for (uint32_t i = threadIdx.x; i < a.rot_pairs; i += blockDim.x) {
            const float x0 = kv[a.rank + 2 * i], x1 = kv[a.rank + 2 * i + 1], c = cosr[i], s = sinr[i];
            cache_store<T>(row + a.rank + 2 * i, x0 * c - x1 * s);
            cache_store<T>(row + a.rank + 2 * i + 1, x1 * c + x0 * s);
        }
        for (uint32_t i = 2 * a.rot_pairs + threadIdx.x; i < a.rot_dim; i += blockDim.x) cache_store<T>(row + a.rank + i, kv[a.rank + i]);
        return;
    }
    if (!a.q) return;
    const uint32_t h = unit - 1;
    const float* src = reinterpret_cast<const float*>(a.q) + (size_t)t * a.q_stride + (size_t)h * (a.dim + a.rot_dim) + a.dim;
    float* out = reinterpret_cast<float*>(a.query) + ((size_t)t * a.heads + h) * width + a.rank;
    for (uint32_t i = threadIdx.x; i < a.rot_pairs; i += blockDim.x) {
        const float x0 = src[2 * i], x1 = src[2 * i + 1], c = cosr[i], s = sinr[i];
        out[2 * i] = x0 * c - x1 * s;
        out[2 * i + 1] = x1 * c + x0 * s;
    }
    for (uint32_t i = 2 * a.rot_pairs + threadIdx.x; i < a.rot_dim; i += blockDim.x) out[i] = src[i];
}

constexpr int LA_HEADS = 8, LA_KEYS = 32;

// words of 4 bytes: one f32 element or two bf16 elements
__device__ __forceinline__ void word_to_f32(const float* p, float* dst) { dst[0] = *p; }
__device__ __forceinline__ void word_to_f32(const __nv_bfloat16* p, float* dst) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(p);
    dst[0] = __uint_as_float(u << 16);
    dst[1] = __uint_as_float(u & 0xffff0000u);
}

// grid (query rows, head groups, key splits). Split s of a query covers the key tiles [s * per, (s + 1) * per) of its causal range; with
// more than one split every CTA leaves (max, normaliser, unnormalised sum) in `partials` and latent_combine_kernel merges them.
template <typename T, int RV>
__global__ void __launch_bounds__(LA_HEADS * 32) latent_attention_kernel(const uzu_latent_attention_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float la_smem[];
    const uint32_t t = blockIdx.x, h0 = blockIdx.y * LA_HEADS, split = blockIdx.z, splits = gridDim.z;
    const uint32_t width = a.rank + a.rot_dim;
    float* qs = la_smem;                       // [LA_HEADS][width]
    float* tile = qs + LA_HEADS * width + ((4 - (LA_HEADS * width) % 4) % 4);   // [LA_KEYS][width], 16-byte aligned
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t keys = prefix + t + 1;      // causal: positions 0 .. own
    const uint32_t lo = (a.window && keys > a.window) ? keys - a.window : 0u;      // first visible key of a sliding window
    // tiles keep their absolute places (a tile starts at a multiple of LA_KEYS, so the flat copy below stays aligned); the keys of the
    // first tile that lie before the window are masked
    const uint32_t tile0 = lo / LA_KEYS;
    const uint32_t tiles = (keys + LA_KEYS - 1) / LA_KEYS - tile0, per = (tiles + splits - 1) / splits;
    const uint32_t j_begin = min(keys, (tile0 + split * per) * LA_KEYS), j_end = min(keys, (tile0 + (split + 1) * per) * LA_KEYS);
    const uint32_t head = h0 + warp;
    const bool head_ok = head < a.heads;
    const float* q = reinterpret_cast<const float*>(a.query) + ((size_t)t * a.heads + h0) * width;
    const uint32_t group_heads = min((uint32_t)LA_HEADS, a.heads - h0);
    if (width % 4 == 0 && (a.query & 15) == 0) {
        for (uint32_t i = tid; i < group_heads * width / 4; i += blockDim.x) reinterpret_cast<float4*>(qs)[i] = reinterpret_cast<const float4*>(q)[i];
    } else {
        for (uint32_t i = tid; i < group_heads * width; i += blockDim.x) qs[i] = q[i];
    }
    const T* cache = reinterpret_cast<const T*>(a.cache);
    // the rows of a tile are contiguous in the cache: one flat copy in 16-byte pieces when the tile's first byte is 16-byte aligned
    constexpr uint32_t EPV = 16 / sizeof(T);   // elements per piece
    const bool vec_ok = ((a.cache & 15) == 0) && (((size_t)LA_KEYS * width * sizeof(T)) % 16 == 0);
    float m = -INFINITY, l = 0.0f, acc[RV];
#pragma unroll
    for (int i = 0; i < RV; ++i) acc[i] = 0.0f;
    const float* myq = qs + warp * width;
    for (uint32_t j0 = j_begin; j0 < j_end; j0 += LA_KEYS) {
        const uint32_t n = min((uint32_t)LA_KEYS, j_end - j0);
        __syncthreads();   // the previous tile is consumed (and, the first time, the queries are staged)
        const T* src = cache + (size_t)j0 * width;
        const uint32_t total = n * width, pieces = vec_ok ? total / EPV : 0;
        for (uint32_t v0 = tid; v0 < pieces; v0 += 4 * blockDim.x) {      // four pieces of a thread in flight
            uint4 raw[4];
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
                const uint32_t v = v0 + u * blockDim.x;
                if (v < pieces) raw[u] = *reinterpret_cast<const uint4*>(src + (size_t)v * EPV);
            }
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
                const uint32_t v = v0 + u * blockDim.x;
                if (v >= pieces) break;
                float* dst = tile + (size_t)v * EPV;
                if constexpr (sizeof(T) == 2) {
                    *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(raw[u].x << 16), __uint_as_float(raw[u].x & 0xffff0000u),
                                                                  __uint_as_float(raw[u].y << 16), __uint_as_float(raw[u].y & 0xffff0000u));
                    *reinterpret_cast<float4*>(dst + 4) = make_float4(__uint_as_float(raw[u].z << 16), __uint_as_float(raw[u].z & 0xffff0000u),
                                                                      __uint_as_float(raw[u].w << 16), __uint_as_float(raw[u].w & 0xffff0000u));
                } else {
                    *reinterpret_cast<uint4*>(dst) = raw[u];
                }
            }
        }
        for (uint32_t i = pieces * EPV + tid; i < total; i += blockDim.x) tile[i] = cache_load(src + i);
        __syncthreads();
        if (!head_ok) continue;
        float s = -INFINITY;
        if (width % 4 == 0) {
            // the warp takes the keys one after the other: every lane multiplies its 16-byte pieces of the query and of the row, the
            // warp adds the 32 partial sums, lane k keeps the score of key k
            const float4* q4 = reinterpret_cast<const float4*>(myq);
            const uint32_t w4 = width / 4;
            // four keys per pass: a query piece is read once for the four rows and the four warp sums overlap
            for (uint32_t k = 0; k < n; k += 4) {
                const float4* r0 = reinterpret_cast<const float4*>(tile + (size_t)k * width);
                const float4* r1 = reinterpret_cast<const float4*>(tile + (size_t)min(k + 1, n - 1) * width);
                const float4* r2 = reinterpret_cast<const float4*>(tile + (size_t)min(k + 2, n - 1) * width);
                const float4* r3 = reinterpret_cast<const float4*>(tile + (size_t)min(k + 3, n - 1) * width);
                float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
                for (uint32_t c = lane; c < w4; c += 32) {
                    const float4 x = q4[c], y0 = r0[c], y1 = r1[c], y2 = r2[c], y3 = r3[c];
                    d0 = fmaf(x.x, y0.x, d0); d0 = fmaf(x.y, y0.y, d0); d0 = fmaf(x.z, y0.z, d0); d0 = fmaf(x.w, y0.w, d0);
                    d1 = fmaf(x.x, y1.x, d1); d1 = fmaf(x.y, y1.y, d1); d1 = fmaf(x.z, y1.z, d1); d1 = fmaf(x.w, y1.w, d1);
                    d2 = fmaf(x.x, y2.x, d2); d2 = fmaf(x.y, y2.y, d2); d2 = fmaf(x.z, y2.z, d2); d2 = fmaf(x.w, y2.w, d2);
                    d3 = fmaf(x.x, y3.x, d3); d3 = fmaf(x.y, y3.y, d3); d3 = fmaf(x.z, y3.z, d3); d3 = fmaf(x.w, y3.w, d3);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    d0 += __shfl_xor_sync(0xffffffffu, d0, o);
                    d1 += __shfl_xor_sync(0xffffffffu, d1, o);
                    d2 += __shfl_xor_sync(0xffffffffu, d2, o);
                    d3 += __shfl_xor_sync(0xffffffffu, d3, o);
                }
                if (lane == k) s = d0 * a.scale;
                if (lane == k + 1 && k + 1 < n) s = d1 * a.scale;
                if (lane == k + 2 && k + 2 < n) s = d2 * a.scale;
                if (lane == k + 3 && k + 3 < n) s = d3 * a.scale;
            }
        } else if (lane < n) {
            // lane = key. Rows are `width` apart, so the lanes start `lane` channels into the dot product and wrap around: in every step
            // the 32 lanes read 32 consecutive query entries and one entry each of 32 rows.
            const float* kr = tile + lane * width;
            float d0 = 0.0f;
            uint32_t c = lane % width;
            for (uint32_t i = 0; i < width; ++i) {
                d0 = fmaf(myq[c], kr[c], d0);
                c = c + 1 == width ? 0 : c + 1;
            }
            s = d0 * a.scale;
        }
        if (j0 + lane < lo) s = -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (lane < n && s != -INFINITY) ? expf(s - m_new) : 0.0f;
        const float corr = m == -INFINITY ? 0.0f : expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < RV; ++i) acc[i] *= corr;
        for (uint32_t k = 0; k < n; ++k) {
            const float pk = __shfl_sync(0xffffffffu, p, k);
            const float* vr = tile + k * width;
#pragma unroll
            for (int i = 0; i < RV; ++i) {
                const uint32_t c = lane + 32 * i;
                if (c < a.rank) acc[i] = fmaf(pk, vr[c], acc[i]);
            }
        }
    }
    if (!head_ok) return;
    if (splits == 1) {
        float* out = reinterpret_cast<float*>(a.out) + ((size_t)t * a.heads + head) * a.rank;
        float inv = 1.0f / (a.sinks ? l + expf(reinterpret_cast<const float*>(a.sinks)[head] - m) : l);
        if (a.head_gate) inv *= 1.0f / (1.0f + expf(-reinterpret_cast<const float*>(a.head_gate)[(size_t)t * a.head_gate_stride + head]));
#pragma unroll
        for (int i = 0; i < RV; ++i) {
            const uint32_t c = lane + 32 * i;
            if (c < a.rank) out[c] = acc[i] * inv;
        }
        return;
    }
    float* part = reinterpret_cast<float*>(a.partials) + (((size_t)t * a.heads + head) * splits + split) * (a.rank + 2);
    if (lane == 0) {
        part[0] = m;
        part[1] = l;
    }
#pragma unroll
    for (int i = 0; i < RV; ++i) {
        const uint32_t c = lane + 32 * i;
        if (c < a.rank) part[2 + c] = acc[i];
    }
}

// grid (query row x head, blocks of 128 channels): out = sum_s e^(m_s - M) acc_s / sum_s e^(m_s - M) l_s, splits taken in order.
// splits <= 64: warp 0 forms the weights of all splits at once, then every thread sums its channel with the loads of a split batch in flight.
// A sink adds exp(sink - M) to the denominator; a head gate multiplies the result by its sigmoid.
__global__ void __launch_bounds__(128) latent_combine_kernel(const float* partials, float* out, uint32_t splits, uint32_t rank, uint32_t heads,
                                                             const float* sinks, const float* head_gate, uint32_t head_gate_stride) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float weight[64];
    __shared__ float inv_total;
    const float* part = partials + (size_t)blockIdx.x * splits * (rank + 2);
    if (threadIdx.x < 32) {
        const uint32_t lane = threadIdx.x;
        const float m0 = lane < splits ? part[(size_t)lane * (rank + 2)] : -INFINITY;
        const float m1 = lane + 32 < splits ? part[(size_t)(lane + 32) * (rank + 2)] : -INFINITY;
        const float l0 = lane < splits ? part[(size_t)lane * (rank + 2) + 1] : 0.0f;
        const float l1 = lane + 32 < splits ? part[(size_t)(lane + 32) * (rank + 2) + 1] : 0.0f;
        const float big = warp_max(fmaxf(m0, m1));
        const float w0 = m0 == -INFINITY ? 0.0f : expf(m0 - big), w1 = m1 == -INFINITY ? 0.0f : expf(m1 - big);
        weight[lane] = w0;
        weight[lane + 32] = w1;
        float total = warp_sum(w0 * l0) + warp_sum(w1 * l1);
        const uint32_t row = blockIdx.x / heads, head = blockIdx.x % heads;
        if (sinks) total += expf(sinks[head] - big);
        float inv = 1.0f / total;
        if (head_gate) inv *= 1.0f / (1.0f + expf(-head_gate[(size_t)row * head_gate_stride + head]));
        if (lane == 0) inv_total = inv;
    }
    __syncthreads();
    const uint32_t c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= rank) return;
    float v = 0.0f;
    uint32_t s = 0;
    for (; s + 8 <= splits; s += 8) {          // eight splits' loads in flight, added in split order
        float x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) x[u] = part[(size_t)(s + u) * (rank + 2) + 2 + c];
#pragma unroll
        for (int u = 0; u < 8; ++u) v = fmaf(weight[s + u], x[u], v);
    }
    for (; s < splits; ++s) v = fmaf(weight[s], part[(size_t)s * (rank + 2) + 2 + c], v);
    out[(size_t)blockIdx.x * rank + c] = v * inv_total;
}

template <typename T, int RV>
static void launch_latent_attention(uzu_command_buffer* cmd, const uzu_latent_attention_args& a) {
    const uint32_t width = a.rank + a.rot_dim;
    const size_t smem = ((size_t)LA_HEADS * width + 4 + (size_t)LA_KEYS * width) * sizeof(float);
    static std::atomic<uint64_t> done{0};
    // the opt-in is made once per instance and device, so it asks for the widest row the entry point accepts (models of different row
    // widths may share an instance in one process)
    if (smem > 48 * 1024) opt_in_dynamic_smem(cmd, latent_attention_kernel<T, RV>, 201 * 1024, done);
    const uint32_t splits = (a.splits > 1 && a.partials) ? std::min(a.splits, 64u) : 1;
    dim3 grid(a.rows, (a.heads + LA_HEADS - 1) / LA_HEADS, splits);
    launch(cmd, "latent_attention_kernel", latent_attention_kernel<T, RV>, grid, dim3(LA_HEADS * 32), smem, a);
    if (splits > 1) {
        launch(cmd, "latent_combine_kernel", latent_combine_kernel, dim3(a.rows * a.heads, (a.rank + 127) / 128), dim3(128), 0, (const float*)a.partials, (float*)a.out,
               splits, a.rank, a.heads, (const float*)a.sinks, (const float*)a.head_gate, a.head_gate_stride);
    }
}

template <typename T>
static void dispatch_latent_attention(uzu_command_buffer* cmd, const uzu_latent_attention_args& a) {
    const uint32_t rv = (a.rank + 31) / 32;
    if (rv <= 2) launch_latent_attention<T, 2>(cmd, a);
    else if (rv <= 4) launch_latent_attention<T, 4>(cmd, a);
    else if (rv <= 8) launch_latent_attention<T, 8>(cmd, a);
    else launch_latent_attention<T, 16>(cmd, a);
}

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_latent_prepare_encode(uzu_command_buffer* cmd, const uzu_latent_prepare_args* a) {
    if (!encodable(cmd, "latent_prepare")) return;
    if ((!a->kv && !a->q && !a->q_latent) || (a->q_latent && (!a->q_latent_out || !a->q_rank)) || (a->kv && !a->cache) || (a->q && !a->query) || (a->rot_pairs && (!a->cosines || !a->sines)) || 2 * a->rot_pairs > a->rot_dim ||
        (a->cache_dt != UZU_DT_BF16 && a->cache_dt != UZU_DT_F32)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "latent_prepare: inconsistent arguments");
        return;
    }
    if (a->rows == 0) return;
    uzu_latent_prepare_args b = *a;
    if (!b.q_latent_stride) b.q_latent_stride = b.q_rank;
    const dim3 grid(b.rows, 1 + (b.q ? b.heads : 0) + (b.q_latent ? 1 : 0));      // without rotated query parts the heads' units are not launched
    if (b.cache_dt == UZU_DT_BF16) launch(cmd, "latent_prepare_kernel", latent_prepare_kernel<__nv_bfloat16>, grid, dim3(128), 0, b);
    else launch(cmd, "latent_prepare_kernel", latent_prepare_kernel<float>, grid, dim3(128), 0, b);
}

void uzu_latent_attention_encode(uzu_command_buffer* cmd, const uzu_latent_attention_args* a) {
    if (!encodable(cmd, "latent_attention")) return;
    if (!a->query || !a->cache || !a->out || a->heads == 0 || a->rank == 0 || a->rank > 512 || (a->cache_dt != UZU_DT_BF16 && a->cache_dt != UZU_DT_F32)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "latent_attention: null operand, or latent size outside 1..512");
        return;
    }
    if ((size_t)(LA_HEADS * (a->rank + a->rot_dim) + LA_KEYS * (a->rank + a->rot_dim + 1)) * 4 > 200 * 1024) {
        cmd->record_error(UZU_ERROR_UNSUPPORTED, "latent_attention: cache row too wide for the shared-memory tile");
        return;
    }
    if (a->rows == 0) return;
    if (a->cache_dt == UZU_DT_BF16) dispatch_latent_attention<__nv_bfloat16>(cmd, *a);
    else dispatch_latent_attention<float>(cmd, *a);
}

}  // extern "C"
