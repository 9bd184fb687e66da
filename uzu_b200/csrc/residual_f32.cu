// Glue kernels of the parallel-block family (f32 residual stream): grouped RMS norm, norm (RMS or Dynamic Tanh) with residual add and
// the next norm, embedding rows into f32, the token-gated gelu unit, the clamped gated unit, tanh, residual add, logit cap, and the routers (by table or by the largest logits: expert-sorted pair lists + weighted, optionally
// gated combine). Everything is f32 arithmetic.
#include "common.cuh"

namespace uzu {

// one CTA per (row, group); a thread keeps up to 8 of the part's elements in registers between the sum and the scaling
__global__ void __launch_bounds__(256) group_rms_norm_kernel(const uzu_group_rms_norm_args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[32];
    const uint32_t row = blockIdx.x, g = blockIdx.y;
    const uint32_t src = a.row_indices ? reinterpret_cast<const uint32_t*>(a.row_indices)[row] : row;
    const uint32_t part = a.n / a.groups, base = g * part;
    const float* in = reinterpret_cast<const float*>(a.input) + (size_t)src * a.in_stride + base;
    float* out = reinterpret_cast<float*>(a.output) + (size_t)row * a.out_stride + base;
    const float* sc = a.scales ? reinterpret_cast<const float*>(a.scales) + base : nullptr;
    float* out2 = a.output2 ? reinterpret_cast<float*>(a.output2) + (size_t)row * a.out_stride + base : nullptr;
    const float* sc2 = a.scales2 ? reinterpret_cast<const float*>(a.scales2) + base : nullptr;
    constexpr int KEEP = 8;
    float v[KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        v[j] = i < part ? in[i] : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < KEEP; ++j) ss = fmaf(v[j], v[j], ss);
    for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < part; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)part + a.epsilon);
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        if (i < part) {
            out[i] = sc ? v[j] * inv * sc[i] : v[j] * inv;
            if (out2) out2[i] = sc2 ? v[j] * inv * sc2[i] : v[j] * inv;
        }
    }
    for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < part; i += blockDim.x) {
        out[i] = sc ? in[i] * inv * sc[i] : in[i] * inv;
        if (out2) out2[i] = sc2 ? in[i] * inv * sc2[i] : in[i] * inv;
    }
}

// One CTA per row. RMS norm: the row's sum of squares first; Dynamic Tanh is elementwise. With a residual the normed row is added into
// it (times mult) and the updated row can be normed again for the next sublayer; a second RMS norm takes a second sum over the row.
__device__ __forceinline__ float norm_add_value(uint32_t kind, float x, float inv, float alpha, const float* w, const float* b, uint32_t i) {
    float v = kind == 1 ? tanhf(alpha * x) : x * inv;
    if (w) v *= w[i];
    if (b) v += b[i];
    return v;
}

// Dynamic Tanh in and (if any) out: nothing crosses an element, so the work is cut over elements, not rows.
__global__ void __launch_bounds__(256) norm_add_elementwise_kernel(const uzu_norm_add_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t row = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.n) return;
    const float* w = reinterpret_cast<const float*>(a.weight);
    const float* b = reinterpret_cast<const float*>(a.bias);
    const float v = norm_add_value(1, reinterpret_cast<const float*>(a.input)[(size_t)row * a.in_stride + i], 1.0f, a.alpha, w, b, i);
    float* out = a.output ? reinterpret_cast<float*>(a.output) + (size_t)row * a.n : nullptr;
    if (!a.residual) { out[i] = v; return; }
    float* res = reinterpret_cast<float*>(a.residual) + (size_t)row * a.n;
    const float x = fmaf(a.mult, v, res[i]);
    res[i] = x;
    if (out) out[i] = norm_add_value(1, x, 1.0f, a.next_alpha, reinterpret_cast<const float*>(a.next_weight), reinterpret_cast<const float*>(a.next_bias), i);
}

// One CTA per row; a thread keeps up to KEEP of the row's elements (input, weights, residual) in registers, all requested before the
// first sum, so a decode step's single row costs one round trip to memory and not one per pass over the row.
__global__ void __launch_bounds__(256) norm_add_kernel(const uzu_norm_add_args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[32];
    const uint32_t row = blockIdx.x;
    const float* in = reinterpret_cast<const float*>(a.input) + (size_t)row * a.in_stride;
    const float* w = reinterpret_cast<const float*>(a.weight);
    const float* b = reinterpret_cast<const float*>(a.bias);
    const float* nw = reinterpret_cast<const float*>(a.next_weight);
    const float* nb = reinterpret_cast<const float*>(a.next_bias);
    float* res = a.residual ? reinterpret_cast<float*>(a.residual) + (size_t)row * a.n : nullptr;
    float* out = a.output ? reinterpret_cast<float*>(a.output) + (size_t)row * a.n : nullptr;
    constexpr int KEEP = 8;
    float x[KEEP], wv[KEEP], bv[KEEP], rv[KEEP], nwv[KEEP], nbv[KEEP];
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        const bool ok = i < a.n;
        x[j] = ok ? in[i] : 0.0f;
        wv[j] = (ok && w) ? w[i] : 1.0f;
        bv[j] = (ok && b) ? b[i] : 0.0f;
        rv[j] = (ok && res) ? res[i] : 0.0f;
        nwv[j] = (ok && nw) ? nw[i] : 1.0f;
        nbv[j] = (ok && nb) ? nb[i] : 0.0f;
    }
    float inv = 1.0f;
    if (a.kind == 0) {
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < KEEP; ++j) ss = fmaf(x[j], x[j], ss);
        for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < a.n; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
        ss = block_sum(ss, red);
        inv = 1.0f / sqrtf(ss / (float)a.n + a.epsilon);
    }
    // first norm, and the residual add
    float ss2 = 0.0f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        float v = (a.kind == 1 ? tanhf(a.alpha * x[j]) : x[j] * inv) * wv[j] + bv[j];
        if (res) v = fmaf(a.mult, v, rv[j]);
        x[j] = v;
        if (i < a.n) {
            ss2 = fmaf(v, v, ss2);
            if (res) res[i] = v;
            else out[i] = v;
        }
    }
    for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < a.n; i += blockDim.x) {
        float v = norm_add_value(a.kind, in[i], inv, a.alpha, w, b, i);
        if (res) { v = fmaf(a.mult, v, res[i]); res[i] = v; }          // read back below by the thread that wrote it
        else out[i] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (!res || !out) return;
    float inv2 = 1.0f;
    if (a.next_kind == 0) {
        ss2 = block_sum(ss2, red);
        inv2 = 1.0f / sqrtf(ss2 / (float)a.n + a.epsilon);
    }
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        if (i < a.n) out[i] = (a.next_kind == 1 ? tanhf(a.next_alpha * x[j]) : x[j] * inv2) * nwv[j] + nbv[j];
    }
    for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < a.n; i += blockDim.x) out[i] = norm_add_value(a.next_kind, res[i], inv2, a.next_alpha, nw, nb, i);
}

template <typename TW>
__global__ void token_gate_kernel(const uzu_token_gate_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)a.rows * a.n) return;
    const uint32_t r = (uint32_t)(idx / a.n), i = (uint32_t)(idx % a.n);
    const uint32_t tok = reinterpret_cast<const uint32_t*>(a.token_ids)[r];
    float e = 0.0f;
    if (tok < a.vocab) {
        const TW* t = reinterpret_cast<const TW*>(a.table) + (size_t)tok * a.table_stride + a.column + i;
        if constexpr (sizeof(TW) == 2) e = __bfloat162float(*t);
        else e = *t;
    }
    const float z = reinterpret_cast<const float*>(a.z)[idx];
    const float g = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    reinterpret_cast<float*>(a.out)[idx] = g * e;
}

template <typename TW>
__global__ void embedding_f32_kernel(const uint32_t* tokens, const TW* table, float* out, uint32_t vocab, uint32_t n, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t row = blockIdx.y;
    const uint32_t tok = tokens[row];
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = 0.0f;
    if (tok < vocab) {
        if constexpr (sizeof(TW) == 2) v = __bfloat162float(table[(size_t)tok * n + i]);
        else v = table[(size_t)tok * n + i];
    }
    out[(size_t)row * n + i] = v * scale;
}

__global__ void rows_to_bf16_kernel(const float* src, uint32_t src_stride, __nv_bfloat16* dst, uint32_t rows, uint32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * n) return;
    const size_t r = idx / n, c = idx % n;
    dst[idx] = __float2bfloat16_rn(src[r * src_stride + c]);
}

__global__ void clamped_glu_kernel(const float* gate_up, float* out, uint32_t rows, uint32_t f, float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * f) return;
    const size_t r = idx / f, c = idx % f;
    const float g = fminf(gate_up[r * 2 * f + c], limit);
    const float u = fminf(fmaxf(gate_up[r * 2 * f + f + c], -limit), limit);
    out[idx] = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
}

__global__ void silu_glu_kernel(const float* gate_up, float* out, uint32_t rows, uint32_t f) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * f) return;
    const size_t r = idx / f, c = idx % f;
    const float g = gate_up[r * 2 * f + c], u = gate_up[r * 2 * f + f + c];
    out[idx] = g * (1.0f / (1.0f + expf(-g))) * u;
}

__global__ void unary_f32_kernel(const float* in, uint32_t in_stride, float* out, uint32_t out_stride, uint32_t rows, uint32_t n, uint32_t op) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * n) return;
    const size_t r = idx / n, c = idx % n;
    const float v = in[r * in_stride + c];
    out[r * out_stride + c] = op == 0 ? tanhf(v) : v;
}

__global__ void residual_add_kernel(float* x, const float* a, const float* b, uint32_t length) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= length) return;
    float s = a[idx];
    if (b) s += b[idx];
    x[idx] += s;
}

__global__ void logit_cap_f32_kernel(float* logits, __nv_bfloat16* copy, uint32_t length, float cap, uint32_t has_cap) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= length) return;
    float v = logits[idx];
    if (has_cap) {
        v = cap * tanhf(v / cap);
        logits[idx] = v;
    }
    if (copy) copy[idx] = __float2bfloat16_rn(v);
}

// Counting sort of the (row, slot) pairs by expert, by one CTA: `pe` (shared memory) holds the expert of every pair, `counts`
// (shared memory, [experts + 1]) is scratch. Pairs of one expert keep token order, so the lists do not depend on the thread schedule.
__device__ void route_sort_pairs(const uint16_t* pe, uint32_t* counts, uint32_t pairs, uint32_t top, uint32_t experts, uint32_t* offsets,
                                 uint32_t* rows_map, uint32_t* pair_pos) {
    for (uint32_t e = threadIdx.x; e <= experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (uint32_t base = 0; base < pairs; base += blockDim.x) {      // one shared-memory add per (warp, expert): lanes with the same expert elect a leader
        const uint32_t p = base + threadIdx.x;
        const bool valid = p < pairs;
        const uint32_t e = valid ? pe[p] : 0x10000u + (threadIdx.x & 31);
        const uint32_t same = __match_any_sync(0xffffffffu, e);
        if (valid && (threadIdx.x & 31) == (uint32_t)(__ffs(same) - 1)) atomicAdd(&counts[e + 1], (uint32_t)__popc(same));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t e = 0; e < experts; ++e) counts[e + 1] += counts[e];
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = counts[e];
    __syncthreads();
    // Stable placement, counts[e] now being the next free position of expert e: pairs are taken in chunks of one per thread, the warps of
    // a chunk one after the other; within a warp the lanes that hold the same expert are ranked by lane and their leader moves the cursor.
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    // Few experts: every warp of a chunk counts its pairs per expert at once, one thread per expert turns the counts into the warps' start
    // positions (in warp order), then every pair is placed: four barriers per chunk instead of one per warp.
    constexpr uint32_t kFew = 64;
    __shared__ uint32_t warp_start[32][kFew];
    if (experts <= kFew && warps <= 32 && pairs > 32) {        // (a single warp's worth of pairs takes the loop below in one step)
        for (uint32_t base = 0; base < pairs; base += blockDim.x) {
            for (uint32_t i = threadIdx.x; i < 32 * kFew; i += blockDim.x) (&warp_start[0][0])[i] = 0;
            __syncthreads();
            const uint32_t p = base + threadIdx.x;
            const bool valid = p < pairs;
            const uint32_t e = valid ? pe[p] : 0x10000u + lane;
            const uint32_t same = __match_any_sync(0xffffffffu, e);
            const uint32_t rank = __popc(same & ((1u << lane) - 1u));
            if (valid && rank == 0) warp_start[warp][e] = __popc(same);
            __syncthreads();
            if (threadIdx.x < experts) {
                uint32_t cur = counts[threadIdx.x];
                for (uint32_t w = 0; w < warps; ++w) {
                    const uint32_t c = warp_start[w][threadIdx.x];
                    warp_start[w][threadIdx.x] = cur;
                    cur += c;
                }
                counts[threadIdx.x] = cur;
            }
            __syncthreads();
            if (valid) {
                const uint32_t at = warp_start[warp][e] + rank;
                rows_map[at] = p / top;
                pair_pos[p] = at;
            }
            __syncthreads();
        }
        return;
    }
    for (uint32_t base = 0; base < pairs; base += blockDim.x) {
        const uint32_t p = base + threadIdx.x;
        const bool valid = p < pairs;
        const uint32_t e = valid ? pe[p] : 0x10000u + lane;          // idle lanes match nobody
        const uint32_t busy = min(warps, (pairs - base + 31) / 32);
        for (uint32_t w = 0; w < busy; ++w) {
            if (warp == w) {
                const uint32_t same = __match_any_sync(0xffffffffu, e);
                const uint32_t rank = __popc(same & ((1u << lane) - 1u));
                uint32_t at = 0;
                if (valid && rank == 0) {
                    at = counts[e];
                    counts[e] = at + __popc(same);
                }
                at = __shfl_sync(0xffffffffu, at, __ffs(same) - 1);
                if (valid) {
                    rows_map[at + rank] = p / top;
                    pair_pos[p] = at + rank;
                }
            }
            __syncthreads();
        }
    }
}

// One CTA; rows * top <= 1024 * top pairs; experts <= 8192. The experts of a token come from a table row.
__global__ void __launch_bounds__(1024) table_route_kernel(const uzu_table_route_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ uint32_t counts[];   // [experts + 1]
    const uint32_t* tokens = reinterpret_cast<const uint32_t*>(a.token_ids);
    const int32_t* table = reinterpret_cast<const int32_t*>(a.table);
    const uint32_t pairs = a.rows * a.top;
    uint16_t* pe = reinterpret_cast<uint16_t*>(counts + a.experts + 1);   // expert of every pair, staged once
    for (uint32_t p = threadIdx.x; p < pairs; p += blockDim.x) {
        const uint32_t tok = tokens[p / a.top];
        const int32_t e = tok < a.vocab ? table[(size_t)tok * a.top + p % a.top] : 0;
        pe[p] = (uint16_t)((e >= 0 && (uint32_t)e < a.experts) ? (uint32_t)e : 0u);
    }
    __syncthreads();
    route_sort_pairs(pe, counts, pairs, a.top, a.experts, reinterpret_cast<uint32_t*>(a.group_offsets), reinterpret_cast<uint32_t*>(a.rows_map),
                     reinterpret_cast<uint32_t*>(a.pair_pos));
}

// One CTA, a warp per row: `top` rounds, each picking the best (logit, lower index first) that comes after the previous pick in that
// order, so no list of the picked experts is kept. Weights: exp(z - z_first) over the sum of the picked ones, or (weight_kind 1) the
// sigmoid of every picked logit on its own. compact_weight gets the same weights in the expert-sorted order of the pair list.
// MODE 0: choice and pair lists in one CTA (short passes). Long passes with a scratch: MODE 1 makes the choice over many CTAs (a warp per
// row, the picked experts go to the scratch), MODE 2 is the one CTA that sorts them into the pair lists.
template <int MODE>
__global__ void __launch_bounds__(1024) topk_route_kernel(const uzu_topk_route_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ uint32_t counts[];   // [experts + 1]
    const uint32_t pairs = a.rows * a.top;
    uint16_t* pe_shared = reinterpret_cast<uint16_t*>(counts + a.experts + 1);
    uint16_t* pe = MODE == 1 ? reinterpret_cast<uint16_t*>(a.scratch) : pe_shared;
    const float* bias = reinterpret_cast<const float*>(a.bias);
    float* weight = reinterpret_cast<float*>(a.pair_weight);
    const uint32_t lane = threadIdx.x & 31, warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), warps = gridDim.x * (blockDim.x >> 5);
    if constexpr (MODE == 2) {
        const uint16_t* chosen = reinterpret_cast<const uint16_t*>(a.scratch);
        for (uint32_t p = threadIdx.x; p < pairs; p += blockDim.x) pe_shared[p] = chosen[p];
    } else {
    // a lane keeps the logit of expert `lane` of its row in a register for all rounds, and requests the next row's before it works on this one
    auto first_logit = [&](uint32_t r) {
        return (r < a.rows && lane < a.experts) ? reinterpret_cast<const float*>(a.logits)[(size_t)r * a.logits_stride + lane] + (bias ? bias[lane] : 0.0f) : 0.0f;
    };
    float next_z = first_logit(warp);
    for (uint32_t r = warp; r < a.rows; r += warps) {
        const float* z = reinterpret_cast<const float*>(a.logits) + (size_t)r * a.logits_stride;
        const float own_z = next_z;
        next_z = first_logit(r + warps);
        float prev_v = INFINITY, first = 0.0f, sum = 0.0f;
        uint32_t prev_i = 0;
        bool any = false;
        for (uint32_t s = 0; s < a.top; ++s) {
            float best_v = -INFINITY;
            uint32_t best_i = 0xFFFFFFFFu;
            for (uint32_t e = lane; e < a.experts; e += 32) {
                const float v = e == lane ? own_z : z[e] + (bias ? bias[e] : 0.0f);
                const bool after = !any || v < prev_v || (v == prev_v && e > prev_i);
                if (after && (best_i == 0xFFFFFFFFu || v > best_v)) { best_v = v; best_i = e; }    // ascending e: the first of equals stays
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
                const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
                if (oi != 0xFFFFFFFFu && (best_i == 0xFFFFFFFFu || ov > best_v || (ov == best_v && oi < best_i))) { best_v = ov; best_i = oi; }
            }
            if (best_i == 0xFFFFFFFFu) { best_i = 0; best_v = first; }      // fewer usable logits than slots (NaNs): keep the lists well-formed
            if (!any) first = best_v;
            any = true;
            prev_v = best_v; prev_i = best_i;
            const float w = a.weight_kind == 1 ? 1.0f / (1.0f + expf(-best_v)) : expf(best_v - first);
            sum += w;
            if (lane == 0) {
                pe[r * a.top + s] = (uint16_t)best_i;
                weight[r * a.top + s] = w;
            }
        }
        __syncwarp();
        if (lane < a.top && a.weight_kind == 0) {
            for (uint32_t s = lane; s < a.top; s += 32) weight[r * a.top + s] /= sum;
        }
    }
    }
    if constexpr (MODE == 1) return;
    __syncthreads();
    route_sort_pairs(pe_shared, counts, pairs, a.top, a.experts, reinterpret_cast<uint32_t*>(a.group_offsets), reinterpret_cast<uint32_t*>(a.rows_map),
                     reinterpret_cast<uint32_t*>(a.pair_pos));
    if (a.compact_weight) {
        __syncthreads();
        const uint32_t* pos = reinterpret_cast<const uint32_t*>(a.pair_pos);
        float* cw = reinterpret_cast<float*>(a.compact_weight);
        for (uint32_t p = threadIdx.x; p < pairs; p += blockDim.x) cw[pos[p]] = weight[p];
    }
}

__global__ void routed_combine_kernel(const uzu_routed_combine_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)a.rows * a.n) return;
    const size_t r = idx / a.n, c = idx % a.n;
    const float* pairs = reinterpret_cast<const float*>(a.pairs);
    const uint32_t* pair_pos = reinterpret_cast<const uint32_t*>(a.pair_pos);
    const float* pw = reinterpret_cast<const float*>(a.pair_weight);
    float s = 0.0f;
    for (uint32_t k = 0; k < a.top; ++k) {
        const float v = pairs[(size_t)pair_pos[r * a.top + k] * a.n + c];
        s = pw ? fmaf(pw[r * a.top + k], v, s) : s + v;
    }
    s *= a.weight;
    if (a.gate) {
        float g = reinterpret_cast<const float*>(a.gate)[r * a.gate_ld + c];
        if (a.gate_bias) g += reinterpret_cast<const float*>(a.gate_bias)[c];
        s *= 1.0f / (1.0f + expf(-g));
    }
    if (a.col_scale) s *= reinterpret_cast<const float*>(a.col_scale)[c];
    float* out = reinterpret_cast<float*>(a.output);
    out[idx] = a.accumulate ? out[idx] + s : s;
}

static inline unsigned blocks256(size_t n) { return (unsigned)((n + 255) / 256); }

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_group_rms_norm_encode(uzu_command_buffer* cmd, const uzu_group_rms_norm_args* a) {
    if (!encodable(cmd, "group_rms_norm")) return;
    if (!a->input || !a->output || a->groups == 0 || a->n % a->groups != 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "group_rms_norm: null operand or the row is not divisible into the groups");
        return;
    }
    if (a->rows == 0 || a->n == 0) return;
    uzu_group_rms_norm_args b = *a;
    if (!b.in_stride) b.in_stride = b.n;
    if (!b.out_stride) b.out_stride = b.n;
    launch(cmd, "group_rms_norm_kernel", group_rms_norm_kernel, dim3(b.rows, b.groups), dim3(256), 0, b);
}

void uzu_embedding_f32_scaled_encode(uzu_command_buffer* cmd, uint64_t token_ids, uint64_t table, uint32_t weights_dt, uint64_t output, uint32_t rows,
                                     uint32_t vocab, uint32_t n, float scale) {
    if (!encodable(cmd, "embedding_f32") || rows == 0 || n == 0) return;
    dim3 grid(blocks256(n), rows);
    if (weights_dt == UZU_DT_BF16)
        launch(cmd, "embedding_f32_kernel", embedding_f32_kernel<__nv_bfloat16>, grid, dim3(256), 0, (const uint32_t*)token_ids, (const __nv_bfloat16*)table, (float*)output, vocab, n, scale);
    else
        launch(cmd, "embedding_f32_kernel", embedding_f32_kernel<float>, grid, dim3(256), 0, (const uint32_t*)token_ids, (const float*)table, (float*)output, vocab, n, scale);
}

void uzu_embedding_f32_encode(uzu_command_buffer* cmd, uint64_t token_ids, uint64_t table, uint32_t weights_dt, uint64_t output, uint32_t rows,
                              uint32_t vocab, uint32_t n) {
    uzu_embedding_f32_scaled_encode(cmd, token_ids, table, weights_dt, output, rows, vocab, n, 1.0f);
}

void uzu_norm_add_encode(uzu_command_buffer* cmd, const uzu_norm_add_args* a) {
    if (!encodable(cmd, "norm_add")) return;
    if (!a->input || (!a->residual && !a->output) || a->kind > 1 || a->next_kind > 1) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "norm_add: null operand or unknown norm kind");
        return;
    }
    if (a->rows == 0 || a->n == 0) return;
    uzu_norm_add_args b = *a;
    if (!b.in_stride) b.in_stride = b.n;
    if (b.kind == 1 && (!b.residual || !b.output || b.next_kind == 1))
        launch(cmd, "norm_add_elementwise_kernel", norm_add_elementwise_kernel, dim3((b.n + 255) / 256, b.rows), dim3(256), 0, b);
    else
        launch(cmd, "norm_add_kernel", norm_add_kernel, dim3(b.rows), dim3(256), 0, b);
}

void uzu_rows_to_bf16_encode(uzu_command_buffer* cmd, uint64_t src, uint32_t src_stride, uint64_t dst, uint32_t rows, uint32_t n) {
    if (!encodable(cmd, "rows_to_bf16") || rows == 0 || n == 0) return;
    if (!src || !dst || src_stride < n) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "rows_to_bf16: null operand or a row stride below the row size");
        return;
    }
    launch(cmd, "rows_to_bf16_kernel", rows_to_bf16_kernel, dim3(blocks256((size_t)rows * n)), dim3(256), 0, (const float*)src, src_stride, (__nv_bfloat16*)dst, rows, n);
}

void uzu_token_gate_encode(uzu_command_buffer* cmd, const uzu_token_gate_args* a) {
    if (!encodable(cmd, "token_gate")) return;
    if (!a->z || !a->token_ids || !a->table || !a->out || (a->weights_dt != UZU_DT_BF16 && a->weights_dt != UZU_DT_F32) || a->column + a->n > a->table_stride) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "token_gate: null operand, bad table type, or columns outside the table");
        return;
    }
    if (a->rows == 0 || a->n == 0) return;
    const dim3 grid(blocks256((size_t)a->rows * a->n));
    if (a->weights_dt == UZU_DT_BF16) launch(cmd, "token_gate_kernel", token_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, *a);
    else launch(cmd, "token_gate_kernel", token_gate_kernel<float>, grid, dim3(256), 0, *a);
}

void uzu_clamped_glu_encode(uzu_command_buffer* cmd, uint64_t gate_up, uint64_t output, uint32_t rows, uint32_t f, float limit, float alpha) {
    if (!encodable(cmd, "clamped_glu") || rows == 0 || f == 0) return;
    launch(cmd, "clamped_glu_kernel", clamped_glu_kernel, dim3(blocks256((size_t)rows * f)), dim3(256), 0, (const float*)gate_up, (float*)output, rows, f, limit, alpha);
}

void uzu_silu_glu_encode(uzu_command_buffer* cmd, uint64_t gate_up, uint64_t output, uint32_t rows, uint32_t f) {
    if (!encodable(cmd, "silu_glu") || rows == 0 || f == 0) return;
    launch(cmd, "silu_glu_kernel", silu_glu_kernel, dim3(blocks256((size_t)rows * f)), dim3(256), 0, (const float*)gate_up, (float*)output, rows, f);
}

void uzu_unary_f32_encode(uzu_command_buffer* cmd, uint64_t input, uint32_t in_stride, uint64_t output, uint32_t out_stride, uint32_t rows,
                          uint32_t n, uint32_t op) {
    if (!encodable(cmd, "unary_f32") || rows == 0 || n == 0) return;
    launch(cmd, "unary_f32_kernel", unary_f32_kernel, dim3(blocks256((size_t)rows * n)), dim3(256), 0, (const float*)input, in_stride, (float*)output, out_stride, rows, n, op);
}

void uzu_residual_add_encode(uzu_command_buffer* cmd, uint64_t x, uint64_t a, uint64_t b, uint32_t length) {
    if (!encodable(cmd, "residual_add") || length == 0) return;
    launch(cmd, "residual_add_kernel", residual_add_kernel, dim3(blocks256(length)), dim3(256), 0, (float*)x, (const float*)a, (const float*)b, length);
}

void uzu_logit_cap_f32_encode(uzu_command_buffer* cmd, uint64_t logits_f32, uint64_t logits_bf16, uint32_t length, float cap, uint32_t has_cap) {
    if (!encodable(cmd, "logit_cap_f32") || length == 0) return;
    launch(cmd, "logit_cap_f32_kernel", logit_cap_f32_kernel, dim3(blocks256(length)), dim3(256), 0, (float*)logits_f32, (__nv_bfloat16*)logits_bf16, length, cap, has_cap);
}

void uzu_table_route_encode(uzu_command_buffer* cmd, const uzu_table_route_args* a) {
    if (!encodable(cmd, "table_route")) return;
    if (!a->token_ids || !a->table || !a->group_offsets || !a->rows_map || !a->pair_pos || a->top == 0 || a->experts == 0 || a->experts > 8192) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "table_route: null operand or bad expert count");
        return;
    }
    if (a->rows == 0) return;
    const size_t smem = (a->experts + 1) * sizeof(uint32_t) + (size_t)a->rows * a->top * sizeof(uint16_t);
    if (smem > 48 * 1024) {
        cmd->record_error(UZU_ERROR_UNSUPPORTED, "table_route: rows * top too large for one pass");
        return;
    }
    launch(cmd, "table_route_kernel", table_route_kernel, dim3(1), dim3(1024), smem, *a);
}

void uzu_topk_route_encode(uzu_command_buffer* cmd, const uzu_topk_route_args* a) {
    if (!encodable(cmd, "topk_route")) return;
    if (!a->logits || !a->group_offsets || !a->rows_map || !a->pair_pos || !a->pair_weight || a->top == 0 || a->experts == 0 || a->experts > 8192 ||
        a->top > a->experts || a->logits_stride < a->experts) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "topk_route: null operand or bad expert / top count");
        return;
    }
    if (a->rows == 0) return;
    const size_t smem = (a->experts + 1) * sizeof(uint32_t) + (size_t)a->rows * a->top * sizeof(uint16_t);
    if (smem > 48 * 1024) {
        cmd->record_error(UZU_ERROR_UNSUPPORTED, "topk_route: rows * top too large for one pass");
        return;
    }
    if (a->scratch && a->rows >= 64) {          // the choice over many CTAs (8 rows each), then the one CTA that builds the lists
        launch(cmd, "topk_route_kernel", topk_route_kernel<1>, dim3((a->rows + 7) / 8), dim3(256), 0, *a);
        launch(cmd, "topk_route_kernel", topk_route_kernel<2>, dim3(1), dim3(1024), smem, *a);
        return;
    }
    launch(cmd, "topk_route_kernel", topk_route_kernel<0>, dim3(1), dim3(1024), smem, *a);
}

void uzu_routed_combine_gated_encode(uzu_command_buffer* cmd, const uzu_routed_combine_args* a) {
    if (!encodable(cmd, "routed_combine") || a->rows == 0 || a->n == 0) return;
    if (!a->pairs || !a->pair_pos || !a->output || a->top == 0 || (a->gate_bias && !a->gate)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "routed_combine: null operand, or a gate bias without a gate");
        return;
    }
    uzu_routed_combine_args b = *a;
    if (!b.gate_ld) b.gate_ld = b.n;
    launch(cmd, "routed_combine_kernel", routed_combine_kernel, dim3(blocks256((size_t)b.rows * b.n)), dim3(256), 0, b);
}

void uzu_routed_combine_encode(uzu_command_buffer* cmd, uint64_t pairs, uint64_t pair_pos, uint64_t output, uint32_t rows, uint32_t top, uint32_t n,
                               float weight, uint32_t accumulate) {
    uzu_routed_combine_args a{};
    a.pairs = pairs; a.pair_pos = pair_pos; a.output = output; a.rows = rows; a.top = top; a.n = n; a.weight = weight; a.accumulate = accumulate;
    uzu_routed_combine_gated_encode(cmd, &a);
}

}  // extern "C"
