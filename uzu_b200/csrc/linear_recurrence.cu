// Linear recurrences with an f32 state carried from token to token, `rows` tokens of one sequence per launch (rows = 1 is the decode step).
//
// minGRU (per channel):   S_t = (1 - z_t) S_(t-1) + z_t c_t,  z = sigmoid(.), c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0); out = S_t * silu(gate)
//   The map S -> a S + b of a token composes associatively, so a CTA of (32 channels x CH chunks of rows) first forms every chunk's
//   (product of a, sum from zero), composes them in chunk order (one thread per channel) and then walks every chunk again from its true
//   start state. The gates are f32 from f32 logits; nothing but roundings depends on how a prompt is cut.
//
// Retention (per head, state S [dim, vdim]):   S_t = decay S_(t-1) + (key_scale k_t) v_t^T,  out_t = S_t^T q_t
//   The state update of an element needs no other thread: only the output is a sum over key channels, and it does not feed back. Grid
//   (blocks of 32 value columns, heads); warp p owns PART key channels, lane c one value column, the slice of the state stays in
//   registers. Tokens are taken in batches of RT_BATCH: q and k rows of the batch go to shared memory (requested one batch ahead), every
//   thread runs the batch with no barrier, leaving per-warp partial outputs in shared memory, which are then added in warp order (a
//   fixed order).
#include "common.cuh"

namespace uzu {

namespace {

__device__ __forceinline__ float lr_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

struct GruStep { float a, b; };     // S <- a S + b

__device__ __forceinline__ GruStep gru_step(float z_logit, float u) {
    const float z = lr_sigmoid(z_logit);
    const float c = u >= 0.0f ? u + 0.5f : lr_sigmoid(u);
    return {1.0f - z, z * c};
}

}  // namespace

constexpr int GRU_CHUNKS = 32;

// block (32, chunks): x = channel of the CTA's 32, y = chunk of rows
__global__ void __launch_bounds__(32 * GRU_CHUNKS) min_gru_kernel(const uzu_min_gru_args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float pa[GRU_CHUNKS][32], pb[GRU_CHUNKS][32];
    const uint32_t c = blockIdx.x * 32 + threadIdx.x, chunk = threadIdx.y, chunks = blockDim.y;
    const bool ok = c < a.n;
    const uint32_t per = (a.rows + chunks - 1) / chunks;
    const uint32_t t0 = min(a.rows, chunk * per), t1 = min(a.rows, t0 + per);
    const float* zl = reinterpret_cast<const float*>(a.z_logit) + c;
    const float* u = reinterpret_cast<const float*>(a.u) + c;
    float* state = reinterpret_cast<float*>(a.state);
    float start = (ok && chunk == 0) ? state[c] : 0.0f;
    if (chunks > 1) {
        float A = 1.0f, B = 0.0f;
        if (ok) {
            for (uint32_t t = t0; t < t1; ++t) {
                const GruStep s = gru_step(zl[(size_t)t * a.z_stride], u[(size_t)t * a.u_stride]);
                A *= s.a;
                B = fmaf(s.a, B, s.b);
            }
        }
        pa[chunk][threadIdx.x] = A;
        pb[chunk][threadIdx.x] = B;
        __syncthreads();
        if (chunk == 0) {           // start states of the chunks, in chunk order (pb is overwritten with them)
            float S = start;
            for (uint32_t q = 0; q < chunks; ++q) {
                const float next = fmaf(pa[q][threadIdx.x], S, pb[q][threadIdx.x]);
                pb[q][threadIdx.x] = S;
                S = next;
            }
        }
        __syncthreads();
        start = pb[chunk][threadIdx.x];
    }
    if (!ok) return;
    const float* gate = a.gate ? reinterpret_cast<const float*>(a.gate) + c : nullptr;
    float* out = reinterpret_cast<float*>(a.out) + c;
    float S = start;
    for (uint32_t t = t0; t < t1; ++t) {
        const GruStep s = gru_step(zl[(size_t)t * a.z_stride], u[(size_t)t * a.u_stride]);
        S = fmaf(s.a, S, s.b);
        float o = S;
        if (gate) { const float g = gate[(size_t)t * a.gate_stride]; o *= g * lr_sigmoid(g); }
        out[(size_t)t * a.out_stride] = o;
    }
    if (t1 == a.rows && t0 < t1) state[c] = S;      // the chunk that holds the last row
}

constexpr int RT_BATCH = 16;

template <int PART>
__global__ void __launch_bounds__(PART == 32 ? 1024 : 512) retention_kernel(const uzu_retention_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float rt_smem[];
    const uint32_t dim = a.dim, vdim = a.vdim, head = blockIdx.y;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, parts = blockDim.x >> 5;
    const uint32_t col = blockIdx.x * 32 + lane;
    const bool col_ok = col < vdim;
    float* qs = rt_smem;                                   // [RT_BATCH][dim]
    float* ks = qs + RT_BATCH * dim;                       // [RT_BATCH][dim]
    float* vs = ks + RT_BATCH * dim;                       // [RT_BATCH][32]
    float* part = vs + RT_BATCH * 32;                      // [RT_BATCH][parts][32]
    const uint32_t i0 = warp * PART;
    const uint32_t cnt = i0 < dim ? min((uint32_t)PART, dim - i0) : 0u;
    float* state = reinterpret_cast<float*>(a.state) + (size_t)head * dim * vdim;
    float S[PART];
#pragma unroll
    for (int i = 0; i < PART; ++i) S[i] = ((uint32_t)i < cnt && col_ok) ? state[(size_t)(i0 + i) * vdim + col] : 0.0f;
    const float decay = reinterpret_cast<const float*>(a.decay)[head];
    const float* pq = reinterpret_cast<const float*>(a.q) + (size_t)head * dim;
    const float* pk = reinterpret_cast<const float*>(a.k) + (size_t)head * dim;
    const float* pv = reinterpret_cast<const float*>(a.v) + (size_t)head * vdim;
    float* out = reinterpret_cast<float*>(a.out) + (size_t)head * vdim;
    // A batch's rows are requested one batch ahead into registers (dim <= 32 warps x PART, so a thread stages at most PART / 2 elements
    // of q and of k and one of v), stored to shared memory at the top of the batch: the loads fly during the previous batch's walk.
    constexpr int STAGE = PART / 2 > 1 ? PART / 2 : 1;
    float pre_q[STAGE], pre_k[STAGE], pre_v[4];       // a CTA has at least 4 warps: 4 x 128 covers the batch's 16 x 32 values
    auto request = [&](uint32_t tb) {
        const uint32_t nb = tb < a.rows ? min((uint32_t)RT_BATCH, a.rows - tb) : 0u;
#pragma unroll
        for (int u = 0; u < STAGE; ++u) {
            const uint32_t i = tid + (uint32_t)u * blockDim.x;
            pre_q[u] = pre_k[u] = 0.0f;
            if (i < nb * dim) {
                const uint32_t r = i / dim, ch = i - r * dim;
                pre_q[u] = pq[(size_t)(tb + r) * a.q_stride + ch];
                pre_k[u] = pk[(size_t)(tb + r) * a.k_stride + ch] * a.key_scale;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t i = tid + (uint32_t)u * blockDim.x, r = i >> 5, cc = blockIdx.x * 32 + (i & 31);
            pre_v[u] = (i < nb * 32 && cc < vdim) ? pv[(size_t)(tb + r) * a.v_stride + cc] : 0.0f;
        }
    };
    const bool vec = (dim % 4 == 0) && (PART % 4 == 0);
    request(0);
    for (uint32_t tb = 0; tb < a.rows; tb += RT_BATCH) {
        const uint32_t nb = min((uint32_t)RT_BATCH, a.rows - tb);
#pragma unroll
        for (int u = 0; u < STAGE; ++u) {
            const uint32_t i = tid + (uint32_t)u * blockDim.x;
            if (i < RT_BATCH * dim) { qs[i] = pre_q[u]; ks[i] = pre_k[u]; }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t i = tid + (uint32_t)u * blockDim.x;
            if (i < RT_BATCH * 32) vs[i] = pre_v[u];
        }
        __syncthreads();
        request(tb + RT_BATCH);
        const float* kr = ks + i0;
        const float* qr = qs + i0;
        float* mine = part + warp * 32 + lane;
        if (vec && cnt == PART) {       // the common case: all of the warp's channels exist, 16-byte reads, no predicates
            for (uint32_t r = 0; r < nb; ++r, kr += dim, qr += dim, mine += parts * 32) {
                const float vv = vs[r * 32 + lane];
                float op = 0.0f;
#pragma unroll
                for (int i = 0; i < PART; i += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kr + i), q4 = *reinterpret_cast<const float4*>(qr + i);
                    S[i] = fmaf(k4.x, vv, decay * S[i]);
                    S[i + 1] = fmaf(k4.y, vv, decay * S[i + 1]);
                    S[i + 2] = fmaf(k4.z, vv, decay * S[i + 2]);
                    S[i + 3] = fmaf(k4.w, vv, decay * S[i + 3]);
                    op = fmaf(S[i], q4.x, op);
                    op = fmaf(S[i + 1], q4.y, op);
                    op = fmaf(S[i + 2], q4.z, op);
                    op = fmaf(S[i + 3], q4.w, op);
                }
                *mine = op;
            }
        } else {
            for (uint32_t r = 0; r < nb; ++r, kr += dim, qr += dim, mine += parts * 32) {
                const float vv = vs[r * 32 + lane];
                float op = 0.0f;
#pragma unroll
                for (int i = 0; i < PART; ++i) {
                    if ((uint32_t)i < cnt) {
                        const float s2 = fmaf(kr[i], vv, decay * S[i]);
                        S[i] = s2;
                        op = fmaf(s2, qr[i], op);
                    }
                }
                *mine = op;
            }
        }
        __syncthreads();
        for (uint32_t i = tid; i < nb * 32; i += blockDim.x) {
            const uint32_t r = i >> 5, l = i & 31, cc = blockIdx.x * 32 + l;
            float o = 0.0f;
            for (uint32_t w = 0; w < parts; ++w) o += part[(r * parts + w) * 32 + l];
            if (cc < vdim) out[(size_t)(tb + r) * a.out_stride + cc] = o;
        }
        // the next batch overwrites qs / ks / vs only after every thread has passed the barrier above, and `part` only after the
        // barrier that follows its staging stores
    }
#pragma unroll
    for (int i = 0; i < PART; ++i)
        if ((uint32_t)i < cnt && col_ok) state[(size_t)(i0 + i) * vdim + col] = S[i];
}

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_min_gru_encode(uzu_command_buffer* cmd, const uzu_min_gru_args* a) {
    if (!encodable(cmd, "min_gru")) return;
    if (!a->z_logit || !a->u || !a->state || !a->out || a->n == 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "min_gru: null operand");
        return;
    }
    if (a->rows == 0) return;
    uzu_min_gru_args b = *a;
    if (!b.z_stride) b.z_stride = b.n;
    if (!b.u_stride) b.u_stride = b.n;
    if (!b.gate_stride) b.gate_stride = b.n;
    if (!b.out_stride) b.out_stride = b.n;
    // a chunk holds at least 8 rows: short passes (and the decode step) run as one chunk with no composition
    const uint32_t chunks = std::max(1u, std::min((uint32_t)GRU_CHUNKS, b.rows / 8));
    launch(cmd, "min_gru_kernel", min_gru_kernel, dim3((b.n + 31) / 32), dim3(32, chunks), 0, b);
}

void uzu_retention_encode(uzu_command_buffer* cmd, const uzu_retention_args* a) {
    if (!encodable(cmd, "retention")) return;
    if (!a->q || !a->k || !a->v || !a->decay || !a->state || !a->out || a->dim == 0 || a->dim > 1024 || a->vdim == 0 || a->heads == 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "retention: null operand or key size outside 1..1024");
        return;
    }
    if (a->rows == 0) return;
    uzu_retention_args b = *a;
    if (!b.q_stride) b.q_stride = b.heads * b.dim;
    if (!b.k_stride) b.k_stride = b.heads * b.dim;
    if (!b.v_stride) b.v_stride = b.heads * b.vdim;
    if (!b.out_stride) b.out_stride = b.heads * b.vdim;
    // key channels per warp: about 16 warps per CTA whatever the key size, at most 32 warps
    int part = 4;
    while (part * 16 < (int)b.dim) part *= 2;
    while ((b.dim + part - 1) / part > 32) part *= 2;
    const uint32_t parts = std::max(4u, (b.dim + part - 1) / part);      // at least 4 warps stage a batch (warps past the last key channel only help there)
    const size_t smem = ((size_t)2 * RT_BATCH * b.dim + (size_t)RT_BATCH * 32 + (size_t)RT_BATCH * parts * 32) * sizeof(float);
    const dim3 grid((b.vdim + 31) / 32, b.heads), block(parts * 32);
    // the opt-in is made once per instance and device: for the longest keys the instance serves (32 warps of `part` channels)
    const uint32_t dim_most = std::min(1024u, (uint32_t)part * 32u);
    const size_t smem_most = ((size_t)2 * RT_BATCH * dim_most + (size_t)RT_BATCH * 32 + (size_t)RT_BATCH * 32 * 32) * sizeof(float);
    auto go = [&](auto kernel, std::atomic<uint64_t>& done) {
        opt_in_dynamic_smem(cmd, kernel, (int)smem_most, done);
        launch(cmd, "retention_kernel", kernel, grid, block, smem, b);
    };
    static std::atomic<uint64_t> done[4];
    if (part == 4) go(retention_kernel<4>, done[0]);
    else if (part == 8) go(retention_kernel<8>, done[1]);
    else if (part == 16) go(retention_kernel<16>, done[2]);
    else go(retention_kernel<32>, done[3]);
}

}  // extern "C"
