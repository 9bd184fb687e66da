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
//   Gated form (matrix memory with exponential gates): decay and input gain change from token to token and come from exp_gates_kernel,
//   S_t = decay_t S_(t-1) + gain_t k_t v_t^T; the gain is folded into the staged value row. A normaliser n_t = decay_t n_(t-1) + gain_t k_t
//   is the same recurrence with the value 1, so it rides along as one more state column whose output n_t . q_t goes to its own array.
//
// Exponential gates (exp_gates_kernel): a warp per head; the lanes form the log gates of 32 tokens at once, the running maximum
// m_t = max(f_t + m_(t-1), i_t) is chained through the warp token by token (an add and a max each), then every lane forms its token's
// decay exp(f + m_(t-1) - m_t), gain exp(i - m_t) and floor exp(-m_t).
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

__global__ void __launch_bounds__(32) exp_gates_kernel(const uzu_exp_gates_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t head = blockIdx.x, lane = threadIdx.x;
    const float* ip = reinterpret_cast<const float*>(a.i_pre) + head;
    const float* fp = reinterpret_cast<const float*>(a.f_pre) + head;
    float* state = reinterpret_cast<float*>(a.state) + head;
    float* decay = reinterpret_cast<float*>(a.token_decay) + head;
    float* gain = reinterpret_cast<float*>(a.token_gain) + head;
    float* floor_out = a.floor ? reinterpret_cast<float*>(a.floor) + head : nullptr;
    const float inv_cap = a.cap > 0.0f ? 1.0f / a.cap : 0.0f;
    float m = *state;
    for (uint32_t t0 = 0; t0 < a.rows; t0 += 32) {
        const uint32_t t = t0 + lane, nb = min(32u, a.rows - t0);
        float ig = 0.0f, fg = 0.0f;
        if (t < a.rows) {
            ig = ip[(size_t)t * a.i_stride];
            fg = fp[(size_t)t * a.f_stride];
            if (a.cap > 0.0f) { ig = a.cap * tanhf(ig * inv_cap); fg = a.cap * tanhf(fg * inv_cap); }
            fg = fminf(fg, 0.0f) - log1pf(expf(-fabsf(fg)));      // log sigmoid
        }
        float m_before = 0.0f, m_after = 0.0f;
        for (uint32_t j = 0; j < nb; ++j) {
            const float fj = __shfl_sync(0xffffffffu, fg, j), ij = __shfl_sync(0xffffffffu, ig, j);
            const float next = fmaxf(fj + m, ij);
            if (lane == j) { m_before = m; m_after = next; }
            m = next;
        }
        if (t < a.rows) {
            decay[(size_t)t * a.heads] = expf(fg + m_before - m_after);
            gain[(size_t)t * a.heads] = expf(ig - m_after);
            if (floor_out) floor_out[(size_t)t * a.heads] = expf(-m_after);
        }
    }
    if (lane == 0) *state = m;
}

template <int PART, bool GATED>
__global__ void __launch_bounds__(PART == 32 ? 1024 : 512) retention_kernel(const uzu_retention_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float rt_smem[];
    const uint32_t dim = a.dim, vdim = a.vdim, head = blockIdx.y;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, parts = blockDim.x >> 5;
    const uint32_t col = blockIdx.x * 32 + lane;
    const bool with_norm = GATED && a.norm_out != 0;
    const uint32_t vcols = with_norm ? vdim + 1 : vdim;      // the normaliser is one more state column (its value is 1)
    const bool col_ok = col < vcols;
    float* qs = rt_smem;                                   // [RT_BATCH][dim]
    float* ks = qs + RT_BATCH * dim;                       // [RT_BATCH][dim]
    float* vs = ks + RT_BATCH * dim;                       // [RT_BATCH][32]
    float* part = vs + RT_BATCH * 32;                      // [RT_BATCH][parts][32]
    float* ds = part + RT_BATCH * parts * 32;              // [RT_BATCH] the tokens' decays (gated form)
    const uint32_t i0 = warp * PART;
    const uint32_t cnt = i0 < dim ? min((uint32_t)PART, dim - i0) : 0u;
    float* state = reinterpret_cast<float*>(a.state) + (size_t)head * dim * vcols;
    float S[PART];
#pragma unroll
    for (int i = 0; i < PART; ++i) S[i] = ((uint32_t)i < cnt && col_ok) ? state[(size_t)(i0 + i) * vcols + col] : 0.0f;
    const float decay_head = GATED ? 1.0f : reinterpret_cast<const float*>(a.decay)[head];
    const float* tdec = GATED ? reinterpret_cast<const float*>(a.token_decay) + head : nullptr;
    const float* tgain = GATED ? reinterpret_cast<const float*>(a.token_gain) + head : nullptr;
    const float qscale = a.query_scale != 0.0f ? a.query_scale : 1.0f;
    const float* pq = reinterpret_cast<const float*>(a.q) + (size_t)head * dim;
    const float* pk = reinterpret_cast<const float*>(a.k) + (size_t)head * dim;
    const float* pv = reinterpret_cast<const float*>(a.v) + (size_t)head * vdim;
    float* out = reinterpret_cast<float*>(a.out) + (size_t)head * vdim;
    // A batch's rows are requested one batch ahead into registers (dim <= 32 warps x PART, so a thread stages at most PART / 2 elements
    // of q and of k and one of v), stored to shared memory at the top of the batch: the loads fly during the previous batch's walk.
    constexpr int STAGE = PART / 2 > 1 ? PART / 2 : 1;
    float pre_q[STAGE], pre_k[STAGE], pre_v[4];       // a CTA has at least 4 warps: 4 x 128 covers the batch's 16 x 32 values
    float pre_d = 1.0f;
    auto request = [&](uint32_t tb) {
        const uint32_t nb = tb < a.rows ? min((uint32_t)RT_BATCH, a.rows - tb) : 0u;
#pragma unroll
        for (int u = 0; u < STAGE; ++u) {
            const uint32_t i = tid + (uint32_t)u * blockDim.x;
            pre_q[u] = pre_k[u] = 0.0f;
            if (i < nb * dim) {
                const uint32_t r = i / dim, ch = i - r * dim;
                pre_q[u] = pq[(size_t)(tb + r) * a.q_stride + ch] * qscale;
                pre_k[u] = pk[(size_t)(tb + r) * a.k_stride + ch] * a.key_scale;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t i = tid + (uint32_t)u * blockDim.x, r = i >> 5, cc = blockIdx.x * 32 + (i & 31);
            pre_v[u] = (i < nb * 32 && cc < vdim) ? pv[(size_t)(tb + r) * a.v_stride + cc] : 0.0f;
            if constexpr (GATED) {
                if (i < nb * 32) {
                    const float gn = tgain[(size_t)(tb + r) * a.heads];
                    pre_v[u] = cc < vdim ? pre_v[u] * gn : (cc == vdim && with_norm ? gn : 0.0f);
                }
            }
        }
        if constexpr (GATED) pre_d = tid < nb ? tdec[(size_t)(tb + tid) * a.heads] : 1.0f;
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
        if constexpr (GATED) { if (tid < RT_BATCH) ds[tid] = pre_d; }
        __syncthreads();
        request(tb + RT_BATCH);
        const float* kr = ks + i0;
        const float* qr = qs + i0;
        float* mine = part + warp * 32 + lane;
        if (vec && cnt == PART) {       // the common case: all of the warp's channels exist, 16-byte reads, no predicates
            for (uint32_t r = 0; r < nb; ++r, kr += dim, qr += dim, mine += parts * 32) {
                const float vv = vs[r * 32 + lane];
                const float decay = GATED ? ds[r] : decay_head;
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
                const float decay = GATED ? ds[r] : decay_head;
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
            else if (with_norm && cc == vdim) reinterpret_cast<float*>(a.norm_out)[(size_t)(tb + r) * a.heads + head] = o;
        }
        // the next batch overwrites qs / ks / vs only after every thread has passed the barrier above, and `part` only after the
        // barrier that follows its staging stores
    }
#pragma unroll
    for (int i = 0; i < PART; ++i)
        if ((uint32_t)i < cnt && col_ok) state[(size_t)(i0 + i) * vcols + col] = S[i];
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
    const bool gated = a->token_decay != 0;
    if (!a->q || !a->k || !a->v || (!gated && !a->decay) || (gated && !a->token_gain) || (!gated && a->norm_out) || !a->state || !a->out || a->dim == 0 ||
        a->dim > 1024 || a->vdim == 0 || a->heads == 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "retention: null operand, per-token factors without their pair, or key size outside 1..1024");
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
    const size_t smem = ((size_t)2 * RT_BATCH * b.dim + (size_t)RT_BATCH * 32 + (size_t)RT_BATCH * parts * 32 + RT_BATCH) * sizeof(float);
    const uint32_t vcols = b.norm_out ? b.vdim + 1 : b.vdim;
    const dim3 grid((vcols + 31) / 32, b.heads), block(parts * 32);
    // the opt-in is made once per instance and device: for the longest keys the instance serves (32 warps of `part` channels)
    const uint32_t dim_most = std::min(1024u, (uint32_t)part * 32u);
    const size_t smem_most = ((size_t)2 * RT_BATCH * dim_most + (size_t)RT_BATCH * 32 + (size_t)RT_BATCH * 32 * 32 + RT_BATCH) * sizeof(float);
    auto go = [&](auto kernel, std::atomic<uint64_t>& done) {
        opt_in_dynamic_smem(cmd, kernel, (int)smem_most, done);
        launch(cmd, "retention_kernel", kernel, grid, block, smem, b);
    };
    static std::atomic<uint64_t> done[8];
    if (gated) {
        if (part == 4) go(retention_kernel<4, true>, done[4]);
        else if (part == 8) go(retention_kernel<8, true>, done[5]);
        else if (part == 16) go(retention_kernel<16, true>, done[6]);
        else go(retention_kernel<32, true>, done[7]);
        return;
    }
    if (part == 4) go(retention_kernel<4, false>, done[0]);
    else if (part == 8) go(retention_kernel<8, false>, done[1]);
    else if (part == 16) go(retention_kernel<16, false>, done[2]);
    else go(retention_kernel<32, false>, done[3]);
}

void uzu_exp_gates_encode(uzu_command_buffer* cmd, const uzu_exp_gates_args* a) {
    if (!encodable(cmd, "exp_gates")) return;
    if (!a->i_pre || !a->f_pre || !a->state || !a->token_decay || !a->token_gain || a->heads == 0 || a->cap < 0.0f) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "exp_gates: null operand or negative cap");
        return;
    }
    if (a->rows == 0) return;
    uzu_exp_gates_args b = *a;
    if (!b.i_stride) b.i_stride = b.heads;
    if (!b.f_stride) b.f_stride = b.heads;
    launch(cmd, "exp_gates_kernel", exp_gates_kernel, dim3(b.heads), dim3(32), 0, b);
}

}  // extern "C"
