// Generalized delta rule (per head a dim x dim f32 state S, key channel x value channel):
//     S <- diag(d) S - (a * u)(u^T S) + k v^T,   out = S^T r
// with decay d = exp(-e^-1/2 * sigmoid(.)), removal rate a = sigmoid(.), unit key u = k / sqrt(sum k^2 + 1e-6), all formed in f32 here
// from the raw projections. One launch walks the `rows` tokens of a pass in order with the state on chip: the value columns of a head are
// independent (u^T S is a per-column dot product), so the grid is (column blocks of 32, heads) and a CTA keeps its dim x 32 slice of
// the state in registers -- warp p owns PART key channels [PART p, PART p + PART), lane c owns column c (PART is chosen per head size
// so that a CTA has about 16 warps). Per token the CTA puts the head's vectors in shared memory, every thread contributes a partial
// of u^T S and of S^T r, and partials meet in shared memory in warp order (a fixed order: one token at a time or a thousand in one
// launch give the same bits). A token's inputs are requested three tokens ahead. Passes of >= 4 tokens that bring a scratch form decay,
// rate * unit key and unit key for all tokens in one parallel launch first (general_delta_prepare_kernel), which takes the exponentials
// and the key norm out of the token-by-token chain. The same kernel is the decode step (rows = 1).
#include <cstdlib>

#include "common.cuh"

namespace uzu {


// PREP: decay, rate * unit key and unit key arrive ready-made (general_delta_prepare_kernel) in decay_logit, rate_logit and `unit`.
template <bool PREP, int PART>
__global__ void __launch_bounds__(1024) general_delta_kernel(const uzu_general_delta_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float gd_smem[];
    const uint32_t dim = a.dim, head = blockIdx.y;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, parts = blockDim.x >> 5;
    const uint32_t col = blockIdx.x * 32 + lane;
    const bool col_ok = col < dim;
    // shared memory: 2 x { d, au, u, k, r : dim each } + 2 x zpart[parts][32] + 2 x opart[parts][32] + 2 x ssq[32]
    float* vec = gd_smem;                                  // [2][5][dim]
    float* zpart = vec + 2 * 5 * dim;                      // [2][parts][32]
    float* opart = zpart + 2 * parts * 32;                 // [2][parts][32]
    float* ssq = opart + 2 * parts * 32;                   // [2][32]
    const uint32_t i0 = warp * PART;
    const uint32_t cnt = i0 < dim ? min((uint32_t)PART, dim - i0) : 0u;
    float* state = reinterpret_cast<float*>(a.state) + (size_t)head * dim * dim;
    float S[PART];
#pragma unroll
    for (int i = 0; i < PART; ++i) S[i] = ((uint32_t)i < cnt && col_ok) ? state[(size_t)(i0 + i) * dim + col] : 0.0f;

    const float* pr = reinterpret_cast<const float*>(a.r);
    const float* pk = reinterpret_cast<const float*>(a.k);
    const float* pv = reinterpret_cast<const float*>(a.v);
    const float* pa = reinterpret_cast<const float*>(a.rate_logit);
    const float* pd = reinterpret_cast<const float*>(a.decay_logit);
    const uint32_t hc = head * dim;
    const bool prep = tid < dim;
    const float rate_b = (prep && a.rate_bias) ? reinterpret_cast<const float*>(a.rate_bias)[hc + tid] : 0.0f;
    const float decay_b = (prep && a.decay_bias) ? reinterpret_cast<const float*>(a.decay_bias)[hc + tid] : 0.0f;
    const float* pu = reinterpret_cast<const float*>(a.unit);
    // a token's inputs are requested three tokens ahead: the token-by-token chain never waits for memory
    struct Inputs { float k, r, a, d, u, v; };
    auto request = [&](uint32_t t) {
        Inputs q{0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        if (t < a.rows) {
            if (prep) {
                q.k = pk[(size_t)t * a.k_stride + hc + tid];
                q.r = pr[(size_t)t * a.r_stride + hc + tid];
                q.a = pa[(size_t)t * a.rate_stride + hc + tid];
                q.d = pd[(size_t)t * a.decay_stride + hc + tid];
                if constexpr (PREP) q.u = pu[(size_t)t * a.heads * dim + hc + tid];
            }
            if (col_ok) q.v = pv[(size_t)t * a.v_stride + hc + col];
        }
        return q;
    };
    Inputs q0 = request(0), q1 = request(1), q2 = request(2);
    for (uint32_t t = 0; t < a.rows; ++t) {
        const uint32_t b = t & 1;
        float* vd = vec + (size_t)b * 5 * dim;
        float *vau = vd + dim, *vu = vau + dim, *vk = vu + dim, *vr = vk + dim;
        const Inputs cur = q0;
        q0 = q1;
        q1 = q2;
        q2 = request(t + 3);
        const float kk = cur.k, rr = cur.r, raw_a = cur.a, raw_d = cur.d, vv = cur.v, uu = cur.u;
        const float al = raw_a + rate_b, dl = raw_d + decay_b;
        if constexpr (PREP) {
            if (prep) {
                vd[tid] = raw_d;
                vau[tid] = raw_a;
                vu[tid] = uu;
                vk[tid] = kk;
                vr[tid] = rr;
            }
        } else {
        const float sq = warp_sum(prep ? kk * kk : 0.0f);
        if (lane == 0) ssq[b * 32 + warp] = sq;
        __syncthreads();
        if (prep) {
            float total = 0.0f;
            for (uint32_t w = 0; w < parts; ++w) total += ssq[b * 32 + w];
            const float u = kk / sqrtf(total + 1e-6f);
            const float rate = 1.0f / (1.0f + expf(-al));
            const float decay = expf(-0.60653065971263342f * (1.0f / (1.0f + expf(-dl))));
            vd[tid] = decay;
            vau[tid] = rate * u;
            vu[tid] = u;
            vk[tid] = kk;
            vr[tid] = rr;
        }
        }
        __syncthreads();
        float zp = 0.0f;
#pragma unroll
        for (int i = 0; i < PART; ++i)
            if ((uint32_t)i < cnt) zp = fmaf(vu[i0 + i], S[i], zp);
        zpart[(b * parts + warp) * 32 + lane] = zp;
        __syncthreads();
        float z = 0.0f;
        for (uint32_t w = 0; w < parts; ++w) z += zpart[(b * parts + w) * 32 + lane];
        float op = 0.0f;
#pragma unroll
        for (int i = 0; i < PART; ++i) {
            if ((uint32_t)i < cnt) {
                const float s = fmaf(vk[i0 + i], vv, fmaf(-vau[i0 + i], z, vd[i0 + i] * S[i]));
                S[i] = s;
                op = fmaf(s, vr[i0 + i], op);
            }
        }
        opart[(b * parts + warp) * 32 + lane] = op;
        __syncthreads();
        if (warp == 0 && col_ok) {
            float o = 0.0f;
            for (uint32_t w = 0; w < parts; ++w) o += opart[(b * parts + w) * 32 + lane];
            reinterpret_cast<float*>(a.out)[(size_t)t * a.heads * dim + hc + col] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < PART; ++i)
        if ((uint32_t)i < cnt && col_ok) state[(size_t)(i0 + i) * dim + col] = S[i];
}

// One warp per (row, head): the per-token vectors of the recurrence for a whole pass at once, in place: decay_logit <- decay,
// rate_logit <- rate * unit key, unit <- unit key. Takes the transcendental functions out of the token-by-token chain of a prompt.
__global__ void __launch_bounds__(128) general_delta_prepare_kernel(const uzu_general_delta_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= a.rows * a.heads) return;
    const uint32_t row = unit / a.heads, h = unit % a.heads, hc = h * a.dim;
    const float* k = reinterpret_cast<const float*>(a.k) + (size_t)row * a.k_stride + hc;
    float* rate = reinterpret_cast<float*>(a.rate_logit) + (size_t)row * a.rate_stride + hc;
    float* decay = reinterpret_cast<float*>(a.decay_logit) + (size_t)row * a.decay_stride + hc;
    float* u = reinterpret_cast<float*>(a.unit) + (size_t)row * a.heads * a.dim + hc;
    const float* rb = a.rate_bias ? reinterpret_cast<const float*>(a.rate_bias) + hc : nullptr;
    const float* db = a.decay_bias ? reinterpret_cast<const float*>(a.decay_bias) + hc : nullptr;
    float ss = 0.0f;
    for (uint32_t i = lane; i < a.dim; i += 32) ss = fmaf(k[i], k[i], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
    for (uint32_t i = lane; i < a.dim; i += 32) {
        const float uu = k[i] * inv;
        const float al = rate[i] + (rb ? rb[i] : 0.0f), dl = decay[i] + (db ? db[i] : 0.0f);
        decay[i] = expf(-0.60653065971263342f * (1.0f / (1.0f + expf(-dl))));
        rate[i] = (1.0f / (1.0f + expf(-al))) * uu;
        u[i] = uu;
    }
}

// one warp per (row, head)
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const uzu_head_norm_gate_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= a.rows * a.heads) return;
    const uint32_t row = unit / a.heads, h = unit % a.heads;
    const float* x = reinterpret_cast<const float*>(a.x) + (size_t)row * a.x_stride + (size_t)h * a.dim;
    const float* gate = a.gate ? reinterpret_cast<const float*>(a.gate) + (size_t)row * a.gate_stride + (size_t)h * a.dim : nullptr;
    const float* sc = a.scales ? reinterpret_cast<const float*>(a.scales) + (size_t)h * a.dim : nullptr;
    float* out = reinterpret_cast<float*>(a.out) + (size_t)row * a.out_stride + (size_t)h * a.dim;
    float inv = 1.0f, pre = 1.0f;
    if (a.denom) {          // the row is first divided by max(|denom|, floor) + denom_epsilon
        float d = fabsf(reinterpret_cast<const float*>(a.denom)[(size_t)row * a.heads + h]);
        if (a.denom_floor) d = fmaxf(d, reinterpret_cast<const float*>(a.denom_floor)[(size_t)row * a.heads + h]);
        pre = 1.0f / (d + a.denom_epsilon);
    }
    if (a.normalize) {
        float ss = 0.0f;
        for (uint32_t i = lane; i < a.dim; i += 32) { const float y = x[i] * pre; ss = fmaf(y, y, ss); }
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)a.dim + a.epsilon);
    }
    for (uint32_t i = lane; i < a.dim; i += 32) {
        float v = x[i] * pre * inv;
        if (sc) v *= sc[i];
        if (gate) v *= a.gate_op == 1 ? gate[i] / (1.0f + expf(-gate[i])) : 1.0f / (1.0f + expf(-gate[i]));
        out[i] = v;
    }
}

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_general_delta_encode(uzu_command_buffer* cmd, const uzu_general_delta_args* a) {
    if (!encodable(cmd, "general_delta")) return;
    if (!a->r || !a->k || !a->v || !a->rate_logit || !a->decay_logit || !a->state || !a->out || a->dim == 0 || a->dim > 512 || a->heads == 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "general_delta: null operand or head size outside 1..512");
        return;
    }
    if (a->rows == 0) return;
    // passes of several tokens with a scratch for the unit keys: the per-token vectors are formed for all tokens at once first
    const bool prepared = a->unit != 0 && a->rows >= 4;
    if (prepared) {
        const uint32_t units = a->rows * a->heads;
        launch(cmd, "general_delta_prepare_kernel", general_delta_prepare_kernel, dim3((units + 3) / 4), dim3(128), 0, *a);
    }
    // key channels per warp: about 16 warps per CTA whatever the head size (4 channels up to 64, 8 at 128, ...), so that a thread's
    // token-by-token chain is short and the schedulers have other warps to issue from. Measured, 1024 tokens, 16 heads: head 128: 2.95 ms
    // with 16 channels per warp, 1.70 ms with 8, 1.74 ms with 4; head 64: 0.98 ms with 4, 1.37 ms with 8; head 48: 0.92 ms with 4.
    static const int part_env = [] { const char* e = getenv("UZU_DELTA_PART"); return e ? atoi(e) : 0; }();   // A/B runs: 4 | 8 | 16 | 32
    int part = 4;
    while (part * 16 < (int)a->dim) part *= 2;
    if (part_env == 4 || part_env == 8 || part_env == 16 || part_env == 32) part = part_env;
    while ((a->dim + part - 1) / part > 32) part *= 2;
    const uint32_t parts = (a->dim + part - 1) / part;
    const size_t smem = ((size_t)2 * 5 * a->dim + (size_t)4 * parts * 32 + 64) * sizeof(float);
    const dim3 grid((a->dim + 31) / 32, a->heads), block(parts * 32);
    auto go = [&](auto kernel, std::atomic<uint64_t>& done) {
        if (smem > 48 * 1024) opt_in_dynamic_smem(cmd, kernel, (int)smem, done);
        launch(cmd, "general_delta_kernel", kernel, grid, block, smem, *a);
    };
    static std::atomic<uint64_t> done[8];
    if (part == 4) prepared ? go(general_delta_kernel<true, 4>, done[0]) : go(general_delta_kernel<false, 4>, done[1]);
    else if (part == 8) prepared ? go(general_delta_kernel<true, 8>, done[2]) : go(general_delta_kernel<false, 8>, done[3]);
    else if (part == 16) prepared ? go(general_delta_kernel<true, 16>, done[4]) : go(general_delta_kernel<false, 16>, done[5]);
    else prepared ? go(general_delta_kernel<true, 32>, done[6]) : go(general_delta_kernel<false, 32>, done[7]);
}

void uzu_head_norm_gate_encode(uzu_command_buffer* cmd, const uzu_head_norm_gate_args* a) {
    if (!encodable(cmd, "head_norm_gate")) return;
    if (!a->x || !a->out || a->dim == 0 || a->heads == 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "head_norm_gate: null operand");
        return;
    }
    if (a->rows == 0) return;
    uzu_head_norm_gate_args b = *a;
    if (!b.x_stride) b.x_stride = b.heads * b.dim;
    if (!b.gate_stride) b.gate_stride = b.heads * b.dim;
    if (!b.out_stride) b.out_stride = b.heads * b.dim;
    const uint32_t units = b.rows * b.heads;
    launch(cmd, "head_norm_gate_kernel", head_norm_gate_kernel, dim3((units + 3) / 4), dim3(128), 0, b);
}

}  // extern "C"
