// Dense (unquantised) prompt GEMM on the 5th-generation tensor cores: D[m, n] (+)= scale * A[m, k] . W[n, k]^T with A and W bf16 in
// memory, f32 accumulators in tensor memory, f32 output. The dense counterpart of the quantised prefill GEMM (prefill_gemm.cu): same
// tile shapes, shared-memory layout and barrier protocol, but the producers have nothing to dequantise -- both operand tiles travel by
// cp.async straight into their swizzled stage, several K blocks ahead, and no thread touches the data.
//
//   CTA = 128 tokens x 128 features, K in blocks of 64, 4 stages of (16 KB activation tile + 16 KB weight tile).
//   warps 0..3 (128 threads): PRODUCERS. Per K block each thread copies 8 + 8 16-byte pieces (8 consecutive lanes per row: whole
//     128-byte lines) into the K-major SWIZZLE_128B layout (8-row x 128-byte atoms, piece index XOR row-in-atom), waits for its copies
//     of the block two iterations back, fences them to the async proxy and arrives on the stage's `full` barrier.
//   warp 4, one lane: MMA ISSUER. Per K block 4 x tcgen05.mma.cta_group::1.kind::f16 (128 x 128 x 16) into 128 TMEM columns, then
//     tcgen05.commit on the stage's `empty` barrier; after the last block a commit on the accumulator barrier.
//   warps 0..3 again: EPILOGUE. tcgen05.ld 32 lanes x 32 columns, scale / sigmoid gate / accumulate, f32 stores.
// Every barrier wait is bounded (about a second): a wait that runs out sets an error word, the CTA stops working, still meets at the
// final barrier, frees its tensor memory and returns.
#include "common.cuh"

namespace uzu {

struct DenseUmmaParams {
    const __nv_bfloat16* a;    // [m, k] bf16 (the caller's f32 rows, converted)
    const __nv_bfloat16* w;    // [n, k]
    float* d;                  // [m, ldd]
    const float* gate;         // optional [m, gate_ld]
    const float* gate_bias;    // optional [n], added to the gate
    const float* col_scale;    // optional [n]
    const float* bias;         // optional [n], added after scale / gate / col_scale
    const float* row_scale;    // optional [m]
    uint32_t m, n, k, ldd, gate_ld, accumulate;
    float scale;
    uint32_t desc_hi, desc_lbo, k_step, idesc;
    unsigned int* error;
};

__device__ unsigned int g_dense_umma_error = 0;

constexpr uint32_t DU_TILE_BYTES = 128 * 64 * 2;
constexpr int DU_STAGES = 4;
constexpr int DU_NP = 128;
constexpr uint32_t DU_STAGE_BYTES = 2 * DU_TILE_BYTES;

__device__ __forceinline__ uint32_t du_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void du_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void du_mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool du_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
// false when the phase did not complete within ~1 s (the caller gives up)
__device__ __forceinline__ bool du_mbar_wait(uint32_t bar, uint32_t parity) {
    if (du_mbar_try_wait(bar, parity)) return true;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    uint32_t spins = 0;
    while (!du_mbar_try_wait(bar, parity)) {
        if ((++spins & 1023u) == 0) {
            uint64_t t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 1000000000ull) return false;
        }
    }
    return true;
}
__device__ __forceinline__ void du_cp_async16(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint32_t du_tile_off(uint32_t row, uint32_t ch) { return row * 128u + ((ch ^ (row & 7u)) << 4); }

__global__ void __launch_bounds__(DU_NP + 32, 1) dense_umma_kernel(const DenseUmmaParams p) {
    extern __shared__ uint8_t du_smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * DU_STAGES + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t gave_up;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t smem_base = du_smem_u32(du_smem_raw);
    const uint32_t pad = (1024u - (smem_base & 1023u)) & 1023u;    // swizzle atoms sit on 1024-byte boundaries
    smem_base += pad;
    const uint32_t bar0 = du_smem_u32(bars);
    auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (DU_STAGES + s); };
    const uint32_t accum_bar = bar0 + 8u * (2 * DU_STAGES);

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < DU_STAGES; ++s) {
                du_mbar_init(full_bar(s), DU_NP);
                du_mbar_init(empty_bar(s), 1);
            }
            du_mbar_init(accum_bar, 1);
            gave_up = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(du_smem_u32(&tmem_slot)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    const uint32_t n0 = blockIdx.x * 128u, m0 = blockIdx.y * 128u;
    const uint32_t nkb = p.k >> 6;
    auto fail = [&](uint32_t code) {
        gave_up = 1;
        atomicCAS(p.error, 0u, code);
    };

    if (tid < (uint32_t)DU_NP) {
        // ================================ producers ================================
        constexpr int PA = DU_STAGES - 2;                       // K blocks in flight ahead of the one being handed over
        auto issue = [&](uint32_t j, uint32_t stage) {
            const uint32_t st = smem_base + stage * DU_STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t c = (uint32_t)i * DU_NP + tid, row = c >> 3, ch = c & 7u;
                const bool a_ok = m0 + row < p.m, w_ok = n0 + row < p.n;     // rows past the edge are zero-filled
                du_cp_async16(st + du_tile_off(row, ch), p.a + (size_t)(a_ok ? m0 + row : 0u) * p.k + (size_t)j * 64u + ch * 8u, a_ok ? 16u : 0u);
                du_cp_async16(st + DU_TILE_BYTES + du_tile_off(row, ch), p.w + (size_t)(w_ok ? n0 + row : 0u) * p.k + (size_t)j * 64u + ch * 8u,
                              w_ok ? 16u : 0u);
            }
        };
        pdl_wait();
        uint32_t a_stage = 0, a_parity = 1, c_stage = 0;
        bool ok = true;
        for (uint32_t t = 0; t < nkb + PA && ok; ++t) {
            if (t < nkb) {
                ok = du_mbar_wait(empty_bar(a_stage), a_parity);
                if (!ok) { fail(1); break; }
                issue(t, a_stage);
                if (++a_stage == (uint32_t)DU_STAGES) { a_stage = 0; a_parity ^= 1u; }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (t < (uint32_t)PA) continue;
            asm volatile("cp.async.wait_group %0;" ::"n"(PA) : "memory");          // this thread's pieces of block t - PA have landed
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            du_mbar_arrive(full_bar(c_stage));
            if (++c_stage == (uint32_t)DU_STAGES) c_stage = 0;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // ================================ epilogue ================================
        if (ok && !du_mbar_wait(accum_bar, 0)) { fail(2); ok = false; }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t row = m0 + warp * 32u + lane;
#pragma unroll 1
            for (uint32_t cb = 0; cb < 4u; ++cb) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((warp * 32u) << 16) + cb * 32u;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, "
                    "[%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const uint32_t col0 = n0 + cb * 32u;
                if (row >= p.m || col0 >= p.n) continue;
                float* out = p.d + (size_t)row * p.ldd + col0;
                const float* gate = p.gate ? p.gate + (size_t)row * p.gate_ld + col0 : nullptr;
                const float rs = p.row_scale ? p.row_scale[row] : 1.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (col0 + (uint32_t)j < p.n) {
                        float val = __uint_as_float(v[j]) * p.scale;
                        if (p.row_scale) val *= rs;
                        if (gate) val *= 1.0f / (1.0f + expf(-(gate[j] + (p.gate_bias ? p.gate_bias[col0 + j] : 0.0f))));
                        if (p.col_scale) val *= p.col_scale[col0 + j];
                        if (p.bias) val += p.bias[col0 + j];
                        if (p.accumulate) val += out[j];
                        out[j] = val;
                    }
                }
            }
        }
    } else {
        // ================================ MMA issuer (one lane) ================================
        if (lane == 0) {
            uint32_t s = 0, parity = 0;
            for (uint32_t kb = 0; kb < nkb; ++kb) {
                if (!du_mbar_wait(full_bar(s), parity)) { fail(3); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_base + s * DU_STAGE_BYTES, b_addr = a_addr + DU_TILE_BYTES;
                const uint64_t hi = (uint64_t)p.desc_hi << 32;
                const uint32_t lbo = p.desc_lbo << 16;
#pragma unroll
                for (uint32_t kk = 0; kk < 4; ++kk) {
                    const uint64_t da = hi | (uint64_t)((((a_addr >> 4) + kk * p.k_step) & 0x3FFFu) | lbo);
                    const uint64_t db = hi | (uint64_t)((((b_addr >> 4) + kk * p.k_step) & 0x3FFFu) | lbo);
                    const uint32_t accumulate = (kb | kk) != 0u ? 1u : 0u;
                    asm volatile("{ .reg .pred q; setp.ne.b32 q, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, q; }" ::"r"(tmem_base), "l"(da),
                                 "l"(db), "r"(p.idesc), "r"(accumulate)
                                 : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty_bar(s)) : "memory");
                if (++s == (uint32_t)DU_STAGES) { s = 0; parity ^= 1u; }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(accum_bar) : "memory");
        }
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
    }
}

// f32 rows (optionally through tanh) -> bf16 [m, k] for the tensor-core operand
__global__ void dense_cast_bf16_kernel(const float* a, uint32_t lda, __nv_bfloat16* out, uint32_t m, uint32_t k, uint32_t a_op) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (idx >= (size_t)m * k) return;
    const size_t r = idx / k, c = idx % k;                       // k is a multiple of 64: the four elements share a row
    float4 v = *reinterpret_cast<const float4*>(a + r * lda + c);
    if (a_op == 1) { v.x = tanhf(v.x); v.y = tanhf(v.y); v.z = tanhf(v.z); v.w = tanhf(v.w); }
    if (a_op == 2) {
        v.x = fmaxf(v.x, 0.0f); v.y = fmaxf(v.y, 0.0f); v.z = fmaxf(v.z, 0.0f); v.w = fmaxf(v.w, 0.0f);
        v.x *= v.x; v.y *= v.y; v.z *= v.z; v.w *= v.w;
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + idx) = o;
}

// Shapes the tensor-memory kernel takes: one plain product (no z-batches or row groups), bf16 weights, >= 128 rows, k a multiple
// of 64, 16-byte aligned operands, and a bf16 workspace of m * k elements from the caller.
bool dense_umma_applicable(const uzu_dense_linear_args& a) {
    static const bool off = getenv("UZU_DENSE_NO_UMMA") != nullptr;      // A/B runs
    if (off || !a.workspace || a.weights_dt != UZU_DT_BF16 || a.batch != 1 || a.group_offsets || a.rows_map || a.pair_rows) return false;
    if (a.m < 128 || a.k % 64u != 0 || a.n < 64) return false;
    if ((a.a & 15u) || (a.w & 15u) || (a.workspace & 15u) || a.lda % 4u != 0) return false;
    return true;
}

void encode_dense_umma(uzu_command_buffer* cmd, const uzu_dense_linear_args& a) {
    if (!a.a_bf16) {
        const size_t quads = (size_t)a.m * a.k / 4;
        launch(cmd, "dense_cast_bf16_kernel", dense_cast_bf16_kernel, dim3((unsigned)((quads + 255) / 256)), dim3(256), 0, (const float*)a.a, a.lda,
               (__nv_bfloat16*)a.workspace, a.m, a.k, a.a_op);
    }
    DenseUmmaParams p{};
    p.a = a.a_bf16 ? (const __nv_bfloat16*)a.a : (const __nv_bfloat16*)a.workspace;
    p.w = (const __nv_bfloat16*)a.w;
    p.d = (float*)a.d;
    p.gate = (const float*)a.gate;
    p.gate_bias = (const float*)a.gate_bias;
    p.col_scale = (const float*)a.col_scale;
    p.bias = (const float*)a.bias;
    p.row_scale = (const float*)a.row_scale;
    p.m = a.m; p.n = a.n; p.k = a.k; p.ldd = a.ldd; p.gate_ld = a.gate_ld; p.accumulate = a.accumulate;
    p.scale = a.scale;
    // shared-memory matrix descriptor: start address >> 4 @ [0,14), LBO >> 4 @ [16,30), SBO >> 4 @ [32,46), version 1 @ [46,48), layout
    // SWIZZLE_128B = 2 @ [61,64); K-major: SBO = 1024 B between 8-row groups, LBO unused (1), UMMA_K = 16 bf16 = 32 B -> +2 per step.
    p.desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    p.desc_lbo = 1;
    p.k_step = 2;
    // instruction descriptor (kind::f16): f32 accumulate @ 4, bf16 A @ 7, bf16 B @ 10, both K-major, N >> 3 @ [17,23), M >> 4 @ [24,29)
    p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
    void* err = nullptr;
    cudaGetSymbolAddress(&err, g_dense_umma_error);
    p.error = (unsigned int*)err;
    constexpr size_t smem = (size_t)DU_STAGES * DU_STAGE_BYTES + 1024;
    static std::atomic<uint64_t> opt_in{0};
    opt_in_dynamic_smem(cmd, dense_umma_kernel, (int)smem, opt_in);
    launch(cmd, "dense_umma_kernel", dense_umma_kernel, dim3((a.n + 127u) / 128u, (a.m + 127u) / 128u), dim3(DU_NP + 32), smem, p);
}

}  // namespace uzu

// 0 = every tensor-memory GEMM so far completed its barrier waits; otherwise the code of the first wait that ran out
extern "C" unsigned int uzu_debug_dense_umma_error(void) {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, uzu::g_dense_umma_error, sizeof v);
    return v;
}
