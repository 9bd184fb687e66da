// Windowed softmax attention on the tensor pipe: bf16 caches and passes of >= 64 rows (the plain kernel of window_attention.cu serves
// everything else). One CTA = 64 query rows of one head (4 warps x 16 rows). It walks only the key tiles of 64 that some row of it can see:
// first the tiles of the kept first tokens that lie before the window, then the tiles from the window's start of the CTA's first row up
// to its last row; the next tile's keys and values arrive by cp.async while the current one is used. mma.sync.m16n8k16 (bf16 x bf16 -> f32):
//   S = (q * scale * temp) . K^T   with q = q_hi + q_lo, two bf16 numbers per f32 query entry (two MMAs per tile of S);
//   soft cap, mask (j <= i and (i - j < window or j < keep_first)) and the running (max, sum) of the softmax in f32 on the accumulator
//   fragment, in units of ln 2; the accumulators of O are rescaled when a row's maximum moves;
//   O += p . V                     with p = p_hi + p_lo again, the fragment of S re-used as the A fragment, V by ldmatrix.trans.
// The split keeps the error of the query and of the weights below 2^-16 relative, so only the cache's own bf16 rounding remains.
// At the end a row's sum is divided by its weight sum and turned back by the row's position (a thread's fragment holds whole pairs).
#include "common.cuh"

namespace uzu {

namespace {

constexpr int WM_BM = 64, WM_BN = 64, WM_PAD = 8;

__device__ __forceinline__ void wm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void wm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void wm_cp_async16(void* smem_ptr, const void* gmem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(gmem_ptr) : "memory");
}

// x = hi + lo with both parts bf16; a pair of values packed for an MMA fragment
__device__ __forceinline__ void wm_split_pair(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
    const __nv_bfloat162 h = __halves2bfloat162(h0, h1);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x0 - __bfloat162float(h0), x1 - __bfloat162float(h1));
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

}  // namespace

// DK = most 16-channel steps of a key row (dim / 16 rounded up to 4 or 8), DV = most 16-column blocks of a value row
template <int DK, int DV>
__global__ void __launch_bounds__(128) window_attention_mma_kernel(const uzu_window_attention_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char wm_raw[];
    const uint32_t dim = a.dim, vdim = a.vdim, ldk = dim + WM_PAD, ldv = vdim + WM_PAD, dk = dim / 16, dv = vdim / 16;
    __nv_bfloat16* q_hi = reinterpret_cast<__nv_bfloat16*>(wm_raw);      // [64][ldk]
    __nv_bfloat16* q_lo = q_hi + WM_BM * ldk;
    __nv_bfloat16* k_s = q_lo + WM_BM * ldk;                             // [2][64][ldk]
    __nv_bfloat16* v_s = k_s + 2 * WM_BN * ldk;                          // [2][64][ldv]
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const uint32_t h = blockIdx.y, kvh = h / (a.heads / a.kv_heads);
    const uint32_t prefix = a.prefix;
    const uint32_t mt = gridDim.x - 1 - blockIdx.x;                      // the row tiles with the most keys first
    const uint32_t m0 = mt * WM_BM;
    const uint32_t rows_here = min((uint32_t)WM_BM, a.rows - m0);
    const uint32_t i_first = prefix + m0, i_last = i_first + rows_here - 1, nkeys = i_last + 1;
    const uint32_t window = a.window ? a.window : 0xFFFFFFFFu, keep = a.keep_first;
    // tiles: [0, keep_tiles) hold kept tokens before the window, then [t_lo, t_hi]
    const uint32_t j_lo = i_first + 1 > window ? i_first + 1 - window : 0u;
    const uint32_t t_lo = j_lo / WM_BN, t_hi = i_last / WM_BN;
    const uint32_t keep_tiles = min((keep + WM_BN - 1) / WM_BN, t_lo);
    const uint32_t ntiles = keep_tiles + (t_hi - t_lo + 1);
    auto tile_of = [&](uint32_t idx) { return idx < keep_tiles ? idx : t_lo + (idx - keep_tiles); };
    constexpr float kLog2e = 1.4426950408889634f;
    const float qscale = a.scale * (a.head_temp ? reinterpret_cast<const float*>(a.head_temp)[h] : 1.0f);
    const bool capped = a.softcap > 0.0f;
    const float cap2 = a.softcap * kLog2e, inv_cap2 = capped ? 2.0f * kLog2e / a.softcap : 0.0f;      // tanh(x) = 1 - 2 / (2^(2 x log2 e) + 1)
    const __nv_bfloat16* keys = reinterpret_cast<const __nv_bfloat16*>(a.keys) + (size_t)kvh * dim;
    const __nv_bfloat16* values = reinterpret_cast<const __nv_bfloat16*>(a.values) + (size_t)kvh * vdim;
    const size_t kstride = (size_t)a.kv_heads * dim, vstride = (size_t)a.kv_heads * vdim;
    // a thread's 16-byte pieces of a tile: piece tid, tid + 128, ... of rows x (row size / 8); row and column advance without divisions
    const uint32_t kc = dim / 8, vc = vdim / 8;
    const uint32_t k_r0 = tid / kc, k_c0 = tid % kc, k_dr = 128 / kc, k_dc = 128 % kc;
    const uint32_t v_r0 = tid / vc, v_c0 = tid % vc, v_dr = 128 / vc, v_dc = 128 % vc;
    auto load_rows = [&](__nv_bfloat16* dst_tile, uint32_t ld, const __nv_bfloat16* src, size_t stride, uint32_t j0, uint32_t r, uint32_t c, uint32_t dr,
                         uint32_t dc, uint32_t pieces_per_row) {
        while (r < WM_BN) {
            __nv_bfloat16* dst = dst_tile + r * ld + c * 8;
            if (j0 + r < nkeys) wm_cp_async16(dst, src + (size_t)(j0 + r) * stride + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            r += dr; c += dc;
            if (c >= pieces_per_row) { c -= pieces_per_row; ++r; }
        }
    };
    auto load_tile = [&](uint32_t idx) {      // rows past the last key are zero: cache pages beyond the context may not exist
        const uint32_t j0 = tile_of(idx) * WM_BN, buf = idx & 1;
        load_rows(k_s + buf * WM_BN * ldk, ldk, keys, kstride, j0, k_r0, k_c0, k_dr, k_dc, kc);
        load_rows(v_s + buf * WM_BN * ldv, ldv, values, vstride, j0, v_r0, v_c0, v_dr, v_dc, vc);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float o[2 * DV][4];
#pragma unroll
    for (int n = 0; n < 2 * DV; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[n][c] = 0.0f;
    float run_m[2] = {-INFINITY, -INFINITY}, run_l[2] = {0.0f, 0.0f};     // rows row_lo and row_lo + 8 (a thread's share of the sum)
    const uint32_t row_lo = warp * 16 + g;                     // this thread's rows of the tile: row_lo and row_lo + 8
    const uint32_t i_lo = i_first + row_lo;
    const uint32_t i_warp_first = i_first + warp * 16, i_warp_last = i_warp_first + 15;
    load_tile(0);
    {   // the query tile, scaled, as hi + lo; sixteen loads of a thread in flight, behind the first tile's requests
        const float* q = reinterpret_cast<const float*>(a.query) + (size_t)m0 * a.heads * dim + (size_t)h * dim;
        const uint32_t pairs = dim / 2, total = WM_BM * pairs;
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
                    wm_split_pair(x[u].x * qscale, x[u].y * qscale, hi, lo);
                    *reinterpret_cast<uint32_t*>(q_hi + r * ldk + c) = hi;
                    *reinterpret_cast<uint32_t*>(q_lo + r * ldk + c) = lo;
                }
            }
        }
    }
    for (uint32_t idx = 0; idx < ntiles; ++idx) {
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();                                       // tile idx is in place, tile idx - 1 is used up
        if (idx + 1 < ntiles) load_tile(idx + 1);
        const uint32_t j0 = tile_of(idx) * WM_BN, j_end = j0 + WM_BN - 1;
        // nothing of this tile is visible to the warp's rows: it lies after them, or before their windows and holds no kept token
        if (j0 > i_warp_last) continue;
        const bool before_window = i_warp_first - min(i_warp_first, j_end) >= window;
        if (before_window && j0 >= keep) continue;
        const __nv_bfloat16* kt = k_s + (idx & 1) * WM_BN * ldk;
        const __nv_bfloat16* vt = v_s + (idx & 1) * WM_BN * ldv;
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
                for (int n = 0; n < 8; ++n) wm_mma(s[n], ah, kb0[n], kb1[n]);
#pragma unroll
                for (int n = 0; n < 8; ++n) wm_mma(s[n], al, kb0[n], kb1[n]);
            }
        }
        // Scores on the fragment: element c of tile n is row row_lo + 8 * (c >> 1), key j0 + n * 8 + t4 * 2 + (c & 1). Only tiles that
        // touch the diagonal, a window's start or the end of the kept tokens need the mask.
        const bool all_visible = j_end <= i_warp_first && (i_warp_last - j0 < window || j_end < keep);
        float tile_m[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float x = s[n][c];
                if (capped) x = cap2 * (1.0f - __fdividef(2.0f, exp2f(x * inv_cap2) + 1.0f));
                else x *= kLog2e;
                if (!all_visible) {
                    const uint32_t i = i_lo + 8 * (c >> 1), j = j0 + n * 8 + t4 * 2 + (c & 1);
                    if (!(j <= i && (i - j < window || j < keep))) x = -INFINITY;
                }
                s[n][c] = x;
                tile_m[c >> 1] = fmaxf(tile_m[c >> 1], x);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            tile_m[r] = fmaxf(tile_m[r], __shfl_xor_sync(0xffffffffu, tile_m[r], 1));
            tile_m[r] = fmaxf(tile_m[r], __shfl_xor_sync(0xffffffffu, tile_m[r], 2));
            const float new_m = fmaxf(run_m[r], tile_m[r]);
            m_use[r] = new_m == -INFINITY ? 0.0f : new_m;          // a row that has seen no key yet: weights and factor are 0
            alpha[r] = exp2f(run_m[r] - m_use[r]);
            run_m[r] = new_m;
            run_l[r] *= alpha[r];
        }
#pragma unroll
        for (int n = 0; n < 2 * DV; ++n) {
            o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
            o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
        }
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float w = exp2f(s[n][c] - m_use[c >> 1]);
                s[n][c] = w;
                run_l[c >> 1] += w;
            }
#pragma unroll
        for (int kk = 0; kk < WM_BN / 16; ++kk) {
            uint32_t ph[4], pl[4];
            wm_split_pair(s[2 * kk][0], s[2 * kk][1], ph[0], pl[0]);
            wm_split_pair(s[2 * kk][2], s[2 * kk][3], ph[1], pl[1]);
            wm_split_pair(s[2 * kk + 1][0], s[2 * kk + 1][1], ph[2], pl[2]);
            wm_split_pair(s[2 * kk + 1][2], s[2 * kk + 1][3], ph[3], pl[3]);
#pragma unroll
            for (int n = 0; n < DV; n += 2) {      // two 16-column blocks at a time: four independent accumulators between hi and lo
                if ((uint32_t)n < dv) {
                    const bool two = (uint32_t)n + 1 < dv;
                    uint32_t b[4], c[4] = {0, 0, 0, 0};
                    const __nv_bfloat16* vb = vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + (lane >> 4) * 8;
                    wm_ldmatrix_x4_trans(b, vb + n * 16);
                    if (two) wm_ldmatrix_x4_trans(c, vb + (n + 1) * 16);
                    wm_mma(o[2 * n], ph, b[0], b[1]);
                    wm_mma(o[2 * n + 1], ph, b[2], b[3]);
                    if (two) {
                        wm_mma(o[2 * n + 2], ph, c[0], c[1]);
                        wm_mma(o[2 * n + 3], ph, c[2], c[3]);
                    }
                    wm_mma(o[2 * n], pl, b[0], b[1]);
                    wm_mma(o[2 * n + 1], pl, b[2], b[3]);
                    if (two) {
                        wm_mma(o[2 * n + 2], pl, c[0], c[1]);
                        wm_mma(o[2 * n + 3], pl, c[2], c[3]);
                    }
                }
            }
        }
    }
    // weight sums of the two rows over the four threads that share them, then the division and the turn back by the row's position
    float inv_l[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = run_l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (a.sinks) l += exp2f(reinterpret_cast<const float*>(a.sinks)[h] * kLog2e - run_m[r]);      // the sink's term (the maximum is in units of ln 2)
        inv_l[r] = 1.0f / l;
        const uint32_t row = row_lo + 8 * r;
        if (a.head_gate && row < rows_here)
            inv_l[r] *= 1.0f / (1.0f + expf(-reinterpret_cast<const float*>(a.head_gate)[(size_t)(m0 + row) * a.head_gate_stride + h]));
    }
    const size_t row_stride = (size_t)a.heads * vdim;
    float* out = reinterpret_cast<float*>(a.out) + (size_t)m0 * row_stride + (size_t)h * vdim;
#pragma unroll
    for (int n = 0; n < 2 * DV; ++n) {
        if ((uint32_t)n < 2 * dv) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint32_t r = row_lo + 8 * half;
                if (r < rows_here) {
                    float x0 = o[n][2 * half] * inv_l[half], x1 = o[n][2 * half + 1] * inv_l[half];
                    const uint32_t pair = n * 4 + t4;
                    if (pair < a.v_pairs) {
                        const size_t at = (size_t)(i_first + r) * a.v_pairs + pair;
                        const float c = reinterpret_cast<const float*>(a.v_cosines)[at], s = reinterpret_cast<const float*>(a.v_sines)[at];
                        const float y0 = x0 * c + x1 * s, y1 = x1 * c - x0 * s;
                        x0 = y0; x1 = y1;
                    }
                    *reinterpret_cast<float2*>(out + (size_t)r * row_stride + n * 8 + t4 * 2) = make_float2(x0, x1);
                }
            }
        }
    }
}

template <int DK, int DV>
static void launch_window_attention_mma(uzu_command_buffer* cmd, const uzu_window_attention_args& a) {
    const size_t smem = ((size_t)4 * WM_BM * (a.dim + WM_PAD) + (size_t)2 * WM_BN * (a.vdim + WM_PAD)) * sizeof(__nv_bfloat16);
    // the opt-in is made once per instance and device: for the largest head sizes the instance serves
    constexpr size_t smem_most = ((size_t)4 * WM_BM * (DK * 16 + WM_PAD) + (size_t)2 * WM_BN * (DV * 16 + WM_PAD)) * sizeof(__nv_bfloat16);
    static std::atomic<uint64_t> opt_in{0};
    opt_in_dynamic_smem(cmd, window_attention_mma_kernel<DK, DV>, (int)smem_most, opt_in);
    launch(cmd, "window_attention_mma_kernel", window_attention_mma_kernel<DK, DV>, dim3((a.rows + WM_BM - 1) / WM_BM, a.heads), dim3(128), smem, a);
}

// Shapes the tensor-pipe kernel takes: bf16 caches, passes of >= 64 rows, key and value sizes multiples of 16 up to 128, 16-byte aligned
// caches and an 8-byte aligned query / output, positions known on the host. Everything else (and every f32 cache) runs the plain kernel.
bool encode_window_attention_mma(uzu_command_buffer* cmd, const uzu_window_attention_args& a) {
    static const bool off = getenv("UZU_WINDOW_NO_MMA") != nullptr;       // A/B runs
    if (off || a.cache_dt != UZU_DT_BF16 || a.rows < WM_BM || a.dim % 16 || a.vdim % 16 || a.dim > 128 || a.vdim > 128) return false;
    if ((a.keys & 15) || (a.values & 15) || (a.query & 7) || (a.out & 7) || a.dynamic_position || ((a.heads * a.vdim) & 1)) return false;
    const bool k8 = a.dim > 64, v8 = a.vdim > 64;
    if (k8 && v8) launch_window_attention_mma<8, 8>(cmd, a);
    else if (k8) launch_window_attention_mma<8, 4>(cmd, a);
    else if (v8) launch_window_attention_mma<4, 8>(cmd, a);
    else launch_window_attention_mma<4, 4>(cmd, a);
    return true;
}

}  // namespace uzu
