// Causal attention forward with online softmax and paged K/V, head_dim 128.
//
// One CTA owns 128 query rows of one head and walks the KV pages that the causal
// mask leaves visible.  It replaces the per-page op sequence of a KTIR attention
// kernel — indirect ktdp.load of a K and a V page through the block table, two
// linalg.matmul, mask / max / exp / sum / rescale in f32 — which the reference
// dispatches op by op (examples/triton-ktir/paged_attention.mlir:183-396,
// ktir_cpu/ops/memory_ops.py:867-915, ktir_cpu/dialects/linalg_ops.py:136-347).
//
// Roles: warp 0 streams Q once and K/V pages into 2-stage shared-memory rings by
// TMA (page id read from the block table); warp 1 issues tcgen05.mma — S = Q K^T
// into one of two TMEM score buffers, then P V into one of two TMEM product
// buffers; warps 2-9 are the softmax: two threads share a query row (each owns half
// of the page's columns and half of the output columns), read their part of S from
// TMEM, apply scale and mask, agree on the running max through shared memory, write
// P (f16) to shared memory in the 128-byte-swizzled K-major layout, and fold the
// previous page's P V product into their f32 output half-row held in registers.  S of
// page j+1 is computed while page j is in the softmax.  All waits are bounded.
//
// Numerics: scores, max, sum and the output accumulator are f32 as in the
// reference; P is rounded to f16 before the second matmul (relative error
// <= 2^-11), which keeps f16 outputs inside the 1e-2 attention tolerance.
#include "tc_common.cuh"

#define AT_BM 128
#define AT_D 128
#define AT_THREADS 320
#define AT_Q_BYTES (AT_BM * AT_D * 2)

static __device__ __forceinline__ void at_tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                                      int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

static __device__ __forceinline__ float at_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

enum { B_QFULL = 0, B_KFULL = 1, B_KEMPTY = 3, B_VFULL = 5, B_VEMPTY = 7, B_SFULL = 9, B_SEMPTY = 11, B_PFULL = 13,
       B_PVFULL = 14, B_PVEMPTY = 16, B_COUNT = 18 };

template <int BN>
__global__ void __launch_bounds__(AT_THREADS, 1)
ktb_attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const ktb_attn_args a, int q_blocks,
                         ktb_status* st) {
    constexpr int KV_BYTES = BN * AT_D * 2;            // one K or V page in shared memory
    constexpr int KV_BLK = BN * 128;                   // bytes of one [BN x 64] block
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;                                // 2 blocks [128 x 64]
    uint8_t* sK = sQ + AT_Q_BYTES;                     // 2 stages
    uint8_t* sV = sK + 2 * KV_BYTES;                   // 2 stages
    uint8_t* sP = sV + 2 * KV_BYTES;                   // [128 x BN] as blocks of [128 x 64] (at least one)
    constexpr int P_BYTES = (BN < 64 ? 64 : BN) * AT_BM * 2;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* xm = reinterpret_cast<float*>(tmem_slot + 4);      // [2 parities][2 halves][128 rows] partial maxima
    float* xl = xm + 2 * 2 * AT_BM;                           // [2 halves][128 rows] partial sums

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // query blocks of one head run back to back (its K/V pages stay in L2); within a head the
    // late blocks, which see the most KV pages, go first
    const int head = blockIdx.x / q_blocks;
    const int qb = q_blocks - 1 - blockIdx.x % q_blocks;
    const int q0 = qb * AT_BM;
    // pages this query block can see: kv position p is visible to row R iff p <= R + delta
    int n = a.num_tiles;
    {
        const long long last = (long long)q0 + AT_BM - 1 + a.causal_delta;
        const long long vis = last < 0 ? 0 : last / BN + 1;
        if (a.causal && vis < n) n = (int)vis;
    }

    if (threadIdx.x == 0) {
        tc_mbar_init(&bars[B_QFULL], 1);
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(&bars[B_KFULL + i], 1);
            tc_mbar_init(&bars[B_KEMPTY + i], 1);
            tc_mbar_init(&bars[B_VFULL + i], 1);
            tc_mbar_init(&bars[B_VEMPTY + i], 1);
            tc_mbar_init(&bars[B_SFULL + i], 1);
            tc_mbar_init(&bars[B_SEMPTY + i], 8);
            tc_mbar_init(&bars[B_PVFULL + i], 1);
            tc_mbar_init(&bars[B_PVEMPTY + i], 8);
        }
        tc_mbar_init(&bars[B_PFULL], 8);
        *abort_flag = 0;
        tc_fence_barrier_init();
    }
    __syncthreads();
    if (warp == 1) tc_tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base;            // 2 x 128 columns
    const uint32_t tmem_pv = tmem_base + 256;     // 2 x 128 columns

    if (warp == 0) {
        if (lane == 0 && n > 0) {
            tc_prefetch_tmap(&map_q);
            tc_prefetch_tmap(&map_k);
            tc_prefetch_tmap(&map_v);
            tc_mbar_expect_tx(&bars[B_QFULL], AT_Q_BYTES);
            tc_tma_load_3d(sQ, &map_q, &bars[B_QFULL], 0, head, q0);
            tc_tma_load_3d(sQ + AT_BM * 128, &map_q, &bars[B_QFULL], 64, head, q0);
            const int32_t* bt32 = reinterpret_cast<const int32_t*>(a.arena) + a.bt_off;
            const int64_t* bt64 = reinterpret_cast<const int64_t*>(a.arena) + a.bt_off;
            for (int j = 0; j < n; ++j) {
                const int s = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                long long page = a.bt_dtype == KTB_I64 ? bt64[j] : (long long)bt32[j];
                if (page < 0) {
                    if (atomicExch(&st->negative_index, 1) == 0) st->bad_index_value = (int32_t)page;
                    page = 0;
                }
                if (!tc_mbar_wait(&bars[B_KEMPTY + s], ph ^ 1, abort_flag, st, 11)) break;
                tc_mbar_expect_tx(&bars[B_KFULL + s], KV_BYTES);
                at_tma_load_4d(sK + s * KV_BYTES, &map_k, &bars[B_KFULL + s], 0, head, 0, (int)page);
                at_tma_load_4d(sK + s * KV_BYTES + KV_BLK, &map_k, &bars[B_KFULL + s], 64, head, 0, (int)page);
                if (!tc_mbar_wait(&bars[B_VEMPTY + s], ph ^ 1, abort_flag, st, 12)) break;
                tc_mbar_expect_tx(&bars[B_VFULL + s], KV_BYTES);
                at_tma_load_4d(sV + s * KV_BYTES, &map_v, &bars[B_VFULL + s], 0, head, 0, (int)page);
                at_tma_load_4d(sV + s * KV_BYTES + KV_BLK, &map_v, &bars[B_VFULL + s], 64, head, 0, (int)page);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n > 0) {
            const uint32_t idesc_s = tc_idesc_f16(AT_BM, BN, 0, 0);
            const uint32_t idesc_pv = tc_idesc_f16(AT_BM, AT_D, 0, 1);
            const uint32_t q_addr = tc_smem_u32(sQ), p_addr = tc_smem_u32(sP);
            auto issue_s = [&](int j) {
                const int s = j & 1;
                const uint32_t k_addr = tc_smem_u32(sK + s * KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < AT_D / 16; ++kk) {
                    const uint64_t ad = tc_smem_desc(q_addr + (kk >> 2) * (AT_BM * 128) + (kk & 3) * 32, 16, 1024);
                    const uint64_t bd = tc_smem_desc(k_addr + (kk >> 2) * KV_BLK + (kk & 3) * 32, 16, 1024);
                    tc_mma_f16(tmem_s + s * 128, ad, bd, idesc_s, kk != 0);
                }
                tc_mma_commit(&bars[B_SFULL + s]);
                tc_mma_commit(&bars[B_KEMPTY + s]);
            };
            bool ok = tc_mbar_wait(&bars[B_QFULL], 0, abort_flag, st, 21) &&
                      tc_mbar_wait(&bars[B_KFULL], 0, abort_flag, st, 22);
            if (ok) {
                tc_fence_after_sync();
                issue_s(0);
            }
            for (int j = 0; ok && j < n; ++j) {
                const int s = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (j + 1 < n) {
                    const int s1 = (j + 1) & 1;
                    const uint32_t ph1 = ((j + 1) >> 1) & 1;
                    if (!tc_mbar_wait(&bars[B_KFULL + s1], ph1, abort_flag, st, 23) ||
                        !tc_mbar_wait(&bars[B_SEMPTY + s1], ph1 ^ 1, abort_flag, st, 24)) { ok = false; break; }
                    tc_fence_after_sync();
                    issue_s(j + 1);
                }
                if (!tc_mbar_wait(&bars[B_PFULL], j & 1, abort_flag, st, 25) ||
                    !tc_mbar_wait(&bars[B_VFULL + s], ph, abort_flag, st, 26) ||
                    !tc_mbar_wait(&bars[B_PVEMPTY + s], ph ^ 1, abort_flag, st, 27)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t v_addr = tc_smem_u32(sV + s * KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t ad = tc_smem_desc(p_addr + (kk >> 2) * (AT_BM * 128) + (kk & 3) * 32, 16, 1024);
                    const uint64_t bd = tc_smem_desc(v_addr + kk * 2048, KV_BLK, 1024);
                    tc_mma_f16(tmem_pv + s * 128, ad, bd, idesc_pv, kk != 0);
                }
                tc_mma_commit(&bars[B_PVFULL + s]);
                tc_mma_commit(&bars[B_VEMPTY + s]);
            }
        }
    } else {
        constexpr int BH = BN / 2;                   // score columns per thread
        constexpr int CW = BH >= 32 ? 32 : 16;       // columns per TMEM load
        constexpr int OH = AT_D / 2;                 // output columns per thread
        const int q = warp & 3;                      // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2;            // which half of the columns this thread owns
        const int r = q * 32 + lane;                 // row inside the query block == TMEM lane
        const int R = q0 + r;
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        const float sl = a.scale * 1.4426950408889634f;
        float m_run = a.m_init * 1.4426950408889634f;          // running max, log2 domain
        float l_run = half == 0 ? a.l_init : 0.f;              // this thread's share of the running sum
        float alpha_prev = 1.f;
        float o[OH];
#pragma unroll
        for (int i = 0; i < OH; ++i) o[i] = 0.f;
        const long long limit = (long long)R + a.causal_delta;  // last visible kv position
        bool ok = true;

        auto fold_pv = [&](int jp, float alpha) {
            const uint32_t base = tmem_pv + (jp & 1) * 128 + lane_off + half * OH;
            uint32_t va[32], vb[32];
            tc_tmem_ld32(base, va);
            tc_tmem_ld_wait();
            tc_tmem_ld32(base + 32, vb);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __fmaf_rn(o[i], alpha, __uint_as_float(va[i]));
            tc_tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[32 + i] = __fmaf_rn(o[32 + i], alpha, __uint_as_float(vb[i]));
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&bars[B_PVEMPTY + (jp & 1)]);
        };
        auto chunk_max = [&](const uint32_t (&v)[CW], long long c_abs, bool need_mask, float& mx) {
#pragma unroll
            for (int i = 0; i < CW; ++i) {
                float t = __uint_as_float(v[i]) * sl;
                if (need_mask && c_abs + i > limit) t = -INFINITY;
                mx = fmaxf(mx, t);
            }
        };
        // probabilities of one chunk -> packed f16 in shared memory, partial row sum
        auto chunk_prob = [&](const uint32_t (&v)[CW], int c0, long long c_abs, bool need_mask, float m_new,
                              float& lsum) {
            uint32_t packed[CW / 2];
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int i = 0; i < CW; i += 2) {
                float p0 = at_ex2(__fmaf_rn(__uint_as_float(v[i]), sl, -m_new));
                float p1 = at_ex2(__fmaf_rn(__uint_as_float(v[i + 1]), sl, -m_new));
                if (need_mask) {
                    if (c_abs + i > limit) p0 = 0.f;
                    if (c_abs + i + 1 > limit) p1 = 0.f;
                }
                s0 += p0;
                s1 += p1;
                const __half2 h = __floats2half2_rn(p0, p1);
                packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            }
            lsum += s0 + s1;
            // CW columns = CW/8 16-byte chunks of this row inside block (c0 / 64)
            uint8_t* blk = sP + (c0 >> 6) * (AT_BM * 128) + r * 128;
            const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
            for (int c = 0; c < CW / 8; ++c) {
                const int phys = (chunk0 + c) ^ (r & 7);
                *reinterpret_cast<uint4*>(blk + phys * 16) =
                    make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
        };

        for (int j = 0; j < n; ++j) {
            const int s = j & 1;
            const uint32_t ph = (j >> 1) & 1;
            // after a failed wait the thread keeps iterating (without touching TMEM) so that the
            // named barriers below are still reached by all 256 softmax threads
            if (ok && !tc_mbar_wait(&bars[B_SFULL + s], ph, abort_flag, st, 31)) ok = false;
            tc_fence_after_sync();
            const int cb = half * BH;                               // first column of this thread
            const long long col0 = (long long)j * BN + cb;
            const bool need_mask = a.causal && ((long long)j * BN + BN - 1 > limit);
            const uint32_t sbase = tmem_s + s * 128 + lane_off + cb;
            // pass 1: maximum of the scaled (masked) scores of this thread's columns
            float mx = -INFINITY;
            if (ok) {
                uint32_t va[CW], vb[CW];
                tc_tmem_ld<CW>(sbase, va);
#pragma unroll
                for (int c0 = 0; c0 < BH; c0 += 2 * CW) {
                    tc_tmem_ld_wait();
                    if (c0 + CW < BH) tc_tmem_ld<CW>(sbase + c0 + CW, vb);
                    chunk_max(va, col0 + c0, need_mask, mx);
                    if (c0 + CW < BH) {
                        tc_tmem_ld_wait();
                        if (c0 + 2 * CW < BH) tc_tmem_ld<CW>(sbase + c0 + 2 * CW, va);
                        chunk_max(vb, col0 + c0 + CW, need_mask, mx);
                    }
                }
            }
            // the two threads of a row agree on the page maximum
            float* slot = xm + (j & 1) * (2 * AT_BM);
            slot[half * AT_BM + r] = mx;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            mx = fmaxf(mx, slot[(half ^ 1) * AT_BM + r]);
            const float m_new = fmaxf(m_run, mx);
            const float alpha = at_ex2(m_run - m_new);
            if (j > 0 && ok) {
                // the previous P V product is complete: P may be overwritten, the product folded in
                const int sp = (j - 1) & 1;
                if (!tc_mbar_wait(&bars[B_PVFULL + sp], ((j - 1) >> 1) & 1, abort_flag, st, 32)) ok = false;
                tc_fence_after_sync();
            }
            // pass 2: probabilities -> f16 -> shared memory (K-major, 128-byte swizzle), row sum in f32
            float lsum = 0.f;
            if (ok) {
                uint32_t va[CW], vb[CW];
                tc_tmem_ld<CW>(sbase, va);
#pragma unroll
                for (int c0 = 0; c0 < BH; c0 += 2 * CW) {
                    tc_tmem_ld_wait();
                    if (c0 + CW < BH) tc_tmem_ld<CW>(sbase + c0 + CW, vb);
                    chunk_prob(va, cb + c0, col0 + c0, need_mask, m_new, lsum);
                    if (c0 + CW < BH) {
                        tc_tmem_ld_wait();
                        if (c0 + 2 * CW < BH) tc_tmem_ld<CW>(sbase + c0 + 2 * CW, va);
                        chunk_prob(vb, cb + c0 + CW, col0 + c0 + CW, need_mask, m_new, lsum);
                    }
                }
            }
            tc_fence_before_sync();          // S buffer fully read
            tc_fence_proxy_async();          // P stores visible to the tensor-core (async) proxy
            __syncwarp();
            if (lane == 0 && ok) {
                tc_mbar_arrive(&bars[B_SEMPTY + s]);
                tc_mbar_arrive(&bars[B_PFULL]);
            }
            if (j > 0 && ok) fold_pv(j - 1, alpha_prev);
            l_run = l_run * alpha + lsum;
            m_run = m_new;
            alpha_prev = alpha;
        }
        if (ok && n > 0) {
            const int sp = (n - 1) & 1;
            if (tc_mbar_wait(&bars[B_PVFULL + sp], ((n - 1) >> 1) & 1, abort_flag, st, 33)) {
                tc_fence_after_sync();
                fold_pv(n - 1, alpha_prev);
            } else {
                ok = false;
            }
        }
        // total row sum = the two partial sums (same rescaling history on both threads)
        xl[half * AT_BM + r] = l_run;
        asm volatile("bar.sync 2, 256;" ::: "memory");
        const float l_tot = xl[r] + xl[AT_BM + r];
        if (ok && *abort_flag == 0 && R < a.seq_q) {
            const float inv = 1.0f / l_tot;
            __half* dst = reinterpret_cast<__half*>(a.arena) + a.o_off + (int64_t)R * a.o_row_stride +
                          (int64_t)head * a.o_head_stride + half * OH;
#pragma unroll
            for (int c = 0; c < OH; c += 8) {
                uint4 w;
                __half2* h = reinterpret_cast<__half2*>(&w);
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(o[c + 2 * i] * inv, o[c + 2 * i + 1] * inv);
                *reinterpret_cast<uint4*>(dst + c) = w;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc_tmem_dealloc(tmem_base, 512);
}

template <int BN>
static int launch_attn(ktb_ctx* ctx, const ktb_attn_args& a, const CUtensorMap& mq, const CUtensorMap& mk,
                       const CUtensorMap& mv) {
    constexpr size_t SMEM = AT_Q_BYTES + 4 * (size_t)(BN * AT_D * 2) + (size_t)(BN < 64 ? 64 : BN) * AT_BM * 2 + 1024 + 512 + 6 * AT_BM * 4;
    static bool attr_set = false;
    if (!attr_set) {
        KTB_CUDA(ctx, cudaFuncSetAttribute(ktb_attention_fwd_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        attr_set = true;
    }
    const int q_blocks = (a.seq_q + AT_BM - 1) / AT_BM;
    ktb_attention_fwd_kernel<BN><<<q_blocks * a.heads, AT_THREADS, SMEM, ctx->stream>>>(mq, mk, mv, a, q_blocks, ctx->dev_status);
    KTB_CHECK_LAUNCH(ctx, "ktb_attention_fwd_kernel");
    return KTB_OK;
}

extern "C" int ktb_launch_attention_fwd(ktb_ctx* ctx, const ktb_attn_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    const ktb_attn_args& a = *args;
    if (a.head_dim != AT_D) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "attention_fwd", "head_dim must be 128");
    if (a.page != 32 && a.page != 64 && a.page != 128)
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "attention_fwd", "KV page must hold 32, 64 or 128 rows");
    if (a.seq_q <= 0 || a.heads <= 0 || a.num_tiles <= 0) return KTB_OK;
    if ((a.q_row_stride % 8) || (a.q_head_stride % 8) || (a.o_row_stride % 8) || (a.o_head_stride % 8) ||
        (a.kv_page_stride % 8) || (a.kv_row_stride % 8) || (a.kv_head_stride % 8) || (a.q_off % 8) || (a.o_off % 8) ||
        (a.k_off % 8) || (a.v_off % 8))
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "attention_fwd", "strides and offsets must be multiples of 8 elements");
    __half* base = reinterpret_cast<__half*>(a.arena);
    CUtensorMap mq, mk, mv;
    {
        const uint64_t dims[3] = {AT_D, (uint64_t)a.heads, (uint64_t)a.seq_q};
        const uint64_t str[2] = {(uint64_t)a.q_head_stride * 2, (uint64_t)a.q_row_stride * 2};
        const uint32_t box[3] = {64, 1, AT_BM};
        if (!tc_make_map_f16(&mq, base + a.q_off, 3, dims, str, box))
            return ktb_fail(ctx, KTB_E_CUDA, "attention_fwd", "cuTensorMapEncodeTiled(Q) failed");
    }
    for (int which = 0; which < 2; ++which) {
        const uint64_t dims[4] = {AT_D, (uint64_t)a.heads, (uint64_t)a.page, (uint64_t)a.n_pages_total};
        const uint64_t str[3] = {(uint64_t)a.kv_head_stride * 2, (uint64_t)a.kv_row_stride * 2, (uint64_t)a.kv_page_stride * 2};
        const uint32_t box[4] = {64, 1, (uint32_t)a.page, 1};
        if (!tc_make_map_f16(which ? &mv : &mk, base + (which ? a.v_off : a.k_off), 4, dims, str, box))
            return ktb_fail(ctx, KTB_E_CUDA, "attention_fwd", "cuTensorMapEncodeTiled(K/V) failed");
    }
    switch (a.page) {
        case 32: return launch_attn<32>(ctx, a, mq, mk, mv);
        case 64: return launch_attn<64>(ctx, a, mq, mk, mv);
        default: return launch_attn<128>(ctx, a, mq, mk, mv);
    }
}
