// C[M,N] = A[M,K] * B[K,N] (+ constant), f16 operands, f32 accumulation in TMEM.
//
// This is what a KTIR tiled-matmul kernel computes once its per-core 64x64xK-step
// tile loop is recognised as one dense GEMM: the reference runs np.matmul per tile
// and K-step (ktir_cpu/ops/arith_ops.py:323-340) and accumulates through
// linalg.matmul's `outs` (ktir_cpu/dialects/linalg_ops.py:307-347).
//
// Design (tensor-bound): persistent CTAs, one per SM, each producing 128 x BN
// output tiles.  Warp 0 streams A (K-major) and B (N-major) tiles into a
// multi-stage shared-memory ring with TMA (128-byte swizzle); warp 1 issues
// tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM accumulators; warps 2-5
// drain the other accumulator (tcgen05.ld), convert and store C, so the epilogue
// of tile i overlaps the main loop of tile i+1.  All waits are bounded.
//
// Tail: with T tiles on G SMs the last T mod G tiles would keep only some SMs busy for a whole
// tile time (4096^3: 512 tiles on 148 SMs = 3 full rounds + 68 tiles: 4 tile times for 3.46 of
// work).  When at most G / 2 tiles are left over, each is cut into its left and right half
// (128 x BN/2) and the halves go to twice as many SMs: the tail takes about half a tile time, the
// k order of every sum is unchanged (results do not depend on how the tiles were dealt out).
#include "tc_common.cuh"

#define GEMM_BM 128
#define GEMM_BK 64
#define GEMM_THREADS 192
#define GEMM_A_STAGE_BYTES (GEMM_BM * GEMM_BK * 2)
#define GEMM_EPI_BYTES (4 * 2 * 4096)       // epilogue staging: two 4 KB buffers per warp

template <int BN>
struct GemmCfg {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int B_STAGE_BYTES = GEMM_BK * BN * 2;
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr size_t SMEM = (size_t)STAGES * (GEMM_A_STAGE_BYTES + B_STAGE_BYTES) + GEMM_EPI_BYTES + 1024 + 256;
};

// Epilogue of one warp: its 32 rows x `bn` accumulator columns (+ the constant initial value) -> C.
// 128 bytes of each row at a time (64 f16 or 32 f32 columns) are converted, written to one of the
// warp's two 4 KB staging buffers in the 128-byte-swizzle layout (row r, 16-byte chunk c at
// r * 128 + ((c ^ (r & 7)) << 4): conflict-free for the warp's 16-byte stores) and handed to a TMA
// tile store, which writes whole 128-byte row segments and clips at the edges of C.
static __device__ __forceinline__ void gemm_store_rows(const CUtensorMap* map_c, const ktb_gemm_args& a, uint8_t* wbuf,
                                                       int& buf, uint32_t t0, int bn, int row0, int n0, int lane) {
    const bool f16 = a.c_dtype == KTB_F16;
    const int step = f16 ? 64 : 32;
#pragma unroll 1
    for (int c0 = 0; c0 < bn; c0 += step) {
        uint32_t r[32], out[32];
        tc_tmem_ld32(t0 + c0, r);
        tc_tmem_ld_wait();
        if (f16) {
            uint32_t r2[32];
            tc_tmem_ld32(t0 + c0 + 32, r2);
            tc_tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                __half2 lo = __floats2half2_rn(__uint_as_float(r[2 * i]) + a.c_init, __uint_as_float(r[2 * i + 1]) + a.c_init);
                __half2 hi = __floats2half2_rn(__uint_as_float(r2[2 * i]) + a.c_init, __uint_as_float(r2[2 * i + 1]) + a.c_init);
                out[i] = *reinterpret_cast<uint32_t*>(&lo);
                out[16 + i] = *reinterpret_cast<uint32_t*>(&hi);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) out[i] = __float_as_uint(__uint_as_float(r[i]) + a.c_init);
        }
        if (row0 >= a.M || n0 + c0 >= a.N) continue;          // nothing of this piece lies inside C (warp-uniform)
        if (lane == 0) tc_bulk_wait_read<1>();                // the store issued from this buffer two steps ago has read it
        __syncwarp();
        uint8_t* dst = wbuf + buf * 4096 + lane * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(dst + ((c ^ (lane & 7)) << 4)) =
                make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
        tc_fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tc_tma_store_2d(map_c, wbuf + buf * 4096, n0 + c0, row0);
            tc_bulk_commit();
        }
        buf ^= 1;
    }
}

// How the tiles (128 x BN for a CTA, 256 x 256 for a CTA pair; "workers" below) are dealt out, in
// row-major tile order: `full_rounds` whole tiles per worker (tile = w + round * G), then the
// `tail_tiles` left-over tiles: whole, one per worker, or (halved) as two half-width units on
// workers 2 t and 2 t + 1.
struct GemmSched {
    int tiles_n, full_rounds, tail_tiles, halved;
};

struct GemmUnit {
    int tm, n0, bn;      // rows [rows-per-tile * tm, ...), columns [n0, n0 + bn)
};

// The i-th unit of worker `w` of `G`; BN = full tile width.
template <int BN>
static __device__ __forceinline__ bool gemm_unit(const GemmSched& sc, int w, int G, int i, GemmUnit& u) {
    int tile, half = 0;
    u.bn = BN;
    if (i < sc.full_rounds) {
        tile = w + i * G;
    } else if (i == sc.full_rounds && !sc.halved && w < sc.tail_tiles) {
        tile = sc.full_rounds * G + w;
    } else if (i == sc.full_rounds && sc.halved && w < 2 * sc.tail_tiles) {
        tile = sc.full_rounds * G + (w >> 1);
        half = w & 1;
        u.bn = BN / 2;
    } else {
        return false;
    }
    u.tm = tile / sc.tiles_n;
    u.n0 = (tile - u.tm * sc.tiles_n) * BN + half * (BN / 2);
    return true;
}

static GemmSched gemm_sched(int tiles_m, int tiles_n, int workers, int* grid_workers) {
    GemmSched sc;
    const int n_tiles = tiles_m * tiles_n;
    sc.tiles_n = tiles_n;
    sc.full_rounds = n_tiles / workers;
    sc.tail_tiles = n_tiles % workers;
    sc.halved = sc.tail_tiles > 0 && 2 * sc.tail_tiles <= workers;
    *grid_workers = sc.full_rounds ? workers : (sc.halved ? 2 * sc.tail_tiles : sc.tail_tiles);
    return sc;
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
ktb_gemm_f16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, const ktb_gemm_args a, const GemmSched sc, ktb_status* st) {
    using Cfg = GemmCfg<BN>;
    constexpr int S = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + (size_t)S * GEMM_A_STAGE_BYTES;
    uint8_t* sC = sB + (size_t)S * Cfg::B_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sC + GEMM_EPI_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + S;
    uint64_t* tfull = bars + 2 * S;
    uint64_t* tempty = bars + 2 * S + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = (a.K + GEMM_BK - 1) / GEMM_BK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            tc_mbar_init(&full[i], 1);
            tc_mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(&tfull[i], 1);
            tc_mbar_init(&tempty[i], 4);
        }
        *abort_flag = 0;
        tc_fence_barrier_init();
    }
    __syncthreads();
    if (warp == 1) tc_tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tc_prefetch_tmap(&map_a);
            tc_prefetch_tmap(&map_b);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            GemmUnit u;
            for (int it = 0; ok && gemm_unit<BN>(sc, blockIdx.x, gridDim.x, it, u); ++it) {
                const int nb = u.bn / 64;
                for (int kt = 0; kt < KT; ++kt) {
                    if (!tc_mbar_wait(&empty[stage], phase ^ 1, abort_flag, st, 1)) { ok = false; break; }
                    tc_mbar_expect_tx(&full[stage], GEMM_A_STAGE_BYTES + GEMM_BK * u.bn * 2);
                    tc_tma_load_2d(sA + (size_t)stage * GEMM_A_STAGE_BYTES, &map_a, &full[stage], kt * GEMM_BK,
                                   u.tm * GEMM_BM);
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        if (j < nb)
                            tc_tma_load_2d(sB + (size_t)stage * Cfg::B_STAGE_BYTES + (size_t)j * (GEMM_BK * 128), &map_b,
                                           &full[stage], u.n0 + j * 64, kt * GEMM_BK);
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            GemmUnit u;
            for (int it = 0; ok && gemm_unit<BN>(sc, blockIdx.x, gridDim.x, it, u); ++it) {
                const uint32_t idesc = tc_idesc_f16(GEMM_BM, u.bn, 0, 1);
                const int acc = it & 1, accphase = (it >> 1) & 1;
                if (!tc_mbar_wait(&tempty[acc], accphase ^ 1, abort_flag, st, 2)) break;
                tc_fence_after_sync();
                const uint32_t d = tmem_base + acc * BN;
                for (int kt = 0; kt < KT; ++kt) {
                    if (!tc_mbar_wait(&full[stage], phase, abort_flag, st, 3)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = tc_smem_u32(sA + (size_t)stage * GEMM_A_STAGE_BYTES);
                    const uint32_t b_addr = tc_smem_u32(sB + (size_t)stage * Cfg::B_STAGE_BYTES);
#pragma unroll
                    for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
                        const uint64_t ad = tc_smem_desc(a_addr + kk * 32, 16, 1024);
                        const uint64_t bd = tc_smem_desc(b_addr + kk * 2048, GEMM_BK * 128, 1024);
                        tc_mma_f16(d, ad, bd, idesc, (kt | kk) != 0);
                    }
                    tc_mma_commit(&empty[stage]);
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_mma_commit(&tfull[acc]);
            }
        }
    } else {
        const int q = warp & 3;                       // TMEM lane quadrant this warp may read
        int cbuf = 0;
        if (lane == 0) tc_prefetch_tmap(&map_c);
        GemmUnit u;
        for (int it = 0; gemm_unit<BN>(sc, blockIdx.x, gridDim.x, it, u); ++it) {
            const int acc = it & 1, accphase = (it >> 1) & 1;
            if (!tc_mbar_wait(&tfull[acc], accphase, abort_flag, st, 4)) break;
            tc_fence_after_sync();
            const uint32_t t0 = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
            gemm_store_rows(&map_c, a, sC + q * 8192, cbuf, t0, u.bn, u.tm * GEMM_BM + q * 32, u.n0, lane);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&tempty[acc]);
        }
        if (lane == 0) tc_bulk_wait_all();           // the tile stores have left shared memory and reached C
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc_tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ---- the same GEMM on CTA pairs -------------------------------------------------------------------
// Two CTAs of a cluster produce a 256 x 256 tile with one tcgen05.mma.cta_group::2 per K = 16: each
// CTA stages its own 128 rows of A and HALF of the tile's B columns, so a k-step costs a CTA 32 KB of
// shared-memory fill instead of 48 KB, six stages fit instead of four, and the loads in flight
// cover the L2 latency that bounded the single-CTA kernel.  Roles per CTA as above; only the
// leader's warp 1 issues MMAs.  Barriers: full[] of the leader collects the bytes of both CTAs'
// loads; empty[] and tfull[] exist in both CTAs and are signalled together by the leader's commit;
// tempty[] of the leader collects the arrivals of both CTAs' epilogue warps.
#define GEMM2_STAGES 6
#define GEMM2_BN 256
#define GEMM2_B_STAGE_BYTES (GEMM_BK * (GEMM2_BN / 2) * 2)
#define GEMM2_SMEM ((size_t)GEMM2_STAGES * (GEMM_A_STAGE_BYTES + GEMM2_B_STAGE_BYTES) + GEMM_EPI_BYTES + 1024 + 256)

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
ktb_gemm_f16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, const ktb_gemm_args a, const GemmSched sc, ktb_status* st) {
    constexpr int S = GEMM2_STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + (size_t)S * GEMM_A_STAGE_BYTES;
    uint8_t* sC = sB + (size_t)S * GEMM2_B_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sC + GEMM_EPI_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + S;
    uint64_t* tfull = bars + 2 * S;
    uint64_t* tempty = bars + 2 * S + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = (a.K + GEMM_BK - 1) / GEMM_BK;
    const uint32_t rank = tc_cluster_ctarank();

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            tc_mbar_init(&full[i], 1);
            tc_mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(&tfull[i], 1);
            tc_mbar_init(&tempty[i], 8);
        }
        *abort_flag = 0;
        tc_fence_barrier_init();
    }
    __syncthreads();
    if (warp == 1) tc_tmem_alloc_pair(tmem_slot, 2 * GEMM2_BN);
    tc_fence_before_sync();
    __syncthreads();
    tc_cluster_sync();                     // both CTAs' barriers exist before either is signalled from outside
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tc_prefetch_tmap(&map_a);
            tc_prefetch_tmap(&map_b);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            GemmUnit u;
            for (int it = 0; ok && gemm_unit<GEMM2_BN>(sc, blockIdx.x >> 1, gridDim.x >> 1, it, u); ++it) {
                const int bcols = u.bn / 2;                       // B columns this CTA stages
                for (int kt = 0; kt < KT; ++kt) {
                    if (!tc_mbar_wait(&empty[stage], phase ^ 1, abort_flag, st, 11)) { ok = false; break; }
                    if (rank == 0) tc_mbar_expect_tx(&full[stage], 2 * (GEMM_A_STAGE_BYTES + GEMM_BK * bcols * 2));
                    const uint32_t bar = tc_mapa(tc_smem_u32(&full[stage]), 0);
                    tc_tma_load_2d_pair(sA + (size_t)stage * GEMM_A_STAGE_BYTES, &map_a, bar, kt * GEMM_BK,
                                        u.tm * 2 * GEMM_BM + (int)rank * GEMM_BM);
#pragma unroll
                    for (int j = 0; j < GEMM2_BN / 128; ++j)
                        if (j * 64 < bcols)
                            tc_tma_load_2d_pair(sB + (size_t)stage * GEMM2_B_STAGE_BYTES + (size_t)j * (GEMM_BK * 128), &map_b,
                                                bar, u.n0 + (int)rank * bcols + j * 64, kt * GEMM_BK);
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            GemmUnit u;
            for (int it = 0; ok && gemm_unit<GEMM2_BN>(sc, blockIdx.x >> 1, gridDim.x >> 1, it, u); ++it) {
                const uint32_t idesc = tc_idesc_f16(2 * GEMM_BM, u.bn, 0, 1);
                const int acc = it & 1, accphase = (it >> 1) & 1;
                if (!tc_mbar_wait(&tempty[acc], accphase ^ 1, abort_flag, st, 12)) break;
                tc_fence_after_sync();
                const uint32_t d = tmem_base + acc * GEMM2_BN;
                for (int kt = 0; kt < KT; ++kt) {
                    if (!tc_mbar_wait(&full[stage], phase, abort_flag, st, 13)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = tc_smem_u32(sA + (size_t)stage * GEMM_A_STAGE_BYTES);
                    const uint32_t b_addr = tc_smem_u32(sB + (size_t)stage * GEMM2_B_STAGE_BYTES);
#pragma unroll
                    for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
                        const uint64_t ad = tc_smem_desc(a_addr + kk * 32, 16, 1024);
                        const uint64_t bd = tc_smem_desc(b_addr + kk * 2048, GEMM_BK * 128, 1024);
                        tc_mma_f16_pair(d, ad, bd, idesc, (kt | kk) != 0);
                    }
                    tc_mma_commit_pair(&empty[stage]);
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_mma_commit_pair(&tfull[acc]);
            }
        }
    } else {
        const int q = warp & 3;
        int cbuf = 0;
        if (lane == 0) tc_prefetch_tmap(&map_c);
        GemmUnit u;
        for (int it = 0; gemm_unit<GEMM2_BN>(sc, blockIdx.x >> 1, gridDim.x >> 1, it, u); ++it) {
            const int acc = it & 1, accphase = (it >> 1) & 1;
            if (!tc_mbar_wait(&tfull[acc], accphase, abort_flag, st, 14)) break;
            tc_fence_after_sync();
            const uint32_t t0 = tmem_base + acc * GEMM2_BN + ((uint32_t)(q * 32) << 16);
            gemm_store_rows(&map_c, a, sC + q * 8192, cbuf, t0, u.bn, u.tm * 2 * GEMM_BM + (int)rank * GEMM_BM + q * 32, u.n0,
                            lane);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive_cluster(tc_mapa(tc_smem_u32(&tempty[acc]), 0));
        }
        if (lane == 0) tc_bulk_wait_all();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_cluster_sync();                     // the peer may still read this CTA's shared memory or signal its barriers
    if (warp == 1) tc_tmem_dealloc_pair(tmem_base, 2 * GEMM2_BN);
}

template <int BN>
static int launch_gemm(ktb_ctx* ctx, const ktb_gemm_args& a, const CUtensorMap& ma, const CUtensorMap& mb,
                       const CUtensorMap& mc) {
    using Cfg = GemmCfg<BN>;
    static bool attr_set[KTB_MAX_DEVICES] = {};     // the attribute is per device
    if (!attr_set[ctx->device & (KTB_MAX_DEVICES - 1)]) {
        KTB_CUDA(ctx, cudaFuncSetAttribute(ktb_gemm_f16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)Cfg::SMEM));
        attr_set[ctx->device & (KTB_MAX_DEVICES - 1)] = true;
    }
    const int tiles_m = (a.M + GEMM_BM - 1) / GEMM_BM, tiles_n = (a.N + BN - 1) / BN;
    int grid = 0;
    const GemmSched sc = gemm_sched(tiles_m, tiles_n, ctx->sm_count, &grid);
    ktb_gemm_f16_kernel<BN><<<grid, GEMM_THREADS, Cfg::SMEM, ctx->stream>>>(ma, mb, mc, a, sc, ctx->dev_status);
    KTB_CHECK_LAUNCH(ctx, "ktb_gemm_f16_kernel");
    return KTB_OK;
}

static int launch_gemm_pair(ktb_ctx* ctx, const ktb_gemm_args& a, const CUtensorMap& ma, const CUtensorMap& mb,
                            const CUtensorMap& mc) {
    static bool attr_set[KTB_MAX_DEVICES] = {};
    if (!attr_set[ctx->device & (KTB_MAX_DEVICES - 1)]) {
        KTB_CUDA(ctx, cudaFuncSetAttribute(ktb_gemm_f16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)GEMM2_SMEM));
        attr_set[ctx->device & (KTB_MAX_DEVICES - 1)] = true;
    }
    const int tiles_m = (a.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM), tiles_n = (a.N + GEMM2_BN - 1) / GEMM2_BN;
    int clusters = 0;
    const GemmSched sc = gemm_sched(tiles_m, tiles_n, ctx->sm_count / 2, &clusters);
    ktb_gemm_f16_pair_kernel<<<2 * clusters, GEMM_THREADS, GEMM2_SMEM, ctx->stream>>>(ma, mb, mc, a, sc, ctx->dev_status);
    KTB_CHECK_LAUNCH(ctx, "ktb_gemm_f16_pair_kernel");
    return KTB_OK;
}

extern "C" int ktb_launch_gemm_f16(ktb_ctx* ctx, const ktb_gemm_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    const ktb_gemm_args& a = *args;
    if (a.M <= 0 || a.N <= 0 || a.K <= 0) return KTB_OK;
    if (a.c_dtype != KTB_F16 && a.c_dtype != KTB_F32) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "gemm_f16", "C must be f16 or f32");
    if ((a.N % 32) || (a.K % 8) || (a.lda % 8) || (a.ldb % 8) || (a.ldc % 8) || (a.a_off % 8) || (a.b_off % 8) || (a.c_off % 8))
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "gemm_f16", "N must be a multiple of 32; K, leading dims and offsets multiples of 8");
    CUtensorMap ma, mb, mc;
    __half* base = reinterpret_cast<__half*>(a.arena);
    {
        const uint64_t dims[2] = {(uint64_t)a.K, (uint64_t)a.M};
        const uint64_t str[1] = {(uint64_t)a.lda * 2};
        const uint32_t box[2] = {GEMM_BK, GEMM_BM};
        if (!tc_make_map_f16(&ma, base + a.a_off, 2, dims, str, box)) return ktb_fail(ctx, KTB_E_CUDA, "gemm_f16", "cuTensorMapEncodeTiled(A) failed");
    }
    {
        const uint64_t dims[2] = {(uint64_t)a.N, (uint64_t)a.K};
        const uint64_t str[1] = {(uint64_t)a.ldb * 2};
        const uint32_t box[2] = {64, GEMM_BK};
        if (!tc_make_map_f16(&mb, base + a.b_off, 2, dims, str, box)) return ktb_fail(ctx, KTB_E_CUDA, "gemm_f16", "cuTensorMapEncodeTiled(B) failed");
    }
    {
        // C as the epilogue stores it: 32 rows x 128 bytes per tile store
        const bool f16 = a.c_dtype == KTB_F16;
        const uint64_t dims[2] = {(uint64_t)a.N, (uint64_t)a.M};
        const uint64_t str[1] = {(uint64_t)a.ldc * (f16 ? 2 : 4)};
        const uint32_t box[2] = {f16 ? 64u : 32u, 32u};
        void* cbase = f16 ? (void*)(base + a.c_off) : (void*)(reinterpret_cast<float*>(a.arena) + a.c_off);
        if (!tc_make_map(&mc, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, cbase, 2, dims, str, box))
            return ktb_fail(ctx, KTB_E_CUDA, "gemm_f16", "cuTensorMapEncodeTiled(C) failed");
    }
    const int row_tiles = (a.M + GEMM_BM - 1) / GEMM_BM;
    if (a.N % 256 == 0 || a.N >= 1024) {
        // CTA pairs work on 256 rows: not for a single row tile, nor where an odd count would idle much of a pair
        if (row_tiles >= 2 && (row_tiles % 2 == 0 || row_tiles >= 9) && ctx->sm_count >= 2)
            return launch_gemm_pair(ctx, a, ma, mb, mc);
        return launch_gemm<256>(ctx, a, ma, mb, mc);
    }
    return launch_gemm<128>(ctx, a, ma, mb, mc);
}
