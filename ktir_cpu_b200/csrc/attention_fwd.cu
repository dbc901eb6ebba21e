// Causal attention forward with online softmax and paged K/V, head_dim 128.
//
// A persistent CTA (one per SM) works through pairs of 128-row query tiles of one head, one pair
// at a time, and walks the KV pages that the causal mask leaves visible.  It replaces the per-page op sequence of a KTIR attention kernel —
// indirect ktdp.load of a K and a V page through the block table, two linalg.matmul,
// mask / max / exp / sum / rescale in f32 — which the reference dispatches op by op
// (examples/triton-ktir/paged_attention.mlir:183-396, ktir_cpu/ops/memory_ops.py:867-915,
// ktir_cpu/dialects/linalg_ops.py:136-347).
//
// Roles: warp 0 streams the Q tiles of a pair once and the K/V pages (page id from the block table)
// through a shared-memory ring by TMA; warps 1 and 2 issue tcgen05.mma for tile 0 and tile 1 —
// S_i = Q_i K^T into a score slot of tile i, P_i V accumulated into the output buffer of tile i,
// both in TMEM; warps 4-7 are the softmax of tile 0, warps 8-11 of tile 1, one thread per query
// row (two with TPR = 2): read the scores from TMEM, mask, running max, P = exp2(..) rounded to
// f16 and written back to TMEM over the scores it came from, row sum in f32.  P V takes its A
// operand straight from TMEM, so shared memory carries only Q, K and V.
//
// A page is walked in steps of 64 kv rows, and every tile has two score slots of 64 TMEM columns:
// while the softmax works on step u the tensor core already holds the scores of step u+1, so in
// the steady state the softmax never waits for a matmul and the tensor core never for a softmax.
//
// The output accumulator never leaves TMEM until the end.  The reference rescales it by
// exp(m_old - m_new) after every page (paged_attention.mlir:330-372); here the exponent
// reference m_ref of a row is only moved when the row maximum has grown by more than 2^8 since
// it was set (then O and l are rescaled once, by the row's own threads, through tcgen05.ld/st).
// P = exp2(s - m_ref) may therefore exceed 1 by at most 2^8, well inside f16 range; the
// normalised result sum(P V) / sum(P) is the same number, only the rounding of P to f16 sees a
// different exponent.  Scores, max, sum and accumulator are f32 as in the reference; P is
// rounded to f16 before the second matmul (relative error <= 2^-11).  All waits are bounded.
#include "tc_common.cuh"

#define AT_BM 128
#define AT_D 128
#define AT_Q_BYTES (AT_BM * AT_D * 2)
#define AT_MAX_STAGES 8
#define AT_RESCALE_GAP 8.0f

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

static __device__ __forceinline__ float at_max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// two f32 lanes in one 64-bit register: Blackwell issues fma / add on such pairs as one instruction
static __device__ __forceinline__ uint64_t at_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
static __device__ __forceinline__ void at_unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
static __device__ __forceinline__ uint64_t at_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
static __device__ __forceinline__ uint64_t at_add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// 2^x for two values at once on the FMA pipe (the exp unit is the busiest unit of the softmax):
// x = r + f with r = round(x), 2^f by a cubic on [-0.5, 0.5] (relative error 7.5e-5, a sixth of
// an f16 ulp), 2^r by an add into the exponent field.  x is clamped to >= -125 so that the
// exponent stays positive (such a term is zero in f16 either way).
static __device__ __forceinline__ void at_ex2_poly2(float x0, float x1, float& p0, float& p1) {
    const float magic = 12582912.f;                     // 1.5 * 2^23: the sum keeps round(x) in the low mantissa bits
    const uint64_t x2 = at_pack2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
    const uint64_t t2 = at_add2(x2, at_pack2(magic, magic));
    const uint64_t r2 = at_add2(t2, at_pack2(-magic, -magic));
    const uint64_t f2 = at_fma2(r2, at_pack2(-1.f, -1.f), x2);
    uint64_t q2 = at_fma2(at_pack2(0.05517164617776871f, 0.05517164617776871f), f2,
                          at_pack2(0.2426111251115799f, 0.2426111251115799f));
    q2 = at_fma2(q2, f2, at_pack2(0.6932609677314758f, 0.6932609677314758f));
    q2 = at_fma2(q2, f2, at_pack2(0.9999280571937561f, 0.9999280571937561f));
    float q0, q1, t0, t1;
    at_unpack2(q2, q0, q1);
    at_unpack2(t2, t0, t1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

// Maximum of CW raw scores.
template <int CW>
static __device__ __forceinline__ float at_chunk_max(const uint32_t (&v)[CW], float mx) {
    if (CW % 8 == 0) {                 // four independent chains: the latency of max is not hidden otherwise
        float m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < CW; i += 8) {
            mx = at_max3(mx, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
            m1 = at_max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            m2 = at_max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
            m3 = at_max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
        }
        return at_max3(mx, m1, fmaxf(m2, m3));
    }
#pragma unroll
    for (int i = 0; i < CW; i += 2) mx = at_max3(mx, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
    return mx;
}

// P = exp2(s * sl - m) for CW scores -> CW/2 packed f16 pairs; the f32 values are added to acc2.
// POLY of every 4 pairs take the polynomial instead of the exp unit.  A score of -inf (a masked
// column) gives 0 on either path (the polynomial clamps it to 2^-125, which is 0 in f16 and
// vanishes in the sum).
template <int CW, int POLY>
static __device__ __forceinline__ void at_chunk_prob(const uint32_t (&v)[CW], float sl, float m, uint64_t& acc2,
                                                     uint32_t (&packed)[CW / 2]) {
    const uint64_t sl2 = at_pack2(sl, sl), nm2 = at_pack2(-m, -m);
#pragma unroll
    for (int i = 0; i < CW; i += 2) {
        float x0, x1;
        at_unpack2(at_fma2(at_pack2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sl2, nm2), x0, x1);
        float p0, p1;
        if (((i >> 1) & 3) < POLY) {
            at_ex2_poly2(x0, x1, p0, p1);
        } else {
            p0 = at_ex2(x0);
            p1 = at_ex2(x1);
        }
        acc2 = at_add2(acc2, at_pack2(p0, p1));
        const __half2 h = __floats2half2_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
    }
}

// S-full and P-full barriers exist per tile and score slot (index tile * 2 + slot)
// cycles the softmax of tile 1 starts behind that of tile 0, so that the two do not need the exp
// unit (and the tensor core) at the same moments
#define AT_STAGGER 800
// barriers: Q full / free per tile; S-full and P-full per tile and score slot (index tile * 2 + slot)
enum { B_QFULL = 0, B_QFREE = 2, B_KVFULL = 4, B_KVEMPTY = B_KVFULL + AT_MAX_STAGES, B_SFULL = B_KVEMPTY + AT_MAX_STAGES,
       B_PFULL = B_SFULL + 4, B_PVDONE = B_PFULL + 4, B_OFINAL = B_PVDONE + 2, B_XCHG = B_OFINAL + 2, B_COUNT = B_XCHG + 2 };

// TPR = threads per query row in the softmax (1: a thread holds the whole score row of a step in
// registers, 384 threads; 2: two threads share a row, 640 threads).
//
// The kernel is persistent: CTA b walks the work items b, b + gridDim.x, ...  An item is the pair of
// query-tile pairs (q_pairs - 1 - r, r) of one head — a late pair, which sees many KV pages, and its
// early complement, so that all items cost the same — and the two halves are processed one after
// the other as "sub-items".  Every role (copy thread, the two issuing warps, the softmax warps)
// derives the same sequence on its own; barrier phases simply keep counting across sub-items.  The
// point of it: the Q tiles and first K/V pages of the next sub-item are fetched while the last steps
// of the current one run, and its first scores are computed while the softmax warps normalise and
// store the output, so a tile pair no longer pays a start-up and a drain of its own.
template <int BN, int TPR, int POLY>
__global__ void __launch_bounds__(128 + 256 * TPR, 1)
ktb_attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const ktb_attn_args a, int q_pairs,
                         int n_items, ktb_status* st) {
    constexpr int KV_BYTES = BN * AT_D * 2;            // one K or V page in shared memory
    constexpr int AT_STAGES = BN == 128 ? 4 : 8;       // ring slots: 128 KB (64 KB for 32-row pages)
    constexpr int KV_BLK = BN * 128;                   // bytes of one [BN x 64] block
    constexpr int SB = BN > 64 ? 64 : BN;              // kv rows of one step (a page is NSUB steps)
    constexpr int NSUB = BN / SB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;                                // 2 tiles x 2 blocks [128 x 64]
    uint8_t* sKV = sQ + 2 * AT_Q_BYTES;                // ring of K / V pages
    float* xbuf = reinterpret_cast<float*>(sKV + AT_STAGES * KV_BYTES);   // [2 tiles][2 parities][2 halves][128 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(xbuf + 2 * 2 * 2 * AT_BM);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    // (through a shuffle, so that the compiler knows the warp index is the same in all lanes)
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
    const int half_pairs = (q_pairs + 1) / 2;          // items per head

    // Sub-item s of this CTA: false when the CTA has run out of items.  n_of[i] = steps (SB kv rows each)
    // tile i can see (kv position p is visible to row R iff p <= R + delta), 0 for a tile that does
    // not exist; nmax = pages to stream.  An item whose two halves coincide has an empty second half.
    auto sub_item = [&](int s, int& head, int& q0, int (&n_of)[2], int& nmax) -> bool {
        const long long item64 = (long long)blockIdx.x + (long long)(s >> 1) * gridDim.x;
        if (item64 >= n_items) return false;
        const int item = (int)item64;
        head = item / half_pairs;
        const int r = item % half_pairs;
        const int qp = (s & 1) ? r : q_pairs - 1 - r;
        q0 = qp * 2 * AT_BM;
        const bool empty = (s & 1) && r == q_pairs - 1 - r;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            int n = a.num_tiles * NSUB;
            const long long last = (long long)q0 + i * AT_BM + AT_BM - 1 + a.causal_delta;
            const long long vis = last < 0 ? 0 : last / SB + 1;
            if (a.causal && vis < n) n = (int)vis;
            if (q0 + i * AT_BM >= a.seq_q) n = 0;      // no second tile in the last pair of an odd count
            n_of[i] = empty ? 0 : n;
        }
        nmax = ((n_of[0] > n_of[1] ? n_of[0] : n_of[1]) + NSUB - 1) / NSUB;
        return true;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(&bars[B_QFULL + i], 1);
            tc_mbar_init(&bars[B_QFREE + i], 1);
        }
        for (int i = 0; i < AT_STAGES; ++i) {
            tc_mbar_init(&bars[B_KVFULL + i], 1);
            tc_mbar_init(&bars[B_KVEMPTY + i], 2);      // both issuing threads
        }
        for (int i = 0; i < 4; ++i) {
            tc_mbar_init(&bars[B_SFULL + i], 1);
            tc_mbar_init(&bars[B_PFULL + i], 4 * TPR);
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(&bars[B_PVDONE + i], 1);
            tc_mbar_init(&bars[B_OFINAL + i], 1);
            tc_mbar_init(&bars[B_XCHG + i], 8);
        }
        *abort_flag = 0;
        tc_fence_barrier_init();
    }
    __syncthreads();
    if (warp == 1) tc_tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    const uint32_t tmem_s = tmem_base;            // per tile two score slots of 64 columns: 2 x 128 columns
    const uint32_t tmem_o = tmem_base + 256;      // O_0, O_1: 2 x 128 columns

    // register budget: the copy/MMA warpgroup needs few registers, the softmax warpgroups hold a
    // row of scores each; the MMA issue loop must not spill, it paces the whole CTA
    // (each setmaxnreg sits at the head of the region it governs, with no join in between)
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");          // (a decrease only for TPR = 1, see below)
    if (warp == 0) {
        if (lane == 0) {
            tc_prefetch_tmap(&map_q);
            tc_prefetch_tmap(&map_k);
            tc_prefetch_tmap(&map_v);
            const int32_t* bt32 = reinterpret_cast<const int32_t*>(a.arena) + a.bt_off;
            const int64_t* bt64 = reinterpret_cast<const int64_t*>(a.arena) + a.bt_off;
            int t = 0;                  // ring loads issued so far: K of a page, then its V; slot t % AT_STAGES
            int q_loads[2] = {0, 0};    // Q tiles loaded so far, per tile
            const int kv_group = a.kv_group > 1 ? a.kv_group : 1;
            bool ok = true;
            for (int s = 0; ok; ++s) {
                int head, q0, n_of[2], nmax;
                if (!sub_item(s, head, q0, n_of, nmax)) break;
                const int kv_head = head / kv_group;   // grouped-query attention: kv_group query heads per K/V head
                for (int i = 0; i < 2 && ok; ++i) {
                    if (n_of[i] == 0) continue;
                    // the tile's Q buffer is free once the last score MMA of its previous sub-item has completed
                    if (q_loads[i] > 0) ok = tc_mbar_wait(&bars[B_QFREE + i], (q_loads[i] - 1) & 1, abort_flag, st, 12);
                    if (!ok) break;
                    ++q_loads[i];
                    tc_mbar_expect_tx(&bars[B_QFULL + i], AT_Q_BYTES);
                    tc_tma_load_3d(sQ + i * AT_Q_BYTES, &map_q, &bars[B_QFULL + i], 0, head, q0 + i * AT_BM);
                    tc_tma_load_3d(sQ + i * AT_Q_BYTES + AT_BM * 128, &map_q, &bars[B_QFULL + i], 64, head, q0 + i * AT_BM);
                }
                for (int l = 0; l < 2 * nmax && ok; ++l, ++t) {
                    const int slot = t % AT_STAGES;
                    const int j = l >> 1;
                    long long page = a.bt_dtype == KTB_I64 ? bt64[j] : (long long)bt32[j];
                    if (page < 0) {
                        if (atomicExch(&st->negative_index, 1) == 0) st->bad_index_value = (int32_t)page;
                        page = 0;
                    }
                    if (!tc_mbar_wait(&bars[B_KVEMPTY + slot], ((t / AT_STAGES) & 1) ^ 1, abort_flag, st, 11)) {
                        ok = false;
                        break;
                    }
                    tc_mbar_expect_tx(&bars[B_KVFULL + slot], KV_BYTES);
                    const CUtensorMap* map = (l & 1) ? &map_v : &map_k;
                    at_tma_load_4d(sKV + slot * KV_BYTES, map, &bars[B_KVFULL + slot], 0, kv_head, 0, (int)page);
                    at_tma_load_4d(sKV + slot * KV_BYTES + KV_BLK, map, &bars[B_KVFULL + slot], 64, kv_head, 0, (int)page);
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // One issuing warp per query tile (warps 1 and 2 sit on different schedulers); the warp runs
        // this code converged and one elected lane executes the tcgen05 instructions.
        // Steps of a tile are numbered g = 0, 1, ... across sub-items.  The scores of step g go to slot
        // g & 1 of the tile, and P(g) is written over the front of the same slot; so S(g+2) is issued
        // right after P V(g) (the tensor core runs one thread's MMAs in issue order), and the scores
        // of step g+1 are already waiting when the softmax finishes step g.  P V(g) needs P(g) in TMEM
        // and the V page in shared memory, S(g) the K page and the tile's Q.  Both issuers release
        // every slot of the ring (two arrivals per slot and round): a tile that sees fewer pages
        // follows the remaining ones along without issuing anything.
        {
            const uint32_t lead = tc_elect_one();
            const int i = warp - 1;
            const uint32_t idesc_s = tc_idesc_f16(AT_BM, SB, 0, 0);
            const uint32_t idesc_pv = tc_idesc_f16(AT_BM, AT_D, 0, 1);
            const uint32_t ts = tmem_s + i * 128, to = tmem_o + i * 128;
            const uint64_t qd0 = tc_smem_desc(tc_smem_u32(sQ + i * AT_Q_BYTES), 16, 1024);
            const uint32_t kv_addr0 = tc_smem_u32(sKV);
            int t0 = 0;                 // ring loads before this sub-item (load t0 + 2 m is K of page m, t0 + 2 m + 1 its V)
            int g0 = 0;                 // steps of this tile before this sub-item
            int q_uses = 0;             // Q tiles consumed so far
            int n = 0;
            auto kv_wait = [&](int t) {
                return __all_sync(0xffffffffu, tc_mbar_wait(&bars[B_KVFULL + t % AT_STAGES], (t / AT_STAGES) & 1, abort_flag, st, 22)) != 0;
            };
            auto kv_release = [&](int t) { tc_mma_commit_p(&bars[B_KVEMPTY + t % AT_STAGES], lead); };
            // Operands of a step are computed ahead of the wait that gates it.
            // step u = rows [h * SB, h * SB + SB) of page m; 64 rows of a block are whole swizzle atoms.
            auto s_desc = [&](int u) {
                const int m = u / NSUB, h = u % NSUB;
                return tc_smem_desc(kv_addr0 + ((t0 + 2 * m) % AT_STAGES) * KV_BYTES + h * SB * 128, 16, 1024);
            };
            auto pv_desc = [&](int u) {
                const int m = u / NSUB, h = u % NSUB;
                return tc_smem_desc(kv_addr0 + ((t0 + 2 * m + 1) % AT_STAGES) * KV_BYTES, KV_BLK, 1024) +
                       (uint32_t)(h * (SB / 16) * 2048 >> 4);
            };
            auto issue_s = [&](int u, uint64_t bd0) {
                // the start-address field is the low 14 bits of the descriptor (in 16-byte units), so
                // stepping along K is an add of a constant; the loop is unrolled
                const int g = g0 + u;
                const uint32_t d = ts + (g & 1) * 64;
#pragma unroll
                for (int kk = 0; kk < AT_D / 16; ++kk) {
                    const uint32_t ao = ((kk >> 2) * (AT_BM * 128) + (kk & 3) * 32) >> 4;
                    const uint32_t bo = ((kk >> 2) * KV_BLK + (kk & 3) * 32) >> 4;
                    tc_mma_f16_p(d, qd0 + ao, bd0 + bo, idesc_s, kk != 0, lead);
                }
                tc_mma_commit_p(&bars[B_SFULL + i * 2 + (g & 1)], lead);
                if (u == n - 1) tc_mma_commit_p(&bars[B_QFREE + i], lead);       // last use of this Q tile
                if (u % NSUB == NSUB - 1 || u == n - 1) kv_release(t0 + 2 * (u / NSUB));
            };
            auto issue_pv = [&](int u, uint64_t bd0) {
                // A = P from TMEM: row r in lane r, 16 f16 of a K step packed in 8 columns
                const int g = g0 + u;
                const uint32_t pa = ts + (g & 1) * 64;
#pragma unroll
                for (int kk = 0; kk < SB / 16; ++kk)
                    tc_mma_f16_ts_p(to, pa + kk * 8, bd0 + (uint32_t)(kk * 2048 >> 4), idesc_pv, (u > 0 || kk > 0) ? 1u : 0u, lead);
                tc_mma_commit_p(&bars[B_PVDONE + i], lead);
                if (u == n - 1) tc_mma_commit_p(&bars[B_OFINAL + i], lead);      // the accumulator is final
                if (u % NSUB == NSUB - 1 || u == n - 1) kv_release(t0 + 2 * (u / NSUB) + 1);
            };
            bool ok = true;
            for (int s = 0; ok; ++s) {
                int head, q0, n_of[2], nmax;
                if (!sub_item(s, head, q0, n_of, nmax)) break;
                n = n_of[i];
                if (n > 0) {
                    ok = __all_sync(0xffffffffu, tc_mbar_wait(&bars[B_QFULL + i], q_uses & 1, abort_flag, st, 21)) != 0;
                    ++q_uses;
                    if (ok) tc_fence_after_sync();
                    // the first P V of a sub-item overwrites the accumulator; that the softmax warps have
                    // read the previous result out is implied by their P(0) arriving (program order there)
                    for (int u = 0; u < 2 && u < n && ok; ++u) {
                        if (u % NSUB == 0) ok = kv_wait(t0 + 2 * (u / NSUB));
                        if (ok) {
                            tc_fence_after_sync();
                            issue_s(u, s_desc(u));
                        }
                    }
                    for (int u = 0; u < n && ok; ++u) {
                        const int g = g0 + u;
                        const uint64_t vd = pv_desc(u), kd = s_desc(u + 2);
                        ok = __all_sync(0xffffffffu, tc_mbar_wait(&bars[B_PFULL + i * 2 + (g & 1)], (g >> 1) & 1, abort_flag, st, 23)) != 0;
                        if (ok && u % NSUB == 0) ok = kv_wait(t0 + 2 * (u / NSUB) + 1);
                        if (!ok) break;
                        tc_fence_after_sync();
                        issue_pv(u, vd);
                        if (u + 2 < n) {
                            if ((u + 2) % NSUB == 0) ok = kv_wait(t0 + 2 * ((u + 2) / NSUB));
                            if (!ok) break;
                            tc_fence_after_sync();
                            issue_s(u + 2, kd);
                        }
                    }
                }
                // pages only the other tile uses: keep the ring's arrival counts in step
                for (int m = (n + NSUB - 1) / NSUB; m < nmax && ok; ++m) {
                    for (int t = t0 + 2 * m; t < t0 + 2 * m + 2 && ok; ++t) {
                        ok = kv_wait(t);
                        if (ok && lead) tc_mbar_arrive(&bars[B_KVEMPTY + t % AT_STAGES]);
                    }
                }
                t0 += 2 * nmax;
                g0 += n;
            }
        }
    }
    } else {
        // TPR = 2: the softmax warpgroups keep the launch allocation of 96 registers.  TPR = 1: 384 threads
        // start with 168 each; the copy/MMA warpgroup gave back 80, the two softmax warpgroups take 40 more
        if (TPR == 1) asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        // Two threads share a query row: `half` 0 owns the first BN/2 score columns and the first 64
        // output columns, `half` 1 the rest.  Their row maxima (and, at the end, row sums) are swapped
        // through shared memory.
        constexpr int HB = SB / TPR;                 // score columns per thread
        constexpr int CW = HB < 32 ? HB : 32;        // columns per TMEM load
        constexpr int NCH = HB / CW;
        constexpr int OH = AT_D / TPR;               // output columns per thread
        const int tile = (warp - 4) / (4 * TPR);     // which query tile this warpgroup (pair) owns
        const int half = TPR == 2 ? ((warp - 4) >> 2) & 1 : 0;
        const int q = warp & 3;                      // TMEM lane quadrant this warp may access
        const int r = q * 32 + lane;                 // row inside the tile == TMEM lane
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        const uint32_t s_addr = tmem_s + tile * 128 + lane_off + half * HB;
        // P (f16, two per 32-bit column) goes over the first SB/2 columns of the score slot
        const uint32_t p_addr = tmem_s + tile * 128 + lane_off + half * (HB / 2);
        const uint32_t o_addr = tmem_o + tile * 128 + lane_off + half * OH;
        float* xrow = xbuf + tile * (2 * 2 * AT_BM) + r;        // + parity * 256 + half * 128
        const float sl = a.scale * 1.4426950408889634f;
        bool ok = true;
        uint32_t xphase = 0;
        int g0 = 0;                  // steps of this tile before the current sub-item
        int finals = 0;              // sub-items of this tile finished so far

        // swap one f32 with the partner thread of the row (slot parity alternates, so a value is
        // not overwritten before the partner has read it)
        auto swap_with_partner = [&](float mine, float& theirs) -> bool {
            float* slot = xrow + (xphase & 1) * (2 * AT_BM);
            slot[half * AT_BM] = mine;
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&bars[B_XCHG + tile]);        // release: orders the stores above
            const bool w = tc_mbar_wait(&bars[B_XCHG + tile], xphase & 1, abort_flag, st, 34);
            ++xphase;
            if (!__all_sync(0xffffffffu, w)) return false;
            theirs = slot[(half ^ 1) * AT_BM];
            return true;
        };

        for (int s = 0; ok; ++s) {
        int head, q0, n_of[2], nmax;
        if (!sub_item(s, head, q0, n_of, nmax)) break;
        const int n = n_of[tile];
        if (n == 0) continue;
        const int R = q0 + tile * AT_BM + r;
        float m_ref = a.m_init * 1.4426950408889634f;           // exponent reference, log2 domain
        float m_run = m_ref;                                    // true running maximum
        float l_run = half == 0 ? a.l_init : 0.f;               // this thread's share of the running sum
        const long long limit = (long long)R + a.causal_delta;  // last visible kv position
        const long long tile_limit = (long long)q0 + tile * AT_BM + a.causal_delta;
        // first step with a hidden column for some row of the tile: (j + 1) * SB - 1 > tile_limit
        // (kept as one int so that the common, unmasked step pays one compare for the mask)
        int j_mask = 0x7fffffff;
        if (a.causal) {
            const long long jm = tile_limit + 1 >= 0 ? (tile_limit + 1) / SB : 0;
            j_mask = jm > 0x7fffffff ? 0x7fffffff : (int)jm;
        }
        for (int j = 0; j < n && ok; ++j) {            // j counts steps of SB kv rows
            const int g = g0 + j;                      // step number of the tile across sub-items
            const uint32_t slot_off = (g & 1) * 64;
            // the whole warp leaves together: the TMEM accesses below are warp-collective.
            // S(g) is issued after P V(g-2), which read the P columns of this slot.
            if (!__all_sync(0xffffffffu, tc_mbar_wait(&bars[B_SFULL + tile * 2 + (g & 1)], (g >> 1) & 1, abort_flag, st, 31))) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            if (g == 0 && tile == 1) {
                const long long t0 = clock64();
                while (clock64() - t0 < AT_STAGGER) {}
            }
            // this thread's part of the score row moves to registers in one go
            uint32_t v[NCH][CW];
#pragma unroll
            for (int c = 0; c < NCH; ++c) tc_tmem_ld<CW>(s_addr + slot_off + c * CW, v[c]);
            tc_tmem_ld_wait();

            // columns of this thread's range the row may see (all of them except on the diagonal pages)
            const bool need_mask = j >= j_mask;          // same for the whole tile
            // hidden columns become -inf once (exp2 turns them into zeros), then every step takes the same path
            if (need_mask) {
                const long long vis_ll = limit - ((long long)j * SB + half * HB) + 1;
                const int vis = vis_ll > HB ? HB : (vis_ll < 0 ? 0 : (int)vis_ll);
#pragma unroll
                for (int c = 0; c < NCH; ++c)
#pragma unroll
                    for (int i = 0; i < CW; ++i)
                        if (c * CW + i >= vis) v[c][i] = 0xff800000u;
            }
            // row maximum of the raw scores (the scale is positive, so it commutes with max)
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < NCH; ++c) mx = at_chunk_max<CW>(v[c], mx);
            float mx_other = mx;
            // after the swap both threads of the row have their scores in registers: P may go over them
            if (TPR == 2 && !swap_with_partner(mx, mx_other)) { ok = false; break; }
            m_run = fmaxf(m_run, fmaxf(mx, mx_other) * sl);
            // move the exponent reference only when the maximum has outgrown it by 2^8
            // (m_run and m_ref are the same on both threads of a row, so they move together)
            const bool move = m_run > m_ref + AT_RESCALE_GAP;
            if (__any_sync(0xffffffffu, move)) {
                const float alpha = move ? at_ex2(m_ref - m_run) : 1.0f;
                if (move) m_ref = m_run;
                l_run *= alpha;
                if (j > 0) {
                    // the accumulator may only be touched once P V(g-1) has completed; P V(g-2) completed
                    // before S(g), so the barrier is in phase g-1 or has just completed it
                    if (!__all_sync(0xffffffffu, tc_mbar_wait(&bars[B_PVDONE + tile], (g - 1) & 1, abort_flag, st, 32))) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll 1
                    for (int c0 = 0; c0 < OH; c0 += 16) {
                        uint32_t o[16];
                        tc_tmem_ld16(o_addr + c0, o);
                        tc_tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tc_tmem_st16(o_addr + c0, o);
                    }
                }
            }
            // P = exp2(s * sl - m_ref) -> f16 pairs -> TMEM (a row that has seen nothing yet keeps zeros, not NaN)
            const float m_exp = m_ref == -INFINITY ? 0.f : m_ref;
            uint64_t acc2 = at_pack2(0.f, 0.f);
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                uint32_t packed[CW / 2];
                at_chunk_prob<CW, POLY>(v[c], sl, m_exp, acc2, packed);
                tc_tmem_st<CW / 2>(p_addr + slot_off + c * (CW / 2), packed);
            }
            float s0, s1;
            at_unpack2(acc2, s0, s1);
            l_run += s0 + s1;
            tc_tmem_st_wait();
            tc_fence_before_sync();          // P (and O) stores of this thread are complete
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&bars[B_PFULL + tile * 2 + (g & 1)]);
        }
        g0 += n;
        if (ok && !__all_sync(0xffffffffu, tc_mbar_wait(&bars[B_OFINAL + tile], finals & 1, abort_flag, st, 33))) ok = false;
        ++finals;
        if (ok) {
            tc_fence_after_sync();
            // total row sum = the two partial sums (same rescaling history on both threads)
            float l_other = 0.f;
            if (TPR == 1 || swap_with_partner(l_run, l_other)) {
                const float inv = 1.0f / (l_run + l_other);
                const bool store = *abort_flag == 0 && R < a.seq_q;
                __half* dst = reinterpret_cast<__half*>(a.arena) + a.o_off + (int64_t)R * a.o_row_stride +
                              (int64_t)head * a.o_head_stride + half * OH;
#pragma unroll
                for (int c0 = 0; c0 < OH; c0 += 32) {
                    uint32_t o[32];
                    tc_tmem_ld32(o_addr + c0, o);
                    tc_tmem_ld_wait();
                    if (store) {
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint4 w;
                            __half2* h = reinterpret_cast<__half2*>(&w);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                h[i] = __floats2half2_rn(__uint_as_float(o[c + 2 * i]) * inv,
                                                         __uint_as_float(o[c + 2 * i + 1]) * inv);
                            *reinterpret_cast<uint4*>(dst + c0 + c) = w;
                        }
                    }
                }
            }
        }
        }   // sub-items
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc_tmem_dealloc(tmem_base, 512);
}

template <int BN, int TPR, int POLY = 0>
static int launch_attn(ktb_ctx* ctx, const ktb_attn_args& a, const CUtensorMap& mq, const CUtensorMap& mk,
                       const CUtensorMap& mv) {
    constexpr int AT_STAGES = BN == 128 ? 4 : 8;
    constexpr size_t SMEM = 2 * AT_Q_BYTES + AT_STAGES * (size_t)(BN * AT_D * 2) + 2 * 2 * 2 * AT_BM * 4 + 1024 + 512;
    static bool attr_set[KTB_MAX_DEVICES] = {};     // the attribute is per device
    if (!attr_set[ctx->device & (KTB_MAX_DEVICES - 1)]) {
        KTB_CUDA(ctx, cudaFuncSetAttribute(ktb_attention_fwd_kernel<BN, TPR, POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        attr_set[ctx->device & (KTB_MAX_DEVICES - 1)] = true;
    }
    const int q_pairs = (a.seq_q + 2 * AT_BM - 1) / (2 * AT_BM);
    // an item = the tile pairs (q_pairs - 1 - r, r) of one head; one persistent CTA per SM walks them
    const long long items = (long long)((q_pairs + 1) / 2) * a.heads;
    if (items > 0x7fffffff) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "attention_fwd", "too many query tiles");
    const int grid = items < ctx->sm_count ? (int)items : ctx->sm_count;
    ktb_attention_fwd_kernel<BN, TPR, POLY><<<grid, 128 + 256 * TPR, SMEM, ctx->stream>>>(mq, mk, mv, a, q_pairs, (int)items, ctx->dev_status);
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
    if (!(a.scale > 0.f)) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "attention_fwd", "score scale must be positive");
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
        const int kvg = a.kv_group > 1 ? a.kv_group : 1;
        const uint64_t dims[4] = {AT_D, (uint64_t)((a.heads + kvg - 1) / kvg), (uint64_t)a.page, (uint64_t)a.n_pages_total};
        const uint64_t str[3] = {(uint64_t)a.kv_head_stride * 2, (uint64_t)a.kv_row_stride * 2, (uint64_t)a.kv_page_stride * 2};
        const uint32_t box[4] = {64, 1, (uint32_t)a.page, 1};
        if (!tc_make_map_f16(which ? &mv : &mk, base + (which ? a.v_off : a.k_off), 4, dims, str, box))
            return ktb_fail(ctx, KTB_E_CUDA, "attention_fwd", "cuTensorMapEncodeTiled(K/V) failed");
    }
    switch (a.page) {
        case 32: return launch_attn<32, 2>(ctx, a, mq, mk, mv);      // two softmax threads per row: a step is only 32 columns
        case 64: return launch_attn<64, 1, 1>(ctx, a, mq, mk, mv);
        default: return launch_attn<128, 1, 1>(ctx, a, mq, mk, mv);
    }
}
