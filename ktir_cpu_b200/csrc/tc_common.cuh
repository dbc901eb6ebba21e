// Blackwell (sm_100a) primitives used by the tensor-core kernels: mbarrier, TMA
// (cp.async.bulk.tensor, no multicast), tcgen05 MMA / TMEM, all as inline PTX.
// Every wait is bounded: a wait that runs out records its site in the status word
// and raises a CTA-wide abort flag so the kernel drains and returns.
#pragma once
#include <cuda.h>

#include "common.cuh"

static __device__ __forceinline__ uint32_t tc_smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

static __device__ __forceinline__ void tc_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem_u32(bar)), "r"(count) : "memory");
}

static __device__ __forceinline__ void tc_fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

static __device__ __forceinline__ void tc_fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

static __device__ __forceinline__ void tc_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem_u32(bar)), "r"(bytes)
                 : "memory");
}

static __device__ __forceinline__ void tc_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem_u32(bar)) : "memory");
}

static __device__ __forceinline__ uint32_t tc_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tc_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}

// Non-blocking test of a phase (for a thread that serves several barriers).
static __device__ __forceinline__ uint32_t tc_mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tc_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}

// Bounded wait (about one second of SM clocks).  Returns false (and records `site`) if the
// phase never completed or the CTA aborted.
static __device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                    ktb_status* st, int site) {
    if (tc_mbar_try_wait(bar, parity)) return true;          // the common case costs no clock read
    const long long start = clock64();
    for (uint32_t i = 0;; ++i) {
        if (tc_mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            if (clock64() - start > 2000000000ll) break;
        }
    }
    *abort_flag = 1;
    if (atomicExch(&st->wait_timeout, 1) == 0) st->wait_site = site;
    return false;
}

static __device__ __forceinline__ void tc_tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                                      int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

static __device__ __forceinline__ void tc_tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                                      int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Tile store shared -> global (clipped at the tensor's edges), tracked by the issuing thread's bulk groups.
static __device__ __forceinline__ void tc_tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(tc_smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
static __device__ __forceinline__ void tc_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// At most N of this thread's bulk groups may still be READING their shared-memory source.
template <int N>
static __device__ __forceinline__ void tc_bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// All of this thread's bulk groups have completed (their writes are done).
static __device__ __forceinline__ void tc_bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

static __device__ __forceinline__ void tc_prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM ---------------------------------------------------------------------------------
static __device__ __forceinline__ void tc_tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

static __device__ __forceinline__ void tc_tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

static __device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

static __device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], f16/bf16 inputs, f32 accumulate.
static __device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// A operand taken from TMEM (e.g. softmax probabilities written back as f16).
static __device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Variants for a warp that runs the issuing code converged and lets one elected lane execute the
// tcgen05 instruction (`go` != 0 on that lane only): with warp-uniform operands the compiler can
// keep descriptors in uniform registers instead of moving them there per instruction.
static __device__ __forceinline__ uint32_t tc_elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred;
}
static __device__ __forceinline__ void tc_mma_f16_p(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                    uint32_t accumulate, uint32_t go) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(go)
        : "memory");
}
static __device__ __forceinline__ void tc_mma_f16_ts_p(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                                       uint32_t accumulate, uint32_t go) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(go)
        : "memory");
}
static __device__ __forceinline__ void tc_mma_commit_p(uint64_t* bar, uint32_t go) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(tc_smem_u32(bar)), "r"(go)
        : "memory");
}

// mbarrier arrives once every previously issued MMA of this thread has completed.
static __device__ __forceinline__ void tc_mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem_u32(bar))
                 : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster, ranks 0 (leader) and 1 ------------------------
// One tcgen05.mma issued by the leader multiplies a 256-row A (128 rows from each CTA's shared memory)
// with B whose columns are split between the two CTAs; each CTA accumulates its 128 rows in its own
// TMEM.  TMA loads of either CTA report to a barrier of the leader; tcgen05.commit reports to the
// barrier at the same shared-memory offset in both.  No load is multicast.
static __device__ __forceinline__ uint32_t tc_cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Address, in the cluster's shared window, of the same variable in CTA `rank`.
static __device__ __forceinline__ uint32_t tc_mapa(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

static __device__ __forceinline__ void tc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

static __device__ __forceinline__ void tc_mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

static __device__ __forceinline__ void tc_tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

static __device__ __forceinline__ void tc_tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// TMA tile load into this CTA's shared memory, completion bytes reported to `bar_cluster_addr`
// (a barrier of the pair's leader).
static __device__ __forceinline__ void tc_tma_load_2d_pair(void* smem_dst, const CUtensorMap* map,
                                                           uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(tc_smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

static __device__ __forceinline__ void tc_mma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The barrier at this shared-memory offset in both CTAs of the pair gets one arrival once every MMA
// issued so far by this thread has completed.
static __device__ __forceinline__ void tc_mma_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(tc_smem_u32(bar)), "h"((uint16_t)3)
        : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit values: thread i of the warp gets row (lane base + i).
static __device__ __forceinline__ void tc_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

static __device__ __forceinline__ void tc_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// one column: thread i of the warp gets / sets the word of row (lane base + i)
static __device__ __forceinline__ uint32_t tc_tmem_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}

static __device__ __forceinline__ void tc_tmem_st1(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}

template <int N>
static __device__ __forceinline__ void tc_tmem_ld(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tc_tmem_ld<32>(uint32_t taddr, uint32_t (&r)[32]) { tc_tmem_ld32(taddr, r); }
template <>
__device__ __forceinline__ void tc_tmem_ld<16>(uint32_t taddr, uint32_t (&r)[16]) { tc_tmem_ld16(taddr, r); }

static __device__ __forceinline__ void tc_tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

static __device__ __forceinline__ void tc_tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
          "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
          "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

static __device__ __forceinline__ void tc_tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

static __device__ __forceinline__ void tc_tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}

template <int N>
static __device__ __forceinline__ void tc_tmem_st(uint32_t taddr, const uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tc_tmem_st<32>(uint32_t taddr, const uint32_t (&r)[32]) { tc_tmem_st32(taddr, r); }
template <>
__device__ __forceinline__ void tc_tmem_st<16>(uint32_t taddr, const uint32_t (&r)[16]) { tc_tmem_st16(taddr, r); }
template <>
__device__ __forceinline__ void tc_tmem_st<8>(uint32_t taddr, const uint32_t (&r)[8]) { tc_tmem_st8(taddr, r); }

static __device__ __forceinline__ void tc_tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- descriptors ----------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version field set.
//   K-major operand  (rows of 64 f16 = 128 B, 8-row atoms of 1024 B): lbo unused (1), sbo = atom stride.
//   MN-major operand (128 B of the MN dim per K row, 8-K-row atoms of 1024 B): lbo = stride between
//   64-element MN blocks, sbo = stride between 8-row K groups.
static __device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;     // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;     // SWIZZLE_128B
    return d;
}

// Instruction descriptor: f16 x f16 -> f32, dense.  a_mn / b_mn: 1 when that operand is MN-major.
static __host__ __device__ __forceinline__ uint32_t tc_idesc_f16(int M, int N, int a_mn, int b_mn) {
    return (1u << 4) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}

// ---- host: tensor maps through the driver entry point (no link against libcuda) ----------------
typedef CUresult (*tc_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline tc_encode_fn tc_get_encode() {
    static tc_encode_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (tc_encode_fn)p;
    }
    return fn;
}

// Tensor of `rank` dims (dims[0] innermost), 128-byte swizzle, zero fill outside.
static inline bool tc_make_map(CUtensorMap* map, CUtensorMapDataType dtype, void* base, int rank, const uint64_t* dims,
                               const uint64_t* strides_bytes /* rank-1 */, const uint32_t* box) {
    tc_encode_fn enc = tc_get_encode();
    if (!enc) return false;
    cuuint64_t gdim[5], gstr[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
    return enc(map, dtype, (cuuint32_t)rank, base, gdim, gstr, bx, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static inline bool tc_make_map_f16(CUtensorMap* map, void* base, int rank, const uint64_t* dims,
                                   const uint64_t* strides_bytes /* rank-1 */, const uint32_t* box) {
    return tc_make_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, base, rank, dims, strides_bytes, box);
}
