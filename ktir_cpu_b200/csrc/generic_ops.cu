// Generic whole-grid steps: the op-by-op path for tile programs that match no fused kernel.
// Every kernel is a grid-stride loop over points x elements; nothing here is tuned — the
// point is to run any traced KTIR program with the reference's rounding behaviour
// (ktir_cpu/dialects/_helpers.py:39-72: f16 tiles compute in f32 and round per op;
// ktir_cpu/dialects/linalg_ops.py:86-133: pairwise halving reduction; ktir_cpu/memory.py:243-291:
// reads outside an allocation give 0, writes outside are dropped, negative indices are errors).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

enum { G_MOV, G_ADD, G_SUB, G_MUL, G_DIV, G_REM, G_MAX, G_MAXNUM, G_MIN, G_MINNUM, G_NEG, G_ABS, G_EXP, G_LOG,
       G_LOG2, G_LOG1P, G_SQRT, G_RSQRT, G_TANH, G_SIN, G_COS, G_CEIL, G_FLOOR, G_FMA, G_POW, G_SELECT,
       G_CMP_EQ, G_CMP_NE, G_CMP_LT, G_CMP_LE, G_CMP_GT, G_CMP_GE, G_CMP_ORD, G_CMP_UNO, G_CMP_TRUE, G_CMP_FALSE,
       G_AND, G_OR, G_XOR, G_SHL, G_SHR, G_DIVT, G_REMT, G_DIVF, G_CDIV, G_BITCAST, G_CMP_UNE, G_CMP_UEQ,
       G_CMP_ULT, G_CMP_ULE, G_CMP_UGT, G_CMP_UGE, G_SIGN };

static __host__ __device__ __forceinline__ bool g_is_float(int dt) { return dt == KTB_F16 || dt == KTB_F32; }
static __host__ __device__ __forceinline__ int g_size(int dt) {
    return dt == KTB_F16 ? 2 : dt == KTB_I64 ? 8 : dt == KTB_I1 ? 1 : 4;
}

static __device__ __forceinline__ float g_ldf(const void* p, int dt, int64_t i) {
    switch (dt) {
        case KTB_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
        case KTB_F32: return reinterpret_cast<const float*>(p)[i];
        case KTB_I32: return (float)reinterpret_cast<const int32_t*>(p)[i];
        case KTB_I64: return (float)reinterpret_cast<const int64_t*>(p)[i];
        default: return (float)reinterpret_cast<const uint8_t*>(p)[i];
    }
}
static __device__ __forceinline__ int64_t g_ldi(const void* p, int dt, int64_t i) {
    switch (dt) {
        case KTB_F16: return (int64_t)truncf(__half2float(reinterpret_cast<const __half*>(p)[i]));
        case KTB_F32: return (int64_t)truncf(reinterpret_cast<const float*>(p)[i]);
        case KTB_I32: return reinterpret_cast<const int32_t*>(p)[i];
        case KTB_I64: return reinterpret_cast<const int64_t*>(p)[i];
        default: return reinterpret_cast<const uint8_t*>(p)[i];
    }
}
static __device__ __forceinline__ void g_stf(void* p, int dt, int64_t i, float v) {
    switch (dt) {
        case KTB_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(v); break;
        case KTB_F32: reinterpret_cast<float*>(p)[i] = v; break;
        case KTB_I32: reinterpret_cast<int32_t*>(p)[i] = (int32_t)(int64_t)truncf(v); break;
        case KTB_I64: reinterpret_cast<int64_t*>(p)[i] = (int64_t)truncf(v); break;
        default: reinterpret_cast<uint8_t*>(p)[i] = (uint8_t)(int64_t)truncf(v); break;
    }
}
static __device__ __forceinline__ void g_sti(void* p, int dt, int64_t i, int64_t v) {
    switch (dt) {
        case KTB_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn((float)v); break;
        case KTB_F32: reinterpret_cast<float*>(p)[i] = (float)v; break;
        case KTB_I32: reinterpret_cast<int32_t*>(p)[i] = (int32_t)v; break;
        case KTB_I64: reinterpret_cast<int64_t*>(p)[i] = v; break;
        default: reinterpret_cast<uint8_t*>(p)[i] = (uint8_t)v; break;
    }
}
// raw element copy between arrays of the same dtype
static __device__ __forceinline__ void g_copy(void* d, int64_t di, const void* s, int64_t si, int size) {
    switch (size) {
        case 1: reinterpret_cast<uint8_t*>(d)[di] = reinterpret_cast<const uint8_t*>(s)[si]; break;
        case 2: reinterpret_cast<uint16_t*>(d)[di] = reinterpret_cast<const uint16_t*>(s)[si]; break;
        case 4: reinterpret_cast<uint32_t*>(d)[di] = reinterpret_cast<const uint32_t*>(s)[si]; break;
        default: reinterpret_cast<uint64_t*>(d)[di] = reinterpret_cast<const uint64_t*>(s)[si]; break;
    }
}
static __device__ __forceinline__ void g_zero(void* d, int64_t di, int size) {
    switch (size) {
        case 1: reinterpret_cast<uint8_t*>(d)[di] = 0; break;
        case 2: reinterpret_cast<uint16_t*>(d)[di] = 0; break;
        case 4: reinterpret_cast<uint32_t*>(d)[di] = 0; break;
        default: reinterpret_cast<uint64_t*>(d)[di] = 0; break;
    }
}

static __device__ __forceinline__ float g_fop(int op, float a, float b, float c) {
    const float nan = __int_as_float(0x7fc00000);
    switch (op) {
        case G_ADD: return a + b;
        case G_SUB: return a - b;
        case G_MUL: return a * b;
        case G_DIV: return a / b;
        case G_REM: return fmodf(a, b);
        // NumPy's selection rules: the first operand wins a tie (max(-0, +0) = -0)
        case G_MAX: return (a >= b || a != a) ? a : b;
        case G_MAXNUM: return (a >= b || b != b) ? a : b;
        case G_MIN: return (a <= b || a != a) ? a : b;
        case G_MINNUM: return (a <= b || b != b) ? a : b;
        case G_NEG: return -a;
        case G_ABS: return fabsf(a);
        case G_EXP: return expf(a);
        case G_LOG: return logf(a);
        case G_LOG2: return log2f(a);
        case G_LOG1P: return log1pf(a);
        case G_SQRT: return sqrtf(a);
        case G_RSQRT: return 1.0f / sqrtf(a);
        case G_TANH: return tanhf(a);
        case G_SIN: return sinf(a);
        case G_COS: return cosf(a);
        case G_CEIL: return ceilf(a);
        case G_FLOOR: return floorf(a);
        case G_FMA: return __fadd_rn(__fmul_rn(a, b), c);
        case G_POW: return powf(a, b);
        case G_SIGN: return a > 0.f ? 1.f : a < 0.f ? -1.f : a == 0.f ? 0.f : a;   // np.sign: +0 for either zero, NaN stays
        default: return a;
    }
}
static __device__ __forceinline__ int64_t g_floordiv(int64_t a, int64_t b) {
    if (b == 0) b = 1;
    int64_t q = a / b;
    if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
    return q;
}
static __device__ __forceinline__ int64_t g_iop(int op, int64_t a, int64_t b) {
    switch (op) {
        case G_ADD: return a + b;
        case G_SUB: return a - b;
        case G_MUL: return a * b;
        case G_DIVF: return g_floordiv(a, b);
        case G_DIVT: return b ? a / b : a;
        case G_REM: return a - g_floordiv(a, b) * (b ? b : 1);
        case G_REMT: return b ? a % b : 0;
        case G_AND: return a & b;
        case G_OR: return a | b;
        case G_XOR: return a ^ b;
        case G_SHL: return a << b;
        case G_SHR: return a >> b;
        case G_MIN: return a < b ? a : b;
        case G_MAX: return a > b ? a : b;
        case G_CDIV: return -g_floordiv(-a, b);
        case G_NEG: return -a;
        case G_ABS: return a < 0 ? -a : a;
        default: return a;
    }
}
template <typename T>
static __device__ __forceinline__ bool g_cmp(int op, T a, T b, bool unordered) {
    switch (op) {
        case G_CMP_EQ: return !unordered && a == b;
        case G_CMP_NE: return !unordered && a != b;
        case G_CMP_LT: return !unordered && a < b;
        case G_CMP_LE: return !unordered && a <= b;
        case G_CMP_GT: return !unordered && a > b;
        case G_CMP_GE: return !unordered && a >= b;
        case G_CMP_ORD: return !unordered;
        case G_CMP_UNO: return unordered;
        case G_CMP_TRUE: return true;
        case G_CMP_FALSE: return false;
        case G_CMP_UNE: return unordered || a != b;
        case G_CMP_UEQ: return unordered || a == b;
        case G_CMP_ULT: return unordered || a < b;
        case G_CMP_ULE: return unordered || a <= b;
        case G_CMP_UGT: return unordered || a > b;
        case G_CMP_UGE: return unordered || a >= b;
        default: return false;
    }
}

#define G_LOOP(i, total) \
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (total); i += (int64_t)gridDim.x * blockDim.x)

__global__ void g_load_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    const int size = g_size(o.dt_dst);
    G_LOOP(i, o.points * o.elems) {
        const int64_t p = i / o.elems, e = i - p * o.elems;
        const int64_t addr = o.dev_base[p] + o.dev_rel[e];
        if (o.kind == KTB_G_ADDR) {
            reinterpret_cast<int64_t*>(o.dst)[i] = addr;
        } else if (addr >= o.lo && addr < o.hi) {
            g_copy(o.dst, i, o.arena, addr, size);
        } else {
            g_zero(o.dst, i, size);
        }
    }
}

__global__ void g_idxadd_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    G_LOOP(i, o.points * o.elems) {
        const int64_t idx = g_ldi(o.b, o.dt_b, i);
        if (idx < 0 && atomicExch(&st->negative_index, 1) == 0) st->bad_index_value = (int32_t)idx;
        reinterpret_cast<int64_t*>(o.dst)[i] = reinterpret_cast<const int64_t*>(o.a)[i] + idx * o.iimm;
    }
}

__global__ void g_gather_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    const int size = g_size(o.dt_dst);
    G_LOOP(i, o.points * o.elems) {
        const int64_t addr = reinterpret_cast<const int64_t*>(o.a)[i];
        if (addr >= o.lo && addr < o.hi) g_copy(o.dst, i, o.arena, addr, size);
        else g_zero(o.dst, i, size);
    }
}

__global__ void g_fillers_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    const int size = g_size(o.dt_dst);
    G_LOOP(i, o.points * o.elems) {
        const int64_t p = i / o.elems, e = i - p * o.elems;
        if (o.kind == KTB_G_CONSTV) {
            g_copy(o.dst, i, o.dev_table, e, size);
        } else if (o.kind == KTB_G_PARAM) {
            g_copy(o.dst, i, o.dev_table, p, size);
        } else if (o.kind == KTB_G_TABLE) {
            g_copy(o.dst, i, o.dev_table, i, size);
        } else if (o.kind == KTB_G_FILL) {
            if (g_is_float(o.dt_dst)) g_stf(o.dst, o.dt_dst, i, (float)o.fimm);
            else g_sti(o.dst, o.dt_dst, i, o.iimm);
        } else {   // IOTA: coordinate of element e along dimension `offset` of `shape`
            int64_t rem = e, coord = 0;
            for (int d = o.ndim - 1; d >= 0; --d) {
                const int64_t c = rem % o.shape[d];
                rem /= o.shape[d];
                if (d == (int)o.offset) coord = c;
            }
            reinterpret_cast<int64_t*>(o.dst)[i] = coord;
        }
    }
}

__global__ void g_map_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    const int size = g_size(o.dt_dst);
    G_LOOP(i, o.points * o.elems) {
        const int64_t p = i / o.elems;
        int64_t rem = i - p * o.elems, src = o.offset;
        for (int d = o.ndim - 1; d >= 0; --d) {
            src += (rem % o.shape[d]) * o.strides[d];
            rem /= o.shape[d];
        }
        g_copy(o.dst, i, o.a, p * o.ea + src, size);
    }
}

static __device__ __forceinline__ void g_ew_one(const ktb_gen_op& o, int op, int64_t di, const void* pa, int dta,
                                                int64_t ia, const void* pb, int dtb, int64_t ib, const void* pc,
                                                int dtc, int64_t ic) {
    const bool dst_f = g_is_float(o.dt_dst);
    if (op == G_MOV) {
        if (dst_f) g_stf(o.dst, o.dt_dst, di, g_ldf(pa, dta, ia));
        else g_sti(o.dst, o.dt_dst, di, g_ldi(pa, dta, ia));
        return;
    }
    if (op == G_BITCAST) {
        if (g_size(o.dt_dst) == g_size(dta)) g_copy(o.dst, di, pa, ia, g_size(o.dt_dst));
        else if (dst_f) g_stf(o.dst, o.dt_dst, di, g_ldf(pa, dta, ia));
        else g_sti(o.dst, o.dt_dst, di, g_ldi(pa, dta, ia));
        return;
    }
    if ((op >= G_CMP_EQ && op <= G_CMP_FALSE) || (op >= G_CMP_UNE && op <= G_CMP_UGE)) {
        bool r;
        if (!(o.flags & 1) && (g_is_float(dta) || g_is_float(dtb))) {
            const float a = g_ldf(pa, dta, ia), b = g_ldf(pb, dtb, ib);
            r = g_cmp<float>(op, a, b, a != a || b != b);
        } else {
            r = g_cmp<int64_t>(op, g_ldi(pa, dta, ia), g_ldi(pb, dtb, ib), false);
        }
        g_sti(o.dst, o.dt_dst, di, r ? 1 : 0);
        return;
    }
    if (op == G_SELECT) {
        const bool cnd = g_ldi(pa, dta, ia) != 0;
        if (dst_f) g_stf(o.dst, o.dt_dst, di, cnd ? g_ldf(pb, dtb, ib) : g_ldf(pc, dtc, ic));
        else g_sti(o.dst, o.dt_dst, di, cnd ? g_ldi(pb, dtb, ib) : g_ldi(pc, dtc, ic));
        return;
    }
    if (dst_f) {
        const float a = g_ldf(pa, dta, ia);
        const float b = pb ? g_ldf(pb, dtb, ib) : 0.f;
        const float c = pc ? g_ldf(pc, dtc, ic) : 0.f;
        g_stf(o.dst, o.dt_dst, di, g_fop(op, a, b, c));
    } else {
        const int64_t a = g_ldi(pa, dta, ia);
        const int64_t b = pb ? g_ldi(pb, dtb, ib) : 0;
        g_sti(o.dst, o.dt_dst, di, g_iop(op, a, b));
    }
}

__global__ void g_ew_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    G_LOOP(i, o.points * o.elems) {
        const int64_t p = i / o.elems, e = i - p * o.elems;
        g_ew_one(o, o.op, i, o.a, o.dt_a, o.ea == 1 ? p : p * o.ea + e, o.b, o.dt_b, o.eb == 1 ? p : p * o.eb + e,
                 o.c, o.dt_c, o.ec == 1 ? p : p * o.ec + e);
    }
}

// one level of the halving tree: dst [outer][h + n%2][inner] from src [outer][n][inner]
__global__ void g_redl_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    const int64_t nm = o.h + (o.n & 1);
    const int size = g_size(o.dt_dst);
    G_LOOP(i, o.points * o.elems) {
        const int64_t p = i / o.elems;
        int64_t rem = i - p * o.elems;
        const int64_t in = rem % o.inner;
        rem /= o.inner;
        const int64_t k = rem % nm, ou = rem / nm;
        const int64_t s0 = p * o.ea + (ou * o.n + k) * o.inner + in;
        if (k < o.h) {
            g_ew_one(o, o.op, i, o.a, o.dt_a, s0, o.a, o.dt_a, s0 + o.h * o.inner, nullptr, 0, 0);
        } else {
            g_copy(o.dst, i, o.a, p * o.ea + (ou * o.n + 2 * o.h) * o.inner + in, size);
        }
    }
}

// dst[p][ou][k][in] = k < n ? a[p][ou][k][in] : b[p][ou][k - n][in]      (n = o.n rows of a, o.h rows of b)
__global__ void g_concat_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    const int size = g_size(o.dt_dst);
    const int64_t rows = o.n + o.h;
    G_LOOP(i, o.points * o.elems) {
        const int64_t p = i / o.elems;
        int64_t rem = i - p * o.elems;
        const int64_t in = rem % o.inner;
        rem /= o.inner;
        const int64_t k = rem % rows, ou = rem / rows;
        if (k < o.n) g_copy(o.dst, i, o.a, p * o.ea + (ou * o.n + k) * o.inner + in, size);
        else g_copy(o.dst, i, o.b, p * o.eb + (ou * o.h + (k - o.n)) * o.inner + in, size);
    }
}

// dst[p][b][m][n] = sum_k a[p][b][m][k] * b[p][b][k][n], f32 accumulation over k in order
__global__ void g_matmul_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    G_LOOP(i, o.points * o.elems) {
        const int64_t p = i / o.elems;
        int64_t rem = i - p * o.elems;
        const int64_t n = rem % o.N;
        rem /= o.N;
        const int64_t m = rem % o.M, b = rem / o.M;
        const int64_t a0 = p * o.ea + (b * o.M + m) * o.K, b0 = p * o.eb + b * o.K * o.N + n;
        float acc = 0.f;
        for (int64_t k = 0; k < o.K; ++k)
            acc = __fadd_rn(acc, __fmul_rn(g_ldf(o.a, o.dt_a, a0 + k), g_ldf(o.b, o.dt_b, b0 + k * o.N)));
        g_stf(o.dst, o.dt_dst, i, acc);
    }
}

__global__ void g_store_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    const int size = g_size(o.dt_a);
    G_LOOP(i, o.points * o.elems) {
        const int64_t p = i / o.elems, e = i - p * o.elems;
        const int64_t addr = o.dev_base[p] + o.dev_rel[e];
        if (addr >= o.lo && addr < o.hi) g_copy(o.arena, addr, o.a, o.ea == 1 ? p : i, size);
    }
}

// indirect store: points in order, elements in order (the last writer of an address wins,
// ktir_cpu/memory.py:281-291).  Duplicate addresses are rare and tiles of this path small,
// so one thread walks the list; the fused row scatter handles the large cases.
__global__ void g_scatter_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    const int size = g_size(o.dt_a);
    for (int64_t i = 0; i < o.points * o.elems; ++i) {
        const int64_t addr = reinterpret_cast<const int64_t*>(o.b)[i];
        const int64_t p = i / o.elems;
        if (addr >= o.lo && addr < o.hi) g_copy(o.arena, addr, o.a, o.ea == 1 ? p : i, size);
    }
}

// the same when the caller knows that no two elements share an address
__global__ void g_scatter_any_order_kernel(const __grid_constant__ ktb_gen_op o, ktb_status* st) {
    const int size = g_size(o.dt_a);
    G_LOOP(i, o.points * o.elems) {
        const int64_t addr = reinterpret_cast<const int64_t*>(o.b)[i];
        if (addr >= o.lo && addr < o.hi) g_copy(o.arena, addr, o.a, o.ea == 1 ? i / o.elems : i, size);
    }
}

// ---- cross-core ring reduce ---------------------------------------------------------------
// dst[p] = fold of a[p] with the partials of the other cores of p's group, in the order the
// reference's ring delivers them to that core (ktir_cpu/ops/comm_ops.py:294-345): core c folds in
// the partial that started on core (c - k) mod n in round k.  A forwarded tile is never modified,
// so the value that arrives equals the source core's own partial, and every fold rounds to the
// tile dtype like one more pass through the combiner region.
//
// CLUSTER: the cores of a group run as one thread-block cluster (one CTA per core, consecutive
// CTAs; dev_rel gives the point of each CTA).  Every CTA puts its partial into its own shared
// memory, the cluster synchronises, and the fold reads the peers' partials straight out of their
// shared memory (distributed shared memory, plain loads, no multicast); the sources of a point are
// then ranks inside the cluster.  Otherwise (groups of unequal size or more than 8 cores) the
// partials are read from global memory and the sources are point indices.
// Only hardware cluster barriers are used: there is no flag to spin on.
#define G_RING_CHUNK 8192          // elements of a partial staged in shared memory at a time
template <bool CLUSTER>
__global__ void __launch_bounds__(256) g_ring_kernel(const __grid_constant__ ktb_gen_op o) {
    extern __shared__ __align__(16) unsigned char g_ring_smem[];
    const int64_t p = CLUSTER ? o.dev_rel[blockIdx.x] : (int64_t)blockIdx.x;
    const int64_t cnt = o.dev_base[p];
    const int64_t* src = reinterpret_cast<const int64_t*>(o.dev_table) + p * o.n;
    const bool swapped = (o.flags & 2) != 0, r16 = o.dt_dst == KTB_F16;
    const int size = g_size(o.dt_a);
    for (int64_t e0 = 0; e0 < o.elems; e0 += G_RING_CHUNK) {
        const int64_t len = o.elems - e0 < G_RING_CHUNK ? o.elems - e0 : G_RING_CHUNK;
        if (CLUSTER) {
            for (int64_t i = threadIdx.x; i < len; i += blockDim.x) g_copy(g_ring_smem, i, o.a, p * o.elems + e0 + i, size);
            cg::this_cluster().sync();                 // every partial of the group is in place
        }
        for (int64_t i = threadIdx.x; i < len; i += blockDim.x) {
            float acc = CLUSTER ? g_ldf(g_ring_smem, o.dt_a, i) : g_ldf(o.a, o.dt_a, p * o.elems + e0 + i);
            for (int64_t j = 0; j < cnt; ++j) {
                float v;
                if (CLUSTER) v = g_ldf(cg::this_cluster().map_shared_rank(g_ring_smem, (unsigned)src[j]), o.dt_a, i);
                else v = g_ldf(o.a, o.dt_a, src[j] * o.elems + e0 + i);
                acc = swapped ? g_fop(o.op, v, acc, 0.f) : g_fop(o.op, acc, v, 0.f);
                if (r16) acc = ktb_round16(acc);
            }
            g_stf(o.dst, o.dt_dst, p * o.elems + e0 + i, acc);
        }
        if (CLUSTER) cg::this_cluster().sync();        // peers are done reading before the next chunk (or exit)
    }
}

static int launch_ring(ktb_ctx* ctx, const ktb_gen_op& o) {
    if (!g_is_float(o.dt_a) || o.dt_a != o.dt_dst) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "generic", "ring reduce of a non-float tile");
    if (o.points > 0x7fffffff) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "generic", "too many points");
    const int cluster = (int)o.h;
    if (cluster <= 1) {
        g_ring_kernel<false><<<(unsigned)o.points, 256, 0, ctx->stream>>>(o);
        return KTB_OK;
    }
    if (cluster > 8 || o.points % cluster) return ktb_fail(ctx, KTB_E_ARG, "generic", "bad cluster size");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)o.points);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = (size_t)(o.elems < G_RING_CHUNK ? o.elems : G_RING_CHUNK) * g_size(o.dt_a);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    KTB_CUDA(ctx, cudaLaunchKernelEx(&cfg, g_ring_kernel<true>, o));
    return KTB_OK;
}

extern "C" int ktb_launch_generic(ktb_ctx* ctx, const ktb_gen_op* op) {
    if (!ctx || !op) return KTB_E_ARG;
    const ktb_gen_op& o = *op;
    if (o.points < 0 || o.elems < 0 || o.ndim < 0 || o.ndim > KTB_G_MAXDIM)
        return ktb_fail(ctx, KTB_E_ARG, "generic", "bad extents");
    const int64_t total = o.points * o.elems;
    if (total == 0) return KTB_OK;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)ctx->sm_count * 32;
    if (blocks > cap) blocks = cap;
#define G_RUN(K) K<<<(unsigned)blocks, 256, 0, ctx->stream>>>(o, ctx->dev_status)
    switch (o.kind) {
        case KTB_G_LOAD:
        case KTB_G_ADDR: G_RUN(g_load_kernel); break;
        case KTB_G_IDXADD: G_RUN(g_idxadd_kernel); break;
        case KTB_G_GATHER: G_RUN(g_gather_kernel); break;
        case KTB_G_CONSTV:
        case KTB_G_FILL:
        case KTB_G_PARAM:
        case KTB_G_TABLE:
        case KTB_G_IOTA: G_RUN(g_fillers_kernel); break;
        case KTB_G_MAP: G_RUN(g_map_kernel); break;
        case KTB_G_EW: G_RUN(g_ew_kernel); break;
        case KTB_G_REDL: G_RUN(g_redl_kernel); break;
        case KTB_G_MATMUL: G_RUN(g_matmul_kernel); break;
        case KTB_G_CONCAT: G_RUN(g_concat_kernel); break;
        case KTB_G_STORE: G_RUN(g_store_kernel); break;
        case KTB_G_SCATTER:
            if (o.flags & 4) G_RUN(g_scatter_any_order_kernel);
            else g_scatter_kernel<<<1, 32, 0, ctx->stream>>>(o, ctx->dev_status);
            break;
        case KTB_G_RING:
            if (int rc = launch_ring(ctx, o)) return rc;
            break;
        default: return ktb_fail(ctx, KTB_E_ARG, "generic", "unknown step kind");
    }
#undef G_RUN
    KTB_CHECK_LAUNCH(ctx, "ktb_generic_kernel");
    return KTB_OK;
}
