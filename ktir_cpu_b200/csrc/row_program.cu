// Fused row programs: elementwise ops and reductions along a row in one launch.
//
// A row of `cols` elements belongs to a group of T threads (T = cols / 64, between 1 and 256; thread t
// owns the 16-byte vectors j * T + t, j < NV), a CTA of 256 threads carries 256 / T rows.  Per row
// the kernel runs the reduction phases of the statement one after the other — evaluate the phase's
// register program on every vector (operand tiles re-read through L1, row scalars broadcast into
// registers), fold the values in the halving order of the reference's linalg.reduce — then the
// scalar programs that have become computable, and finally the output program, whose result is
// stored.  Replaces the per-op dispatch of a normalisation kernel: linalg.reduce
// (ktir_cpu/dialects/linalg_ops.py:136-246), the arith / math ops on the reduced tile, the broadcast
// back (linalg_ops.py:349-465) and the elementwise ops around them, with the same rounding points
// (f16 tiles round after every op, f32 tiles do not).
#include "row_fold.cuh"
#include "vm.cuh"

template <int NV>
static __device__ __forceinline__ float rp_fold(const float (&x)[NV][8], const ktb_rp_phase& ph, int T, int t, int group,
                                                float* xchg, float* bcast) {
    if (ph.op == KTB_RP_ADD)
        return ph.round16 ? row_fold<NV, 1, false, true>(x, T, t, group, xchg, bcast)
                          : row_fold<NV, 1, false, false>(x, T, t, group, xchg, bcast);
    return ph.op == KTB_RP_MAXNUM ? row_fold<NV, 0, true, false>(x, T, t, group, xchg, bcast)
                                  : row_fold<NV, 0, false, false>(x, T, t, group, xchg, bcast);
}

static __device__ __forceinline__ void rp_load8(const void* arena, int64_t off, int dtype, float (&x)[8]) {
    if (dtype == KTB_F16) {
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(arena) + off);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            x[2 * i] = f.x;
            x[2 * i + 1] = f.y;
        }
    } else {
        const float* p = reinterpret_cast<const float*>(arena) + off;
        const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
        x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
        x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
    }
}

// The interpreter's registers live in shared memory, [register][element][thread]: consecutive threads hit
// consecutive banks, and 8 registers x 8 elements x 256 threads are 64 KB per CTA.  (As per-thread arrays
// they were local memory, more of it per SM than L1 holds, and every op waited on L2.)
#define RP_REG(q, v) (((q) * 8 + (v)) * 256)
#define RP_REGS_BYTES (KTB_VM_REGS * 8 * 256 * sizeof(float))

// The register program on one 8-element vector; the result stays in its register.  Not inlined on purpose:
// the kernel calls it from every phase and vector, and a copy of the interpreter at each call site (some
// dozens of KB of code) made the kernel wait for instructions more than for data.
#define RP_CASE(CODE, EXPR)                                                  \
    case CODE:                                                               \
        _Pragma("unroll") for (int v = 0; v < 8; ++v) {                      \
            const float a = A[v], b = B[v], c = Cc[v];                       \
            (void)a; (void)b; (void)c;                                       \
            R[v] = (EXPR);                                                   \
        }                                                                    \
        break;
static __device__ __noinline__ void rp_vm8(const ktb_vm_program& prog, float* regs /* this thread's slice */) {
    for (int i = 0; i < prog.n_ops; ++i) {
        const ktb_vm_op op = prog.ops[i];
        float A[8], B[8], Cc[8], R[8];
#pragma unroll
        for (int v = 0; v < 8; ++v) {
            A[v] = regs[RP_REG(op.a, v)];
            B[v] = regs[RP_REG(op.b, v)];
            Cc[v] = regs[RP_REG(op.c, v)];
        }
        const float imm = op.imm;
        switch (op.opcode & 0xff) {
            RP_CASE(KTB_VM_MOV, a)
            RP_CASE(KTB_VM_CONST, imm)
            RP_CASE(KTB_VM_ADD, a + b)
            RP_CASE(KTB_VM_SUB, a - b)
            RP_CASE(KTB_VM_MUL, a * b)
            RP_CASE(KTB_VM_DIV, a / b)
            RP_CASE(KTB_VM_SQRT, sqrtf(a))
            default:
#pragma unroll
                for (int v = 0; v < 8; ++v) R[v] = ktb_vm_apply(op.opcode & 0xff, A[v], B[v], Cc[v], imm);
        }
        if (op.opcode & KTB_VM_ROUND16) {
#pragma unroll
            for (int v = 0; v < 8; ++v) R[v] = ktb_round16(R[v]);
        }
#pragma unroll
        for (int v = 0; v < 8; ++v) regs[RP_REG(op.dst, v)] = R[v];
    }
}

// ... and on one value per row (row scalars, per-row results); registers 0.. hold the reduction results.  The
// registers are the caller's words of shared memory, `stride` floats apart: as a per-thread array they were
// local memory, which the streaming rows keep evicting from L1, and with every op waiting on L2 for its
// operands one evaluation took several microseconds during which the whole CTA stood at a barrier.
static __device__ __forceinline__ float rp_vm1_here(const ktb_vm_program& prog, const float* red, float* regs, int stride) {
#pragma unroll
    for (int q = 0; q < KTB_RP_MAX_RED; ++q) regs[q * stride] = red[q];
    for (int i = 0; i < prog.n_ops; ++i) {
        const ktb_vm_op op = prog.ops[i];
        const float a = (op.opcode & KTB_VM_IMM_A) ? op.imm : regs[op.a * stride];
        const float b = (op.opcode & KTB_VM_IMM_B) ? op.imm : regs[op.b * stride];
        float x;
        switch (op.opcode & 0xff) {                      // the handful of ops row values are made of, then the rest
            case KTB_VM_CONST: x = op.imm; break;
            case KTB_VM_ADD: x = a + b; break;
            case KTB_VM_SUB: x = a - b; break;
            case KTB_VM_MUL: x = a * b; break;
            case KTB_VM_DIV: x = a / b; break;
            case KTB_VM_SQRT: x = sqrtf(a); break;
            default: x = ktb_vm_apply(op.opcode & 0xff, a, b, regs[op.c * stride], op.imm);
        }
        regs[op.dst * stride] = (op.opcode & KTB_VM_ROUND16) ? ktb_round16(x) : x;
    }
    return regs[prog.result_reg * stride];
}

// Out of line for the interpreting kernel, which calls it from many places; the skeleton kernels call the
// inlined body, whose op fetches are then plain constant-bank reads of the argument block instead of loads
// through a generic pointer into it (layer norm 8192 x 1024: 37.9 -> 33.8 us).
static __device__ __noinline__ float rp_vm1(const ktb_vm_program& prog, const float* red, float* regs, int stride) {
    return rp_vm1_here(prog, red, regs, stride);
}

// Per-row results stored beside the output tile: programs over the finished reduction results of row `row`.
// (`from_scal[s]` >= 0: the result is row scalar `scal[from_scal[s]]`, computed already.)
static __device__ __forceinline__ void rp_store_sides(const ktb_rowprog_args& a, int64_t row, const float* red,
                                                      float* vmr, int vm_stride, const float* scal = nullptr,
                                                      const int* from_scal = nullptr) {
    const int64_t item = (uint32_t)row / (uint32_t)a.rows_per_item;
    const int64_t* offs = a.dev_item_offsets + item * (a.n_in + 1 + a.n_side) + a.n_in + 1;
    for (int s = 0; s < a.n_side; ++s) {
        const float o = from_scal && from_scal[s] >= 0 ? scal[from_scal[s]] : rp_vm1(a.side[s].prog, red, vmr, vm_stride);
        const int64_t go = offs[s] + (row - item * a.rows_per_item) * a.side[s].row_stride;
        if (a.side[s].dtype == KTB_F16) reinterpret_cast<__half*>(a.arena)[go] = __float2half_rn(o);
        else reinterpret_cast<float*>(a.arena)[go] = o;
    }
}

template <int NV>
__global__ void __launch_bounds__(256, NV >= 8 ? 2 : 3)
ktb_row_program_kernel(const __grid_constant__ ktb_rowprog_args a, int T, int64_t total_rows) {
    __shared__ float xchg[256 * 8];
    __shared__ float bcast[8];
    extern __shared__ float rp_reg_file[];
    float* regs = rp_reg_file + threadIdx.x;
    const int groups = 256 / T;
    const int group = threadIdx.x / T;
    const int t = threadIdx.x - group * T;
    // the trip count is the same for every thread of the CTA (the folds use group barriers and full-warp
    // shuffles); a group past the last row recomputes row 0 and skips the store
    const int64_t n_iter = (total_rows + groups - 1) / groups;
    for (int64_t it = blockIdx.x; it < n_iter; it += gridDim.x) {
        const bool live = it * groups + group < total_rows;
        const int64_t row = live ? it * groups + group : 0;
        const int64_t item = (uint32_t)row / (uint32_t)a.rows_per_item;      // (the launcher refuses 2^31 rows and more)
        const int64_t r = row - item * a.rows_per_item;
        int64_t off[KTB_VM_MAX_IN + 1];
#pragma unroll
        for (int k = 0; k <= KTB_VM_MAX_IN; ++k)
            off[k] = k <= a.n_in ? a.dev_item_offsets[item * (a.n_in + 1 + a.n_side) + k] + r * a.row_stride[k] : 0;

        float red[KTB_RP_MAX_RED] = {0.f, 0.f, 0.f};
        float scal[KTB_RP_MAX_SCAL] = {0.f, 0.f, 0.f, 0.f};
        int scal_done = 0;
        for (int p = 0; p <= a.n_red; ++p) {
            if (p == a.n_red && a.out_per_row) {
                // one value per row: a program over the reduction results, stored by the group's first thread
                const float o = rp_vm1(a.out.prog, red, regs, 8 * 256);
                if (live && t == 0) {
                    if (a.dtype[a.n_in] == KTB_F16) reinterpret_cast<__half*>(a.arena)[off[a.n_in]] = __float2half_rn(o);
                    else reinterpret_cast<float*>(a.arena)[off[a.n_in]] = o;
                }
                break;
            }
            if (p == a.n_red && a.n_side && live && t == 0) rp_store_sides(a, row, red, regs, 8 * 256);
            // row scalars that only need the reductions done so far
            for (; scal_done < a.n_scal && a.scal[scal_done].ready_after < p; ++scal_done)
                scal[scal_done] = rp_vm1(a.scal[scal_done].prog, red, regs, 8 * 256);
            const ktb_rp_phase& ph = p < a.n_red ? a.red[p] : a.out;
            const int nb = ph.blocked ? a.n_blocks : 1;
            const bool accumulate = ph.blocked && p < a.n_red;
            float x[NV][8];
            if (accumulate) {
#pragma unroll
                for (int j = 0; j < NV; ++j)
#pragma unroll
                    for (int v = 0; v < 8; ++v) x[j][v] = ph.acc_init;
            }
#pragma unroll
            for (int s = 0; s < KTB_RP_MAX_SCAL; ++s)
                if (s < a.n_scal && a.n_in + s < KTB_VM_REGS) {
#pragma unroll
                    for (int v = 0; v < 8; ++v) regs[RP_REG(a.n_in + s, v)] = scal[s];
                }
            for (int jb = 0; jb < nb; ++jb) {
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const int64_t col = ((int64_t)j * T + t) * 8;
                    float val[8];
                    if (ph.prog.n_ops == 0) {         // the phase reduces (or stores) an operand as it is
                        const int k = ph.prog.result_reg;
                        rp_load8(a.arena, off[k] + jb * a.blk_stride[k] + col, a.dtype[k], val);
                    } else {
#pragma unroll
                        for (int k = 0; k < KTB_VM_MAX_IN; ++k)
                            if (k < a.n_in && ((ph.load_mask >> k) & 1)) {
                                float in[8];
                                rp_load8(a.arena, off[k] + jb * a.blk_stride[k] + col, a.dtype[k], in);
#pragma unroll
                                for (int v = 0; v < 8; ++v) regs[RP_REG(k, v)] = in[v];
                            }
                        rp_vm8(ph.prog, regs);       // (x[] is not passed by address: it stays in registers)
#pragma unroll
                        for (int v = 0; v < 8; ++v) val[v] = regs[RP_REG(ph.prog.result_reg, v)];
                    }
                    if (accumulate) {
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            const float sacc = x[j][v] + val[v];
                            x[j][v] = ph.acc_round16 ? ktb_round16(sacc) : sacc;
                        }
                    } else if (p < a.n_red) {
#pragma unroll
                        for (int v = 0; v < 8; ++v) x[j][v] = val[v];
                    } else if (live) {
                        ktb_store_vec<8>(a.arena, off[a.n_in] + jb * a.blk_stride[a.n_in] + col, a.dtype[a.n_in], val);
                    }
                }
            }
            if (p < a.n_red) red[p] = rp_fold<NV>(x, ph, T, t, group, xchg, bcast);
        }
    }
}

// ---- normalisation skeletons without the interpreter --------------------------------------------------
// The vector programs of layer norm and RMS norm are always the same few ops; only the per-row values
// (how the mean and the scale come out of the sums) differ from kernel to kernel.  When the phases have
// one of these shapes, all in f32,
//     RMS:    red0 = sum(x * x);                          out = x * s [* w] [+ b]
//     mean:   red0 = sum(x);                              (per-row result only)
//     layer:  red0 = sum(x);  red1 = sum((x - m)^2);      out = (x - m) * s [* w] [+ b]
// (m, s: row scalars, any programs; operands of the commutative ops in either order; an optional final
// rounding to f16; or, instead of `out`, one value per row that is any program over the sums), the row is
// kept in registers and the skeleton runs as straight code with the same ops in the same order — same
// bits, a fraction of the time.  Row scalars and per-row results still go through rp_vm1.
enum { RP_RMS = 0, RP_MEAN = 1, RP_LAYER = 2 };
struct rp_norm {
    int mode, has_w, has_b, out_round16;
    int r16;                // every op (and every fold and accumulation) rounds to f16: an all-f16 kernel
    int blocked;            // the phases walk column blocks
    float acc_init;
    int x, w, b;            // operand indices
    int s_mean, s_scale;    // row scalar indices
    int side_scal[KTB_RP_MAX_SIDE];   // per-row side result s is row scalar side_scal[s] (same program), or -1
};

static thread_local int rp_round16 = 0;   // rounding mode the matcher expects of every op (set at the top of a match)
static bool rp_is(const ktb_vm_op& o, int code) {
    return (o.opcode & 0xff) == code && ((o.opcode & KTB_VM_ROUND16) != 0) == (rp_round16 != 0);
}

// o = code(p, q) with {p, q} = {cur, other}: returns `other`, or -1
static int rp_other(const ktb_vm_op& o, int code, int cur) {
    if (!rp_is(o, code)) return -1;
    if (o.a == cur) return o.b;
    if (o.b == cur) return o.a;
    return -1;
}

static bool rp_same_program(const ktb_vm_program& p, const ktb_vm_program& q) {
    if (p.n_in != q.n_in || p.n_ops != q.n_ops || p.result_reg != q.result_reg) return false;
    for (int i = 0; i < p.n_ops; ++i) {
        const ktb_vm_op &x = p.ops[i], &y = q.ops[i];
        if (x.opcode != y.opcode || x.dst != y.dst || x.a != y.a || x.b != y.b || x.c != y.c ||
            memcmp(&x.imm, &y.imm, sizeof(float)) != 0)
            return false;
    }
    return true;
}

static bool rp_match_norm_phases(const ktb_rowprog_args& a, rp_norm& m);
static bool rp_match_norm(const ktb_rowprog_args& a, rp_norm& m) {
    if (!rp_match_norm_phases(a, m)) return false;
    // a side result that is one of the two row scalars the skeleton computes anyway (the Mean and Rstd a layer
    // norm stores are its mean and its scale) is stored from there
    for (int s = 0; s < KTB_RP_MAX_SIDE; ++s) {
        m.side_scal[s] = -1;
        if (s >= a.n_side || a.out_per_row) continue;
        if (m.s_mean >= 0 && rp_same_program(a.side[s].prog, a.scal[m.s_mean].prog)) m.side_scal[s] = m.s_mean;
        else if (m.s_scale >= 0 && rp_same_program(a.side[s].prog, a.scal[m.s_scale].prog)) m.side_scal[s] = m.s_scale;
    }
    return true;
}

static bool rp_match_norm_phases(const ktb_rowprog_args& a, rp_norm& m) {
    if (a.n_red < 1 || a.n_red > 2) return false;
    m = rp_norm{};
    m.w = m.b = m.s_mean = m.s_scale = -1;
    // one rounding mode and one way of walking the row for all phases
    m.r16 = a.red[0].round16 != 0;
    m.blocked = a.red[0].blocked != 0;
    m.acc_init = a.red[0].acc_init;
    for (int p = 0; p < a.n_red; ++p) {
        const ktb_rp_phase& ph = a.red[p];
        if (ph.op != KTB_RP_ADD || (ph.round16 != 0) != (m.r16 != 0) || (ph.blocked != 0) != (m.blocked != 0)) return false;
        if (ph.blocked && ((ph.acc_round16 != 0) != (m.r16 != 0) || ph.acc_init != m.acc_init)) return false;
    }
    if (!a.out_per_row && (a.out.blocked != 0) != (m.blocked != 0)) return false;
    rp_round16 = m.r16;
    const int n_in = a.n_in;
    auto is_load = [&](int r) { return r >= 0 && r < n_in; };
    auto is_scal = [&](int r) { return r >= n_in && r < n_in + a.n_scal; };
    // the sums
    const ktb_vm_program& r0 = a.red[0].prog;
    if (r0.n_ops == 0 && is_load(r0.result_reg)) {
        m.x = r0.result_reg;
        m.mode = RP_MEAN;
    } else if (r0.n_ops == 1 && rp_is(r0.ops[0], KTB_VM_MUL) && r0.ops[0].a == r0.ops[0].b && is_load(r0.ops[0].a) &&
               r0.result_reg == r0.ops[0].dst) {
        m.x = r0.ops[0].a;
        m.mode = RP_RMS;
    } else {
        return false;
    }
    int mean_reg = -1;
    if (a.n_red == 2) {
        const ktb_vm_program& r1 = a.red[1].prog;
        if (m.mode != RP_MEAN || r1.n_ops != 2 || !rp_is(r1.ops[0], KTB_VM_SUB) || r1.ops[0].a != m.x ||
            !is_scal(r1.ops[0].b) || !rp_is(r1.ops[1], KTB_VM_MUL) || r1.ops[1].a != r1.ops[0].dst ||
            r1.ops[1].b != r1.ops[0].dst || r1.result_reg != r1.ops[1].dst)
            return false;
        m.mode = RP_LAYER;
        mean_reg = r1.ops[0].b;
        m.s_mean = mean_reg - n_in;
        if (a.scal[m.s_mean].ready_after > 0) return false;
    }
    if (a.out_per_row) return true;                      // any program over the sums
    if (m.mode == RP_MEAN) return false;
    // the stored expression
    const ktb_vm_program& o = a.out.prog;
    int i = 0, cur, sc;
    if (m.mode == RP_RMS) {
        if (o.n_ops < 1) return false;
        sc = rp_other(o.ops[0], KTB_VM_MUL, m.x);
        cur = o.ops[0].dst;
        i = 1;
    } else {
        if (o.n_ops < 2 || !rp_is(o.ops[0], KTB_VM_SUB) || o.ops[0].a != m.x || o.ops[0].b != mean_reg) return false;
        sc = rp_other(o.ops[1], KTB_VM_MUL, o.ops[0].dst);
        cur = o.ops[1].dst;
        i = 2;
    }
    if (!is_scal(sc) || sc == mean_reg) return false;
    m.s_scale = sc - n_in;
    if (i < o.n_ops) {                                   // [* w]
        const int w = rp_other(o.ops[i], KTB_VM_MUL, cur);
        if (is_load(w) && w != m.x) {
            m.w = w;
            m.has_w = 1;
            cur = o.ops[i++].dst;
        }
    }
    if (i < o.n_ops) {                                   // [+ b]
        const int b = rp_other(o.ops[i], KTB_VM_ADD, cur);
        if (is_load(b) && b != m.x && b != m.w) {
            m.b = b;
            m.has_b = 1;
            cur = o.ops[i++].dst;
        }
    }
    if (!m.r16 && i < o.n_ops && (o.ops[i].opcode & 0xff) == KTB_VM_MOV && (o.ops[i].opcode & KTB_VM_ROUND16) && o.ops[i].a == cur) {
        m.out_round16 = 1;
        cur = o.ops[i++].dst;
    }
    return i == o.n_ops && o.result_reg == cur;
}

template <int NV, int MODE, bool PER_ROW>
#ifndef KTB_RP_NORM_OCC
#define KTB_RP_NORM_OCC 3
#endif
__global__ void __launch_bounds__(256, NV >= 8 ? 1 : NV >= 4 ? KTB_RP_NORM_OCC : NV >= 2 ? 3 : 4)
ktb_row_norm_kernel(const __grid_constant__ ktb_rowprog_args a, const rp_norm m, int T, int64_t total_rows) {
    __shared__ float xchg[256 * 8];
    __shared__ float bcast[8];
    __shared__ float s_red[256][KTB_RP_MAX_RED];
    __shared__ float s_scal[256][KTB_RP_MAX_SCAL];
    __shared__ float s_vm[KTB_VM_REGS * 256];            // registers of the row-value programs, [register][thread]
    const int groups = 256 / T;
    const int group = threadIdx.x / T;
    const int t = threadIdx.x - group * T;
    const int64_t n_iter = (total_rows + groups - 1) / groups;
    for (int64_t it = blockIdx.x; it < n_iter; it += gridDim.x) {
        const bool live = it * groups + group < total_rows;
        const int64_t row = live ? it * groups + group : 0;
        const int64_t item = (uint32_t)row / (uint32_t)a.rows_per_item;
        const int64_t r = row - item * a.rows_per_item;
        const int64_t* offs = a.dev_item_offsets + item * (a.n_in + 1 + a.n_side);
        const int64_t x_off = offs[m.x] + r * a.row_stride[m.x];
        const int64_t y_off = offs[a.n_in] + r * a.row_stride[a.n_in];
        float x[NV][8];
#pragma unroll
        for (int j = 0; j < NV; ++j) rp_load8(a.arena, x_off + ((int64_t)j * T + t) * 8, a.dtype[m.x], x[j]);

        // Row values are computed "sideways": the first thread of every row group parks the row's sums, then
        // thread g of the CTA runs the scalar programs of row g — all rows of the CTA in the lanes of one or
        // a few warps instead of the same program once per warp of every row.
        float mean = 0.f;
        if (MODE != RP_RMS) {
            const float r0 = row_fold<NV, 1, false, false>(x, T, t, group, xchg, bcast);
            if (t == 0) s_red[group][0] = r0;
            if (MODE == RP_LAYER) {
                __syncthreads();
                if (threadIdx.x < groups)
                    s_scal[threadIdx.x][m.s_mean] = rp_vm1_here(a.scal[m.s_mean].prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                __syncthreads();
                mean = s_scal[group][m.s_mean];
            }
        }
        if (MODE != RP_MEAN) {
            float sq[NV][8];
#pragma unroll
            for (int j = 0; j < NV; ++j)
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    const float d = MODE == RP_LAYER ? x[j][v] - mean : x[j][v];
                    sq[j][v] = d * d;
                }
            const float r1 = row_fold<NV, 1, false, false>(sq, T, t, group, xchg, bcast);
            if (t == 0) s_red[group][MODE == RP_LAYER ? 1 : 0] = r1;
        }
        __syncthreads();
        if (threadIdx.x < groups) {
            const int64_t grow = it * groups + threadIdx.x;
            if (PER_ROW) {
                const float o = rp_vm1_here(a.out.prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                if (grow < total_rows) {
                    const int64_t gitem = (uint32_t)grow / (uint32_t)a.rows_per_item;
                    const int64_t go = a.dev_item_offsets[gitem * (a.n_in + 1 + a.n_side) + a.n_in] +
                                       (grow - gitem * a.rows_per_item) * a.row_stride[a.n_in];
                    if (a.dtype[a.n_in] == KTB_F16) reinterpret_cast<__half*>(a.arena)[go] = __float2half_rn(o);
                    else reinterpret_cast<float*>(a.arena)[go] = o;
                }
            } else {
                s_scal[threadIdx.x][m.s_scale] = rp_vm1_here(a.scal[m.s_scale].prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                if (a.n_side && grow < total_rows) rp_store_sides(a, grow, s_red[threadIdx.x], s_vm + threadIdx.x, 256, s_scal[threadIdx.x], m.side_scal);
            }
        }
        __syncthreads();                                 // (also keeps the next iteration's sums off this one's readers)
        if (PER_ROW) continue;
        float scal[KTB_RP_MAX_SCAL];
#pragma unroll
        for (int q = 0; q < KTB_RP_MAX_SCAL; ++q) scal[q] = s_scal[group][q];
        const float scale = scal[m.s_scale];
        if (!live) continue;
        const int64_t w_off = m.has_w ? offs[m.w] + r * a.row_stride[m.w] : 0;
        const int64_t b_off = m.has_b ? offs[m.b] + r * a.row_stride[m.b] : 0;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int64_t col = ((int64_t)j * T + t) * 8;
            float y[8], w[8], b[8];
            if (m.has_w) rp_load8(a.arena, w_off + col, a.dtype[m.w], w);
            if (m.has_b) rp_load8(a.arena, b_off + col, a.dtype[m.b], b);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                float q = MODE == RP_LAYER ? x[j][v] - mean : x[j][v];
                q = q * scale;
                if (m.has_w) q = q * w[v];
                if (m.has_b) q = q + b[v];
                y[v] = m.out_round16 ? ktb_round16(q) : q;
            }
            ktb_store_vec<8>(a.arena, y_off + col, a.dtype[a.n_in], y);
        }
    }
}

// The same skeletons for rows given as NB column blocks and / or all-f16 arithmetic (the form of
// examples/triton-ktir/layernorm_fwd_ktir.mlir): the whole row — NB blocks x NV vectors per thread — sits in
// registers, the sums are accumulated block after block and folded, every op rounds to f16 where the tile
// dtype is f16.  Mode, rounding and per-row output are run-time switches here (uniform branches).
template <int NB, int NV>
__global__ void __launch_bounds__(256, NB * NV >= 8 ? 2 : 3)
ktb_row_norm_blocks_kernel(const __grid_constant__ ktb_rowprog_args a, const rp_norm m, int T, int64_t total_rows) {
    __shared__ float xchg[256 * 8];
    __shared__ float bcast[8];
    __shared__ float s_red[256][KTB_RP_MAX_RED];
    __shared__ float s_scal[256][KTB_RP_MAX_SCAL];
    __shared__ float s_vm[KTB_VM_REGS * 256];            // registers of the row-value programs, [register][thread]
    const int groups = 256 / T;
    const int group = threadIdx.x / T;
    const int t = threadIdx.x - group * T;
    const bool r16 = m.r16 != 0;
    auto rnd = [&](float v) { return r16 ? ktb_round16(v) : v; };
    auto fold = [&](const float (&v)[NV][8]) {
        return r16 ? row_fold<NV, 1, false, true>(v, T, t, group, xchg, bcast)
                   : row_fold<NV, 1, false, false>(v, T, t, group, xchg, bcast);
    };
    const int64_t n_iter = (total_rows + groups - 1) / groups;
    for (int64_t it = blockIdx.x; it < n_iter; it += gridDim.x) {
        const bool live = it * groups + group < total_rows;
        const int64_t row = live ? it * groups + group : 0;
        const int64_t item = (uint32_t)row / (uint32_t)a.rows_per_item;
        const int64_t r = row - item * a.rows_per_item;
        const int64_t* offs = a.dev_item_offsets + item * (a.n_in + 1 + a.n_side);
        const int64_t x_off = offs[m.x] + r * a.row_stride[m.x];
        const int64_t y_off = offs[a.n_in] + r * a.row_stride[a.n_in];
        float x[NB][NV][8];
#pragma unroll
        for (int jb = 0; jb < NB; ++jb)
#pragma unroll
            for (int j = 0; j < NV; ++j)
                rp_load8(a.arena, x_off + jb * a.blk_stride[m.x] + ((int64_t)j * T + t) * 8, a.dtype[m.x], x[jb][j]);

        float mean = 0.f;
        if (m.mode != RP_RMS) {
            float acc[NV][8];
#pragma unroll
            for (int j = 0; j < NV; ++j)
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    float s_ = m.blocked ? rnd(m.acc_init + x[0][j][v]) : x[0][j][v];
#pragma unroll
                    for (int jb = 1; jb < NB; ++jb) s_ = rnd(s_ + x[jb][j][v]);
                    acc[j][v] = s_;
                }
            const float r0 = fold(acc);
            if (t == 0) s_red[group][0] = r0;
            if (m.mode == RP_LAYER) {
                __syncthreads();
                if (threadIdx.x < groups) s_scal[threadIdx.x][m.s_mean] = rp_vm1_here(a.scal[m.s_mean].prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                __syncthreads();
                mean = s_scal[group][m.s_mean];
            }
        }
        if (m.mode != RP_MEAN) {
            float acc[NV][8];
#pragma unroll
            for (int j = 0; j < NV; ++j)
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    float s_ = 0.f;
#pragma unroll
                    for (int jb = 0; jb < NB; ++jb) {
                        const float d = m.mode == RP_LAYER ? rnd(x[jb][j][v] - mean) : x[jb][j][v];
                        const float q = rnd(d * d);
                        s_ = jb == 0 ? (m.blocked ? rnd(m.acc_init + q) : q) : rnd(s_ + q);
                    }
                    acc[j][v] = s_;
                }
            const float r1 = fold(acc);
            if (t == 0) s_red[group][m.mode == RP_LAYER ? 1 : 0] = r1;
        }
        __syncthreads();
        if (threadIdx.x < groups) {
            const int64_t grow = it * groups + threadIdx.x;
            if (a.out_per_row) {
                const float o = rp_vm1_here(a.out.prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                if (grow < total_rows) {
                    const int64_t gitem = (uint32_t)grow / (uint32_t)a.rows_per_item;
                    const int64_t go = a.dev_item_offsets[gitem * (a.n_in + 1 + a.n_side) + a.n_in] +
                                       (grow - gitem * a.rows_per_item) * a.row_stride[a.n_in];
                    if (a.dtype[a.n_in] == KTB_F16) reinterpret_cast<__half*>(a.arena)[go] = __float2half_rn(o);
                    else reinterpret_cast<float*>(a.arena)[go] = o;
                }
            } else {
                s_scal[threadIdx.x][m.s_scale] = rp_vm1_here(a.scal[m.s_scale].prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                if (a.n_side && grow < total_rows) rp_store_sides(a, grow, s_red[threadIdx.x], s_vm + threadIdx.x, 256, s_scal[threadIdx.x], m.side_scal);
            }
        }
        __syncthreads();
        if (a.out_per_row) continue;
        const float scale = s_scal[group][m.s_scale];
        if (!live) continue;
        const int64_t w_off = m.has_w ? offs[m.w] + r * a.row_stride[m.w] : 0;
        const int64_t b_off = m.has_b ? offs[m.b] + r * a.row_stride[m.b] : 0;
#pragma unroll
        for (int jb = 0; jb < NB; ++jb)
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int64_t col = ((int64_t)j * T + t) * 8;
                float y[8], w[8], b[8];
                if (m.has_w) rp_load8(a.arena, w_off + jb * a.blk_stride[m.w] + col, a.dtype[m.w], w);
                if (m.has_b) rp_load8(a.arena, b_off + jb * a.blk_stride[m.b] + col, a.dtype[m.b], b);
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    float q = m.mode == RP_LAYER ? rnd(x[jb][j][v] - mean) : x[jb][j][v];
                    q = rnd(q * scale);
                    if (m.has_w) q = rnd(q * w[v]);
                    if (m.has_b) q = rnd(q + b[v]);
                    y[v] = m.out_round16 ? ktb_round16(q) : q;
                }
                ktb_store_vec<8>(a.arena, y_off + jb * a.blk_stride[a.n_in] + col, a.dtype[a.n_in], y);
            }
    }
}

// ... and when everything is f16 — operand tiles, the stored tile, every op rounding to f16 — the arithmetic
// runs on packed halves: an f16 add, subtract or multiply of f16 values is the f32 op rounded to f16 (the
// double rounding cannot show: 24 >= 2 * 11 + 2 significand bits), so these are the bits of the kernel
// above without its two conversions per op, which is what bounded it (layer norm f16[4096, 8192] in eight
// column blocks: 176 us there).  The row sits in registers as it came from memory.
#ifndef KTB_RP_H_OCC
#define KTB_RP_H_OCC 4
#endif
template <int NB, int NV>
__global__ void __launch_bounds__(256, KTB_RP_H_OCC)
ktb_row_norm_h_kernel(const __grid_constant__ ktb_rowprog_args a, const rp_norm m, int T, int64_t total_rows) {
    __shared__ float xchg[256 * 8];
    __shared__ float bcast[8];
    __shared__ float s_red[256][KTB_RP_MAX_RED];
    __shared__ float s_scal[256][KTB_RP_MAX_SCAL];
    __shared__ float s_vm[KTB_VM_REGS * 256];            // registers of the row-value programs, [register][thread]
    const int groups = 256 / T;
    const int group = threadIdx.x / T;
    const int t = threadIdx.x - group * T;
    const __half* arena = reinterpret_cast<const __half*>(a.arena);
    const __half2 init = __float2half2_rn(m.acc_init);
    auto load4 = [&](int64_t off, __half2 (&v)[4]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(arena + off);
        v[0] = *reinterpret_cast<const __half2*>(&raw.x);
        v[1] = *reinterpret_cast<const __half2*>(&raw.y);
        v[2] = *reinterpret_cast<const __half2*>(&raw.z);
        v[3] = *reinterpret_cast<const __half2*>(&raw.w);
    };
    const int64_t n_iter = (total_rows + groups - 1) / groups;
    for (int64_t it = blockIdx.x; it < n_iter; it += gridDim.x) {
        const bool live = it * groups + group < total_rows;
        const int64_t row = live ? it * groups + group : 0;
        const int64_t item = (uint32_t)row / (uint32_t)a.rows_per_item;
        const int64_t r = row - item * a.rows_per_item;
        const int64_t* offs = a.dev_item_offsets + item * (a.n_in + 1 + a.n_side);
        const int64_t x_off = offs[m.x] + r * a.row_stride[m.x];
        const int64_t y_off = offs[a.n_in] + r * a.row_stride[a.n_in];
        __half2 x[NB][NV][4];
#pragma unroll
        for (int jb = 0; jb < NB; ++jb)
#pragma unroll
            for (int j = 0; j < NV; ++j) load4(x_off + jb * a.blk_stride[m.x] + ((int64_t)j * T + t) * 8, x[jb][j]);

        __half2 mean = __half2();
        if (m.mode != RP_RMS) {
            __half2 acc[NV][4];
#pragma unroll
            for (int j = 0; j < NV; ++j)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    __half2 s_ = m.blocked ? __hadd2_rn(init, x[0][j][q]) : x[0][j][q];
#pragma unroll
                    for (int jb = 1; jb < NB; ++jb) s_ = __hadd2_rn(s_, x[jb][j][q]);
                    acc[j][q] = s_;
                }
            const float r0 = row_fold_h<NV>(acc, T, t, group, xchg, bcast);
            if (t == 0) s_red[group][0] = r0;
            if (m.mode == RP_LAYER) {
                __syncthreads();
                if (threadIdx.x < groups) s_scal[threadIdx.x][m.s_mean] = rp_vm1_here(a.scal[m.s_mean].prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                __syncthreads();
                mean = __float2half2_rn(s_scal[group][m.s_mean]);
            }
        }
        if (m.mode != RP_MEAN) {
            __half2 acc[NV][4];
#pragma unroll
            for (int j = 0; j < NV; ++j)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    __half2 s_ = __half2();
#pragma unroll
                    for (int jb = 0; jb < NB; ++jb) {
                        const __half2 d = m.mode == RP_LAYER ? __hsub2_rn(x[jb][j][q], mean) : x[jb][j][q];
                        const __half2 sq = __hmul2_rn(d, d);
                        s_ = jb == 0 ? (m.blocked ? __hadd2_rn(init, sq) : sq) : __hadd2_rn(s_, sq);
                    }
                    acc[j][q] = s_;
                }
            const float r1 = row_fold_h<NV>(acc, T, t, group, xchg, bcast);
            if (t == 0) s_red[group][m.mode == RP_LAYER ? 1 : 0] = r1;
        }
        __syncthreads();
        if (threadIdx.x < groups) {
            const int64_t grow = it * groups + threadIdx.x;
            if (a.out_per_row) {
                const float o = rp_vm1_here(a.out.prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                if (grow < total_rows) {
                    const int64_t gitem = (uint32_t)grow / (uint32_t)a.rows_per_item;
                    const int64_t go = a.dev_item_offsets[gitem * (a.n_in + 1 + a.n_side) + a.n_in] +
                                       (grow - gitem * a.rows_per_item) * a.row_stride[a.n_in];
                    if (a.dtype[a.n_in] == KTB_F16) reinterpret_cast<__half*>(a.arena)[go] = __float2half_rn(o);
                    else reinterpret_cast<float*>(a.arena)[go] = o;
                }
            } else {
                s_scal[threadIdx.x][m.s_scale] = rp_vm1_here(a.scal[m.s_scale].prog, s_red[threadIdx.x], s_vm + threadIdx.x, 256);
                if (a.n_side && grow < total_rows) rp_store_sides(a, grow, s_red[threadIdx.x], s_vm + threadIdx.x, 256, s_scal[threadIdx.x], m.side_scal);
            }
        }
        __syncthreads();
        if (a.out_per_row) continue;
        const __half2 scale = __float2half2_rn(s_scal[group][m.s_scale]);
        if (!live) continue;
        const int64_t w_off = m.has_w ? offs[m.w] + r * a.row_stride[m.w] : 0;
        const int64_t b_off = m.has_b ? offs[m.b] + r * a.row_stride[m.b] : 0;
#pragma unroll
        for (int jb = 0; jb < NB; ++jb)
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int64_t col = ((int64_t)j * T + t) * 8;
                __half2 w[4], b[4];
                uint4 y;
                __half2* yh = reinterpret_cast<__half2*>(&y);
                if (m.has_w) load4(w_off + jb * a.blk_stride[m.w] + col, w);
                if (m.has_b) load4(b_off + jb * a.blk_stride[m.b] + col, b);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    __half2 v = m.mode == RP_LAYER ? __hsub2_rn(x[jb][j][q], mean) : x[jb][j][q];
                    v = __hmul2_rn(v, scale);
                    if (m.has_w) v = __hmul2_rn(v, w[q]);
                    if (m.has_b) v = __hadd2_rn(v, b[q]);
                    yh[q] = v;
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.arena) + y_off + jb * a.blk_stride[a.n_in] + col) = y;
            }
    }
}

template <int NB, int NV>
static void rp_launch_norm_blocks(ktb_ctx* ctx, const ktb_rowprog_args& a, const rp_norm& m, int T, int64_t total_rows) {
    const int groups = 256 / T;
    const int64_t iters = (total_rows + groups - 1) / groups;
    const unsigned blocks = (unsigned)(iters < (int64_t)ctx->sm_count * 4 ? iters : (int64_t)ctx->sm_count * 4);
    // all f16, every op rounding to f16: packed-half arithmetic
    bool halves = m.r16 && a.dtype[m.x] == KTB_F16 && (a.out_per_row || a.dtype[a.n_in] == KTB_F16) &&
                  (!m.has_w || a.dtype[m.w] == KTB_F16) && (!m.has_b || a.dtype[m.b] == KTB_F16);
#ifdef KTB_RP_NO_HALVES
    halves = false;
#endif
    if (halves) {
        ktb_row_norm_h_kernel<NB, NV><<<blocks, 256, 0, ctx->stream>>>(a, m, T, total_rows);
    } else {
        ktb_row_norm_blocks_kernel<NB, NV><<<blocks, 256, 0, ctx->stream>>>(a, m, T, total_rows);
    }
}

// NB blocks x NV vectors per thread, at most 8 together; false if the row does not fit that way
static bool rp_try_norm_blocks(ktb_ctx* ctx, const ktb_rowprog_args& a, const rp_norm& m, int64_t total_rows) {
    const int NB = m.blocked ? a.n_blocks : 1;
    if (NB != 1 && NB != 2 && NB != 4 && NB != 8) return false;
    const int vecs = a.cols / 8;
    int NV = 8 / NB;                                     // as many vectors per thread as still fit ...
    while (NV > 1 && (vecs / NV < 1 || total_rows / (256 / (vecs / NV > 256 ? 256 : vecs / NV)) < 2 * (int64_t)ctx->sm_count)) NV /= 2;
    if (vecs / NV > 256) return false;                   // ... (fewer when there are few rows) and the row must fit a CTA
    if (vecs % NV) return false;
    const int T = vecs / NV;
#define RP_NB(B, V) if (NB == B && NV == V) { rp_launch_norm_blocks<B, V>(ctx, a, m, T, total_rows); return true; }
    RP_NB(1, 1) RP_NB(1, 2) RP_NB(1, 4) RP_NB(1, 8)
    RP_NB(2, 1) RP_NB(2, 2) RP_NB(2, 4)
    RP_NB(4, 1) RP_NB(4, 2)
    RP_NB(8, 1)
#undef RP_NB
    return false;
}

template <int NV>
static void rp_launch_norm(ktb_ctx* ctx, const ktb_rowprog_args& a, const rp_norm& m, unsigned blocks, int T, int64_t total_rows) {
#define RP_NORM(M, P) ktb_row_norm_kernel<NV, M, P><<<blocks, 256, 0, ctx->stream>>>(a, m, T, total_rows)
    switch (m.mode * 2 + (a.out_per_row ? 1 : 0)) {
        case RP_RMS * 2: RP_NORM(RP_RMS, false); break;
        case RP_RMS * 2 + 1: RP_NORM(RP_RMS, true); break;
        case RP_MEAN * 2 + 1: RP_NORM(RP_MEAN, true); break;
        case RP_LAYER * 2: RP_NORM(RP_LAYER, false); break;
        default: RP_NORM(RP_LAYER, true); break;
    }
#undef RP_NORM
}

static int rp_check_program(ktb_ctx* ctx, const ktb_vm_program& p, int n_in, bool row_value = false) {
    if (p.n_in != n_in || p.n_ops < 0 || p.n_ops > KTB_VM_MAX_OPS || p.result_reg < 0 || p.result_reg >= KTB_VM_REGS)
        return ktb_fail(ctx, KTB_E_ARG, "row_program", "bad program header");
    for (int i = 0; i < p.n_ops; ++i) {
        const ktb_vm_op& o = p.ops[i];
        if ((o.opcode & 0xff) >= KTB_VM_NOPS || o.dst < 0 || o.dst >= KTB_VM_REGS || o.a < 0 || o.a >= KTB_VM_REGS ||
            o.b < 0 || o.b >= KTB_VM_REGS || o.c < 0 || o.c >= KTB_VM_REGS)
            return ktb_fail(ctx, KTB_E_ARG, "row_program", "bad program op");
        if (!row_value && (o.opcode & (KTB_VM_IMM_A | KTB_VM_IMM_B)))
            return ktb_fail(ctx, KTB_E_ARG, "row_program", "immediate operands are for row-value programs only");
    }
    return KTB_OK;
}

extern "C" int ktb_launch_row_program(ktb_ctx* ctx, const ktb_rowprog_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    const ktb_rowprog_args& a = *args;
    if (a.n_items <= 0 || a.rows_per_item <= 0) return KTB_OK;
    if (a.n_in < 1 || a.n_in > KTB_VM_MAX_IN || a.n_red < 0 || a.n_red > KTB_RP_MAX_RED || a.n_scal < 0 ||
        a.n_scal > KTB_RP_MAX_SCAL || a.n_in + a.n_scal > KTB_VM_REGS)
        return ktb_fail(ctx, KTB_E_ARG, "row_program", "bad operand / phase counts");
    if (a.cols < 8 || a.cols > 16384 || (a.cols & (a.cols - 1)) != 0)
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "cols must be a power of two in [8, 16384]");
    bool any_blocked = a.out.blocked != 0;
    for (int p = 0; p < a.n_red; ++p) any_blocked = any_blocked || a.red[p].blocked;
    if (a.n_blocks < 1 || a.n_blocks > 4096 || (!any_blocked && a.n_blocks != 1) || (a.out.blocked && a.out_per_row))
        return ktb_fail(ctx, KTB_E_ARG, "row_program", "bad column-block count");
    for (int k = 0; any_blocked && k <= a.n_in; ++k)
        if (a.blk_stride[k] % 8) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "block strides must be multiples of 8 elements");
    for (int k = 0; k <= a.n_in; ++k) {
        if (a.dtype[k] != KTB_F16 && a.dtype[k] != KTB_F32)
            return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "operand dtype must be f16 or f32");
        if (a.row_stride[k] % 8 && !(k == a.n_in && a.out_per_row))
            return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "row strides must be multiples of 8 elements");
    }
    if (a.n_side < 0 || a.n_side > KTB_RP_MAX_SIDE || (a.n_side && a.out_per_row))
        return ktb_fail(ctx, KTB_E_ARG, "row_program", "bad side result count");
    int rc;
    for (int s = 0; s < a.n_side; ++s) {
        if ((rc = rp_check_program(ctx, a.side[s].prog, a.n_red, true))) return rc;
        if (a.side[s].dtype != KTB_F16 && a.side[s].dtype != KTB_F32)
            return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "side result dtype must be f16 or f32");
    }
    for (int p = 0; p < a.n_red; ++p) {
        if ((rc = rp_check_program(ctx, a.red[p].prog, a.n_in + a.n_scal))) return rc;
        if (a.red[p].op != KTB_RP_ADD && a.red[p].op != KTB_RP_MAX && a.red[p].op != KTB_RP_MAXNUM)
            return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "reduction must be add or max");
    }
    if ((rc = rp_check_program(ctx, a.out.prog, a.out_per_row ? a.n_red : a.n_in + a.n_scal, a.out_per_row != 0))) return rc;
    for (int s = 0; s < a.n_scal; ++s) {
        if ((rc = rp_check_program(ctx, a.scal[s].prog, a.n_red, true))) return rc;
        if (a.scal[s].ready_after < -1 || a.scal[s].ready_after >= a.n_red || (s && a.scal[s].ready_after < a.scal[s - 1].ready_after))
            return ktb_fail(ctx, KTB_E_ARG, "row_program", "row scalars must be sorted by the last reduction they read");
    }
    // eight vectors per thread where the row is long enough (the fold pairs the same elements whatever the
    // split; fewer, longer threads per row need fewer exchanges between warps: layer norm 8192 x 1024 takes
    // 133 us with 8 vectors per thread, 145 with 4, 162 with 2, 221 with 1)
    const int vecs = a.cols / 8;
    int T = vecs / 8;
    if (T < 1) T = 1;
    if (T > 256) T = 256;
    // ... but few rows (of many column blocks, say) must still give every SM a couple of CTAs: more threads per row
    while (T < vecs && T < 256 && a.n_items * (int64_t)a.rows_per_item / (256 / T) < 2 * (int64_t)ctx->sm_count) T *= 2;
    const int NV = vecs / T;
    const int64_t total_rows = a.n_items * (int64_t)a.rows_per_item;
    if (total_rows >= (1ll << 31)) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "more than 2^31 rows");
    const int groups = 256 / T;
    const int64_t n_iter = (total_rows + groups - 1) / groups;
    int64_t blocks = (int64_t)ctx->sm_count * 8;
    if (blocks > n_iter) blocks = n_iter;
#ifndef KTB_RP_NO_NORM
    rp_norm nm;
    const bool matched = rp_match_norm(a, nm);
    if (matched && (nm.blocked || nm.r16)) {
        if (rp_try_norm_blocks(ctx, a, nm, total_rows)) {
            KTB_CHECK_LAUNCH(ctx, "ktb_row_norm_blocks_kernel");
            return KTB_OK;
        }
    } else if (matched) {
        // four vectors per thread (the row and its squares sit in registers): two CTAs per SM
#ifndef KTB_RP_NORM_VPT
#define KTB_RP_NORM_VPT 4
#endif
        int Tn = vecs / KTB_RP_NORM_VPT;
        if (Tn < 1) Tn = 1;
        if (Tn > 256) Tn = 256;
        const int NVn = vecs / Tn, gn = 256 / Tn;
        const int64_t iters = (total_rows + gn - 1) / gn;
        const unsigned bn = (unsigned)(iters < (int64_t)ctx->sm_count * 4 ? iters : (int64_t)ctx->sm_count * 4);
        switch (NVn) {
            case 1: rp_launch_norm<1>(ctx, a, nm, bn, Tn, total_rows); break;
            case 2: rp_launch_norm<2>(ctx, a, nm, bn, Tn, total_rows); break;
            case 4: rp_launch_norm<4>(ctx, a, nm, bn, Tn, total_rows); break;
            case 8: rp_launch_norm<8>(ctx, a, nm, bn, Tn, total_rows); break;
            default: return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "unsupported row width");
        }
        KTB_CHECK_LAUNCH(ctx, "ktb_row_norm_kernel");
        return KTB_OK;
    }
#endif
    static bool ready = false;
    if (!ready) {
        cudaFuncSetAttribute(ktb_row_program_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RP_REGS_BYTES);
        cudaFuncSetAttribute(ktb_row_program_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RP_REGS_BYTES);
        cudaFuncSetAttribute(ktb_row_program_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RP_REGS_BYTES);
        cudaFuncSetAttribute(ktb_row_program_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RP_REGS_BYTES);
        ready = true;
    }
    switch (NV) {
        case 1: ktb_row_program_kernel<1><<<(unsigned)blocks, 256, RP_REGS_BYTES, ctx->stream>>>(a, T, total_rows); break;
        case 2: ktb_row_program_kernel<2><<<(unsigned)blocks, 256, RP_REGS_BYTES, ctx->stream>>>(a, T, total_rows); break;
        case 4: ktb_row_program_kernel<4><<<(unsigned)blocks, 256, RP_REGS_BYTES, ctx->stream>>>(a, T, total_rows); break;
        case 8: ktb_row_program_kernel<8><<<(unsigned)blocks, 256, RP_REGS_BYTES, ctx->stream>>>(a, T, total_rows); break;
        default: return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_program", "unsupported row width");
    }
    KTB_CHECK_LAUNCH(ctx, "ktb_row_program_kernel");
    return KTB_OK;
}
