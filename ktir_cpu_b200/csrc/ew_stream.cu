// Fused tile load -> elementwise program -> tile store, all grid cores and loop
// iterations of one KTIR statement in a single launch.  HBM-bound: every thread
// moves 16-byte vectors (8 f16 / two float4) with unit-stride, fully coalesced
// accesses; the op itself is a handful of FP32 instructions per vector.
//
// Reference path replaced: ktdp.load / arith.* / ktdp.store executed per core by
// KTIRInterpreter._execute_op (ktir_cpu/interpreter.py:196-281) through
// MemoryOps.load/store (ktir_cpu/ops/memory_ops.py:723-865).
#include "vm.cuh"

// SPECIAL >= 0: the program is the single op SPECIAL applied to inputs (0, 1);
// SPECIAL < 0: general register program.
template <int V, int SPECIAL, typename IDX>
__global__ void __launch_bounds__(256) ktb_ew_stream_kernel(const ktb_ew_args args, uint32_t chunks_per_row,
                                                            uint32_t chunks_per_item, uint64_t total_chunks) {
    const uint64_t chunk64 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (chunk64 >= total_chunks) return;
    const IDX chunk = (IDX)chunk64;
    const IDX item = chunk / (IDX)chunks_per_item;
    const uint32_t rem = (uint32_t)(chunk - item * (IDX)chunks_per_item);
    const uint32_t row = rem / chunks_per_row;
    const uint32_t col = (rem - row * chunks_per_row) * V;
    const int n_in = args.program.n_in;
    const int64_t* offs = args.dev_item_offsets + (int64_t)item * (n_in + 1);

    float out[V];
    if (SPECIAL >= 0) {
        float a[V], b[V];
        ktb_load_vec<V>(args.arena, offs[0] + (int64_t)row * args.row_stride[0] + col, args.dtype[0], a);
        if (n_in > 1)
            ktb_load_vec<V>(args.arena, offs[1] + (int64_t)row * args.row_stride[1] + col, args.dtype[1], b);
        const bool r16 = (args.program.ops[0].opcode & KTB_VM_ROUND16) != 0;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float x = ktb_vm_apply(SPECIAL, a[v], n_in > 1 ? b[v] : 0.f, 0.f, args.program.ops[0].imm);
            out[v] = r16 ? ktb_round16(x) : x;
        }
    } else {
        float regs[KTB_VM_REGS][V];
        for (int i = 0; i < n_in; ++i) {
            float x[V];
            ktb_load_vec<V>(args.arena, offs[i] + (int64_t)row * args.row_stride[i] + col, args.dtype[i], x);
#pragma unroll
            for (int v = 0; v < V; ++v) regs[i][v] = x[v];
        }
        ktb_vm_run<V>(args.program, regs, out);
    }
    ktb_store_vec<V>(args.arena, offs[n_in] + (int64_t)row * args.row_stride[n_in] + col, args.dtype[n_in], out);
}

// All operands f16, one op: every thread takes U chunks of 8 elements, a block 256 * U consecutive chunks
// (thread t the chunks t, t + 256, ...: each warp access stays one contiguous 512-byte run), and issues the
// 16-byte loads of all its chunks before it touches any of them.  Chunk indices are 32-bit when they fit: the
// two divisions that find a chunk's item, row and column cost a multiple of the add itself in 64 bits.
// Vector add of 2^26 elements: 71.7 us with the general kernel, 63.5 with U = 1, 59.4 with U = 2, 63.5 with
// U = 4, 73.7 with U = 8 (fewer resident threads).
#ifndef KTB_EW_U
#define KTB_EW_U 2
#endif
template <int U, int OP, typename IDX>
__global__ void __launch_bounds__(256) ktb_ew_f16_kernel(const ktb_ew_args args, uint32_t chunks_per_row,
                                                         uint32_t chunks_per_item, uint64_t total_chunks) {
    const uint64_t first = (uint64_t)blockIdx.x * (256u * U) + threadIdx.x;
    const bool two = args.program.n_in > 1;
    const int n_in = args.program.n_in;
    const __half* arena = reinterpret_cast<const __half*>(args.arena);
    uint4 ra[U], rb[U];
    int64_t dst[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const uint64_t chunk = first + (uint64_t)u * 256u;
        dst[u] = -1;
        if (chunk < total_chunks) {
            const IDX c = (IDX)chunk;
            const IDX item = c / (IDX)chunks_per_item;
            const uint32_t rem = (uint32_t)(c - item * (IDX)chunks_per_item);
            const uint32_t row = rem / chunks_per_row;
            const uint32_t col = (rem - row * chunks_per_row) * 8;
            const int64_t* offs = args.dev_item_offsets + (int64_t)item * (n_in + 1);
            ra[u] = __ldcs(reinterpret_cast<const uint4*>(arena + offs[0] + (int64_t)row * args.row_stride[0] + col));
            if (two) rb[u] = __ldcs(reinterpret_cast<const uint4*>(arena + offs[1] + (int64_t)row * args.row_stride[1] + col));
            dst[u] = offs[n_in] + (int64_t)row * args.row_stride[n_in] + col;
        }
    }
    const bool r16 = (args.program.ops[0].opcode & KTB_VM_ROUND16) != 0;
    const float imm = args.program.ops[0].imm;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        if (dst[u] < 0) continue;
        const __half2* ha = reinterpret_cast<const __half2*>(&ra[u]);
        const __half2* hb = reinterpret_cast<const __half2*>(&rb[u]);
        uint4 o;
        __half2* ho = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __half22float2(ha[i]);
            const float2 b = two ? __half22float2(hb[i]) : make_float2(0.f, 0.f);
            float x = ktb_vm_apply(OP, a.x, b.x, 0.f, imm), y = ktb_vm_apply(OP, a.y, b.y, 0.f, imm);
            if (r16) {
                x = ktb_round16(x);
                y = ktb_round16(y);
            }
            ho[i] = __floats2half2_rn(x, y);
        }
        __stcs(reinterpret_cast<uint4*>(const_cast<__half*>(arena) + dst[u]), o);
    }
}

template <int V>
static void launch_ew(ktb_ctx* ctx, const ktb_ew_args& a, int special, uint32_t cpr, uint32_t cpi, uint64_t total) {
    const unsigned blocks = (unsigned)((total + 255) / 256);
    bool f16 = V == 8 && special >= 0;
    for (int i = 0; i <= a.program.n_in; ++i) f16 = f16 && a.dtype[i] == KTB_F16;
    const unsigned fblocks = (unsigned)((total + 256 * KTB_EW_U - 1) / (256 * KTB_EW_U));
#define KTB_EW_CASE(OP)                                                                                   \
    case OP:                                                                                              \
        if (f16 && total < (1ull << 32))                                                                  \
            ktb_ew_f16_kernel<KTB_EW_U, OP, uint32_t><<<fblocks, 256, 0, ctx->stream>>>(a, cpr, cpi, total); \
        else if (f16)                                                                                     \
            ktb_ew_f16_kernel<KTB_EW_U, OP, uint64_t><<<fblocks, 256, 0, ctx->stream>>>(a, cpr, cpi, total); \
        else if (total < (1ull << 32))                                                                    \
            ktb_ew_stream_kernel<V, OP, uint32_t><<<blocks, 256, 0, ctx->stream>>>(a, cpr, cpi, total);   \
        else                                                                                              \
            ktb_ew_stream_kernel<V, OP, uint64_t><<<blocks, 256, 0, ctx->stream>>>(a, cpr, cpi, total);   \
        break;
    switch (special) {
        KTB_EW_CASE(KTB_VM_MOV)
        KTB_EW_CASE(KTB_VM_ADD)
        KTB_EW_CASE(KTB_VM_SUB)
        KTB_EW_CASE(KTB_VM_MUL)
        KTB_EW_CASE(KTB_VM_DIV)
        KTB_EW_CASE(KTB_VM_MAX)
        KTB_EW_CASE(KTB_VM_MIN)
        default:
            if (total < (1ull << 32)) ktb_ew_stream_kernel<V, -1, uint32_t><<<blocks, 256, 0, ctx->stream>>>(a, cpr, cpi, total);
            else ktb_ew_stream_kernel<V, -1, uint64_t><<<blocks, 256, 0, ctx->stream>>>(a, cpr, cpi, total);
    }
#undef KTB_EW_CASE
}

extern "C" int ktb_launch_ew_stream(ktb_ctx* ctx, const ktb_ew_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    const ktb_ew_args& a = *args;
    const ktb_vm_program& p = a.program;
    if (p.n_in < 1 || p.n_in > KTB_VM_MAX_IN || p.n_ops < 0 || p.n_ops > KTB_VM_MAX_OPS ||
        p.result_reg < 0 || p.result_reg >= KTB_VM_REGS)
        return ktb_fail(ctx, KTB_E_ARG, "ew_stream", "bad program header");
    for (int i = 0; i < p.n_ops; ++i) {
        const ktb_vm_op& o = p.ops[i];
        if ((o.opcode & 0xff) >= KTB_VM_NOPS || o.dst < 0 || o.dst >= KTB_VM_REGS || o.a < 0 ||
            o.a >= KTB_VM_REGS || o.b < 0 || o.b >= KTB_VM_REGS || o.c < 0 || o.c >= KTB_VM_REGS)
            return ktb_fail(ctx, KTB_E_ARG, "ew_stream", "bad program op");
    }
    for (int i = 0; i <= p.n_in; ++i)
        if (a.dtype[i] != KTB_F16 && a.dtype[i] != KTB_F32)
            return ktb_fail(ctx, KTB_E_UNSUPPORTED, "ew_stream", "operand dtype must be f16 or f32");
    if (a.n_items <= 0 || a.rows <= 0 || a.cols <= 0) return KTB_OK;

    // Single-op programs over inputs (0,1) run the specialised kernel.
    int special = -1;
    // (a binary op whose two operands are the SAME input tile, x + x, takes the general path)
    if (p.n_ops == 1 && p.ops[0].a == 0 && p.ops[0].dst == p.result_reg &&
        ((p.ops[0].opcode & 0xff) == KTB_VM_MOV || (p.n_in >= 2 && p.ops[0].b == 1)))
        special = p.ops[0].opcode & 0xff;
    if (p.n_ops == 0 && p.result_reg == 0) special = KTB_VM_MOV;

    const bool vec = a.vector_ok && (a.cols % 8) == 0;
    if (vec) {
        const uint32_t cpr = a.cols / 8;
        const uint64_t cpi64 = (uint64_t)cpr * a.rows;
        if (cpi64 >= (1ull << 31)) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "ew_stream", "tile too large");
        launch_ew<8>(ctx, a, special, cpr, (uint32_t)cpi64, cpi64 * a.n_items);
    } else {
        const uint64_t cpi64 = (uint64_t)a.cols * a.rows;
        if (cpi64 >= (1ull << 31)) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "ew_stream", "tile too large");
        launch_ew<1>(ctx, a, special, a.cols, (uint32_t)cpi64, cpi64 * a.n_items);
    }
    KTB_CHECK_LAUNCH(ctx, "ktb_ew_stream_kernel");
    return KTB_OK;
}
