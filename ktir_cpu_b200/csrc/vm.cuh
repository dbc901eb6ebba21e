// Register-program evaluator shared by the streaming and scatter kernels.
// A program is a short straight-line list of ops over f32 registers holding V
// elements each.  NumPy evaluates f16 tiles by computing in f32 and rounding to
// f16 after every ufunc (ktir_cpu/dialects/_helpers.py:39-54); KTB_VM_ROUND16
// reproduces that rounding point.  No FMA contraction: the library is compiled
// with --fmad=false so a*b+c keeps two roundings like two separate NumPy calls.
#pragma once
#include "common.cuh"

static __device__ __forceinline__ float ktb_vm_apply(int op, float a, float b, float c, float imm) {
    switch (op) {
        case KTB_VM_MOV: return a;
        case KTB_VM_CONST: return imm;
        case KTB_VM_ADD: return a + b;
        case KTB_VM_SUB: return a - b;
        case KTB_VM_MUL: return a * b;
        case KTB_VM_DIV: return a / b;
        // NumPy's selection rules (np.maximum / np.fmax / np.minimum / np.fmin on half and float): the
        // first operand wins a tie, so max(-0, +0) = -0 and max(+0, -0) = +0
        case KTB_VM_MAX: return (a >= b || a != a) ? a : b;
        case KTB_VM_MAXNUM: return (a >= b || b != b) ? a : b;
        case KTB_VM_MIN: return (a <= b || a != a) ? a : b;
        case KTB_VM_MINNUM: return (a <= b || b != b) ? a : b;
        case KTB_VM_NEG: return -a;
        case KTB_VM_ABS: return fabsf(a);
        case KTB_VM_EXP: return expf(a);
        case KTB_VM_LOG: return logf(a);
        case KTB_VM_LOG2: return log2f(a);
        case KTB_VM_SQRT: return sqrtf(a);
        case KTB_VM_RSQRT: return 1.0f / sqrtf(a);
        case KTB_VM_TANH: return tanhf(a);
        case KTB_VM_SIN: return sinf(a);
        case KTB_VM_COS: return cosf(a);
        case KTB_VM_FMA: return __fadd_rn(__fmul_rn(a, b), c);
        default: return a;
    }
}

// Runs `prog` on registers preloaded with the inputs; returns the result register.
template <int V>
static __device__ __forceinline__ void ktb_vm_run(const ktb_vm_program& prog,
                                                  float (&regs)[KTB_VM_REGS][V], float (&out)[V]) {
    for (int i = 0; i < prog.n_ops; ++i) {
        const ktb_vm_op op = prog.ops[i];
        const int code = op.opcode & 0xff;
        const bool r16 = (op.opcode & KTB_VM_ROUND16) != 0;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float x = ktb_vm_apply(code, regs[op.a][v], regs[op.b][v], regs[op.c][v], op.imm);
            regs[op.dst][v] = r16 ? ktb_round16(x) : x;
        }
    }
#pragma unroll
    for (int v = 0; v < V; ++v) out[v] = regs[prog.result_reg][v];
}

// 8-element vector load/store of f16 or f32 data as f32 values.
template <int V>
static __device__ __forceinline__ void ktb_load_vec(const void* base, int64_t elem_off, int dtype, float (&x)[V]) {
    if (dtype == KTB_F16) {
        const __half* p = reinterpret_cast<const __half*>(base) + elem_off;
        if (V == 8) {
            uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p));      // touched once: do not keep it in L2
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 f = __half22float2(h[i]);
                x[2 * i] = f.x;
                x[2 * i + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) x[i] = __half2float(p[i]);
        }
    } else {
        const float* p = reinterpret_cast<const float*>(base) + elem_off;
        if (V == 8) {
            float4 a = __ldcs(reinterpret_cast<const float4*>(p));
            float4 b = __ldcs(reinterpret_cast<const float4*>(p + 4));
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
            x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) x[i] = p[i];
        }
    }
}

template <int V>
static __device__ __forceinline__ void ktb_store_vec(void* base, int64_t elem_off, int dtype, const float (&x)[V]) {
    if (dtype == KTB_F16) {
        __half* p = reinterpret_cast<__half*>(base) + elem_off;
        if (V == 8) {
            uint4 raw;
            __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
            __stcs(reinterpret_cast<uint4*>(p), raw);
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) p[i] = __float2half_rn(x[i]);
        }
    } else {
        float* p = reinterpret_cast<float*>(base) + elem_off;
        if (V == 8) {
            __stcs(reinterpret_cast<float4*>(p), make_float4(x[0], x[1], x[2], x[3]));
            __stcs(reinterpret_cast<float4*>(p + 4), make_float4(x[4], x[5], x[6], x[7]));
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) p[i] = x[i];
        }
    }
}

// Compact evaluator for the row gather / scatter kernels: the register file lives in shared
// memory (register k of a thread is regs[k * stride], one float4 per thread, conflict-free), so
// operands can be indexed dynamically without local memory, and the routine is a single
// out-of-line copy, which keeps the kernels small enough for the instruction cache.  The opcode
// is decoded once per op, not once per element.
#define KTB_VM4(EXPR)                                                                      \
    {                                                                                      \
        float a, b, c;                                                                     \
        a = A.x; b = B.x; c = Cc.x; R.x = (EXPR);                                          \
        a = A.y; b = B.y; c = Cc.y; R.y = (EXPR);                                          \
        a = A.z; b = B.z; c = Cc.z; R.z = (EXPR);                                          \
        a = A.w; b = B.w; c = Cc.w; R.w = (EXPR);                                          \
        (void)a; (void)b; (void)c;                                                         \
    }                                                                                      \
    break;

static __device__ __noinline__ float4 ktb_vm_run_smem4(const ktb_vm_program& prog, float4* regs, int stride) {
    for (int i = 0; i < prog.n_ops; ++i) {
        const ktb_vm_op op = prog.ops[i];
        const float4 A = regs[op.a * stride], B = regs[op.b * stride], Cc = regs[op.c * stride];
        const float imm = op.imm;
        float4 R = A;
        switch (op.opcode & 0xff) {
            case KTB_VM_MOV: break;
            case KTB_VM_CONST: R = make_float4(imm, imm, imm, imm); break;
            case KTB_VM_ADD: KTB_VM4(a + b)
            case KTB_VM_SUB: KTB_VM4(a - b)
            case KTB_VM_MUL: KTB_VM4(a * b)
            case KTB_VM_DIV: KTB_VM4(a / b)
            case KTB_VM_MAXNUM: KTB_VM4((a >= b || b != b) ? a : b)
            case KTB_VM_MINNUM: KTB_VM4((a <= b || b != b) ? a : b)
            case KTB_VM_NEG: KTB_VM4(-a)
            case KTB_VM_ABS: KTB_VM4(fabsf(a))
            default: KTB_VM4(ktb_vm_apply(op.opcode & 0xff, a, b, c, imm))
        }
        if (op.opcode & KTB_VM_ROUND16)
            R = make_float4(ktb_round16(R.x), ktb_round16(R.y), ktb_round16(R.z), ktb_round16(R.w));
        regs[op.dst * stride] = R;
    }
    return regs[prog.result_reg * stride];
}
