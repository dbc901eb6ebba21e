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
        case KTB_VM_MAX: return (a != a || b != b) ? __int_as_float(0x7fc00000) : fmaxf(a, b);
        case KTB_VM_MAXNUM: return fmaxf(a, b);
        case KTB_VM_MIN: return (a != a || b != b) ? __int_as_float(0x7fc00000) : fminf(a, b);
        case KTB_VM_MINNUM: return fminf(a, b);
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
            uint4 raw = *reinterpret_cast<const uint4*>(p);
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
            float4 a = *reinterpret_cast<const float4*>(p);
            float4 b = *reinterpret_cast<const float4*>(p + 4);
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
            *reinterpret_cast<uint4*>(p) = raw;
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) p[i] = __float2half_rn(x[i]);
        }
    } else {
        float* p = reinterpret_cast<float*>(base) + elem_off;
        if (V == 8) {
            *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
            *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) p[i] = x[i];
        }
    }
}

// Register-only evaluation for programs in single-assignment form (op i writes register
// n_in + i, which is how the host emits them).  Operands are fetched with predicated moves over
// the registers defined so far, so nothing is indexed dynamically and nothing lives in local
// memory.  Used where a warp runs the program on 4-element slices (row gather / scatter).
#define KTB_VM_SEL_OPS 8
template <int V, int NIN>
static __device__ __forceinline__ void ktb_vm_run_sel(const ktb_vm_program& prog, const float (&in)[NIN][V],
                                                      float (&out)[V]) {
    float r[NIN + KTB_VM_SEL_OPS][V];
#pragma unroll
    for (int k = 0; k < NIN; ++k)
#pragma unroll
        for (int v = 0; v < V; ++v) r[k][v] = in[k][v];
    const int n_in = prog.n_in;
#pragma unroll
    for (int i = 0; i < KTB_VM_SEL_OPS; ++i) {
#pragma unroll
        for (int v = 0; v < V; ++v) r[NIN + i][v] = 0.f;
        if (i < prog.n_ops) {
            const ktb_vm_op op = prog.ops[i];
            const int ia = op.a < n_in ? op.a : op.a - n_in + NIN;
            const int ib = op.b < n_in ? op.b : op.b - n_in + NIN;
            const int ic = op.c < n_in ? op.c : op.c - n_in + NIN;
            float av[V], bv[V], cv[V];
#pragma unroll
            for (int v = 0; v < V; ++v) av[v] = bv[v] = cv[v] = 0.f;
#pragma unroll
            for (int s = 0; s < NIN + i; ++s) {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    av[v] = s == ia ? r[s][v] : av[v];
                    bv[v] = s == ib ? r[s][v] : bv[v];
                    cv[v] = s == ic ? r[s][v] : cv[v];
                }
            }
            const int code = op.opcode & 0xff;
            const bool r16 = (op.opcode & KTB_VM_ROUND16) != 0;
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float x = ktb_vm_apply(code, av[v], bv[v], cv[v], op.imm);
                r[NIN + i][v] = r16 ? ktb_round16(x) : x;
            }
        }
    }
    const int ir = prog.result_reg < n_in ? prog.result_reg : prog.result_reg - n_in + NIN;
#pragma unroll
    for (int v = 0; v < V; ++v) out[v] = 0.f;
#pragma unroll
    for (int s = 0; s < NIN + KTB_VM_SEL_OPS; ++s)
#pragma unroll
        for (int v = 0; v < V; ++v) out[v] = s == ir ? r[s][v] : out[v];
}
