// Fused row softmax: one pass over HBM (the row is read once and written once).
//
// A row of `cols` elements is held in registers by a group of T threads
// (T = cols/64, between 1 and 256; 8 vectors of 8 elements per thread at most),
// thread t owning the 16-byte vectors j*T + t, so global accesses are unit-stride
// and 128-bit.  A CTA of 256 threads carries 256/T independent row groups; groups
// wider than a warp synchronise on their own named barrier, narrower ones need no
// barrier at all, so many rows are in flight per SM and the kernel stays HBM-bound.
//
// Both reductions fold x[i] (op) x[i + h] for h = cols/2 ... 1 — the halving order
// of the reference's linalg.reduce (ktir_cpu/dialects/linalg_ops.py:86-133): first
// across a thread's own vectors, then across the warps of the group (one shared
// memory exchange, combined in the same pairing), then by warp shuffle, then
// across the 8 elements of the remaining vector.
#include <stdlib.h>

#include "row_fold.cuh"

static __device__ __forceinline__ float sm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int NV, bool MAXNUM, bool R16>
__global__ void __launch_bounds__(256, NV >= 8 ? 2 : 3) ktb_row_softmax_kernel(const ktb_softmax_args a, int T, int64_t total_rows) {
    __shared__ float xchg[256 * 8];
    __shared__ float bcast[8];
    const int groups = 256 / T;
    const int group = threadIdx.x / T;
    const int t = threadIdx.x - group * T;
    const __half* in16 = reinterpret_cast<const __half*>(a.arena);
    const float* in32 = reinterpret_cast<const float*>(a.arena);

    // the trip count is the same for every thread of the CTA (shuffles use full-warp masks);
    // a group past the last row recomputes row 0 and skips the store
    const int64_t n_iter = (total_rows + groups - 1) / groups;
    for (int64_t it = blockIdx.x; it < n_iter; it += gridDim.x) {
        const bool live = it * groups + group < total_rows;
        const int64_t row = live ? it * groups + group : 0;
        // (32-bit: the launcher refuses more than 2^31 rows; a 64-bit division costs as much as a fifth of the row's arithmetic)
        const int64_t item = (uint32_t)row / (uint32_t)a.rows_per_item;
        const int64_t r = row - item * a.rows_per_item;
        const int64_t in_off = a.dev_item_offsets[item * 2] + r * a.in_row_stride;
        const int64_t out_off = a.dev_item_offsets[item * 2 + 1] + r * a.out_row_stride;

        float x[NV][8];
        if (a.in_dtype == KTB_F16) {
            uint4 raw[NV];
#pragma unroll
            for (int j = 0; j < NV; ++j)
                raw[j] = __ldcs(reinterpret_cast<const uint4*>(in16 + in_off + ((int64_t)j * T + t) * 8));
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const __half2* h = reinterpret_cast<const __half2*>(&raw[j]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(h[i]);
                    x[j][2 * i] = f.x;
                    x[j][2 * i + 1] = f.y;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const float* p = in32 + in_off + ((int64_t)j * T + t) * 8;
                const float4 lo = __ldcs(reinterpret_cast<const float4*>(p));
                const float4 hi = __ldcs(reinterpret_cast<const float4*>(p + 4));
                x[j][0] = lo.x; x[j][1] = lo.y; x[j][2] = lo.z; x[j][3] = lo.w;
                x[j][4] = hi.x; x[j][5] = hi.y; x[j][6] = hi.z; x[j][7] = hi.w;
            }
        }

        float mx = row_fold<NV, 0, MAXNUM, R16>(x, T, t, group, xchg, bcast);
        mx = sm_max<MAXNUM>(mx, a.max_init);
        // f32 path: exp(x - mx) = 2^(x*log2e - mx*log2e), one FMA and one MUFU per element
        // (relative error <= ~1e-6 for |x - mx| < 16, inside the 1e-5 f32 tolerance).
        // f16 path keeps the reference's rounding points: round(x - mx), round(exp(.)).
        const float mxs = mx * 1.4426950408889634f;
#pragma unroll
        for (int j = 0; j < NV; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (R16) {
                    const float d = ktb_round16(x[j][k] - mx);
                    x[j][k] = ktb_round16(expf(d));
                } else {
                    x[j][k] = sm_ex2(__fmaf_rn(x[j][k], 1.4426950408889634f, -mxs));
                }
            }
        float sum = row_fold<NV, 1, MAXNUM, R16>(x, T, t, group, xchg, bcast);
        sum = sum + a.sum_init;
        if (R16) sum = ktb_round16(sum);
        const float inv = 1.0f / sum;

        if (!live) continue;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int64_t e = out_off + ((int64_t)j * T + t) * 8;
            float y[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) y[k] = R16 ? x[j][k] / sum : x[j][k] * inv;
            if (a.out_dtype == KTB_F16) {
                uint4 raw;
                __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
                __stcs(reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.arena) + e), raw);
            } else {
                float* p = reinterpret_cast<float*>(a.arena) + e;
                __stcs(reinterpret_cast<float4*>(p), make_float4(y[0], y[1], y[2], y[3]));
                __stcs(reinterpret_cast<float4*>(p + 4), make_float4(y[4], y[5], y[6], y[7]));
            }
        }
    }
}

// ---- fast path: f16 input, f32 statistics -------------------------------------------------------
// max is exact in any order, so it is taken on the packed f16 data (one HMNMX2 per two elements);
// exp is ex2.approx of an FMA-scaled argument and therefore not bit-comparable with NumPy anyway,
// so the sum uses a plain per-thread accumulation + butterfly instead of the halving order.
// About 6 instructions per element; the row is read once and written once.
static __device__ __forceinline__ void sm_row_exp(const uint4& raw, float mxs, float (&p)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        p[2 * i] = sm_ex2(__fmaf_rn(f.x, 1.4426950408889634f, -mxs));
        p[2 * i + 1] = sm_ex2(__fmaf_rn(f.y, 1.4426950408889634f, -mxs));
    }
}

// Two f32 values in one 64-bit register: Blackwell issues fma / add / mul on such a pair as ONE instruction,
// which takes a third off the instruction count of a row (the kernel is issue-bound next to HBM-bound).
static __device__ __forceinline__ uint64_t sm_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
static __device__ __forceinline__ void sm_unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
static __device__ __forceinline__ uint64_t sm_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
static __device__ __forceinline__ uint64_t sm_add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
static __device__ __forceinline__ uint64_t sm_mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// exp of the 8 values of one vector, parked in place as f16: p * 2^15 = 2^(x log2e - (m log2e - 15)), the scale
// folded into the exponent (0 < p <= 1, so p * 2^15 keeps 11 significant bits down to p = 2^-29); the two
// accumulators collect the same scaled values in f32.
static __device__ __forceinline__ void sm_row_exp_park(uint4& raw, uint64_t l2e2, uint64_t negm2, uint64_t& acc0, uint64_t& acc1) {
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        float x0, x1;
        sm_unpack2(sm_fma2(sm_pack2(f.x, f.y), l2e2, negm2), x0, x1);
        const float p0 = sm_ex2(x0), p1 = sm_ex2(x1);
        if (i & 1) acc1 = sm_add2(acc1, sm_pack2(p0, p1));
        else acc0 = sm_add2(acc0, sm_pack2(p0, p1));
        h[i] = __floats2half2_rn(p0, p1);
    }
}

// The row stays in registers as packed f16 (NV x 4 registers) instead of NV x 8 f32 values: half
// the registers, twice the resident rows per SM.  f16 output: exp is evaluated once and parked as
// f16 (x 2^15) in the registers the input occupied (one extra rounding, <= 2^-11 relative, inside
// the f16 tolerance of this op); f32 output evaluates exp twice (same instruction sequence, so
// the same bits) and loses nothing.
template <int NV, bool MAXNUM>
__global__ void __launch_bounds__(256, NV >= 16 ? 2 : NV >= 8 ? 4 : 6)
ktb_row_softmax_fast_kernel(const ktb_softmax_args a, int T, int64_t total_rows) {
    __shared__ float xmax[8], xsum[8];            // one slot per warp of the CTA
    const int groups = 256 / T;
    const int group = threadIdx.x / T;
    const int t = threadIdx.x - group * T;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpg = T >> 5;                        // warps per row group (0 when T < 32)
    const __half* in16 = reinterpret_cast<const __half*>(a.arena);
    const int w = T < 32 ? T : 32;
    const int64_t n_iter = (total_rows + groups - 1) / groups;
    const bool pack = a.out_dtype == KTB_F16;
    for (int64_t it = blockIdx.x; it < n_iter; it += gridDim.x) {
        const bool live = it * groups + group < total_rows;
        const int64_t row = live ? it * groups + group : 0;
        // (32-bit: the launcher refuses more than 2^31 rows; a 64-bit division costs as much as a fifth of the row's arithmetic)
        const int64_t item = (uint32_t)row / (uint32_t)a.rows_per_item;
        const int64_t r = row - item * a.rows_per_item;
        const int64_t in_off = a.dev_item_offsets[item * 2] + r * a.in_row_stride;
        const int64_t out_off = a.dev_item_offsets[item * 2 + 1] + r * a.out_row_stride;
        const uint4* src = reinterpret_cast<const uint4*>(in16 + in_off) + t;

        uint4 raw[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) raw[j] = __ldcs(src + (int64_t)j * T);

        __half2 m2 = *reinterpret_cast<const __half2*>(&raw[0].x);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const __half2* h = reinterpret_cast<const __half2*>(&raw[j]);
#pragma unroll
            for (int i = 0; i < 4; ++i) m2 = MAXNUM ? __hmax2(m2, h[i]) : __hmax2_nan(m2, h[i]);
        }
        for (int d = w >> 1; d >= 1; d >>= 1) {
            uint32_t o = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<uint32_t*>(&m2), d, w);
            const __half2 oh = *reinterpret_cast<__half2*>(&o);
            m2 = MAXNUM ? __hmax2(m2, oh) : __hmax2_nan(m2, oh);
        }
        float mx = sm_max<MAXNUM>(__low2float(m2), __high2float(m2));
        if (wpg > 1) {
            if (lane == 0) xmax[warp] = mx;
            group_barrier(1 + group, T);
            const int w0 = warp - (warp % wpg);
            mx = xmax[w0];
            for (int k = 1; k < wpg; ++k) mx = sm_max<MAXNUM>(mx, xmax[w0 + k]);
        }
        mx = sm_max<MAXNUM>(mx, a.max_init);
        const float mxs = mx * 1.4426950408889634f;

        float sum;
        if (pack) {
            const uint64_t l2e2 = sm_pack2(1.4426950408889634f, 1.4426950408889634f);
            const uint64_t negm2 = sm_pack2(15.f - mxs, 15.f - mxs);
            uint64_t acc0 = sm_pack2(0.f, 0.f), acc1 = acc0;
#pragma unroll
            for (int j = 0; j < NV; ++j) sm_row_exp_park(raw[j], l2e2, negm2, acc0, acc1);
            float a0, a1, b0, b1;
            sm_unpack2(acc0, a0, a1);
            sm_unpack2(acc1, b0, b1);
            sum = (a0 + a1) + (b0 + b1);
        } else {
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                float q[8];
                sm_row_exp(raw[j], mxs, q);
                s0 += q[0] + q[1];
                s1 += q[2] + q[3];
                s2 += q[4] + q[5];
                s3 += q[6] + q[7];
            }
            sum = (s0 + s1) + (s2 + s3);
        }
        for (int d = w >> 1; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d, w);
        if (wpg > 1) {
            if (lane == 0) xsum[warp] = sum;
            group_barrier(1 + group, T);
            const int w0 = warp - (warp % wpg);
            sum = xsum[w0];
            for (int k = 1; k < wpg; ++k) sum += xsum[w0 + k];
        }
        // (the parked values and their sum carry the factor 2^15)
        const float inv = 1.0f / (pack ? sum + a.sum_init * 32768.f : sum + a.sum_init);
        if (!live) continue;
        if (pack) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.arena) + out_off) + t;
            const uint64_t inv2 = sm_pack2(inv, inv);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                uint4 o;
                __half2* h = reinterpret_cast<__half2*>(&o);
                const __half2* hp = reinterpret_cast<const __half2*>(&raw[j]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(hp[i]);
                    float y0, y1;
                    sm_unpack2(sm_mul2(sm_pack2(f.x, f.y), inv2), y0, y1);
                    h[i] = __floats2half2_rn(y0, y1);
                }
                __stcs(dst + (int64_t)j * T, o);
            }
        } else {
            // opaque to the optimiser: otherwise the converted values of the first evaluation are
            // kept alive for the second one, which is the register footprint this form avoids
#pragma unroll
            for (int j = 0; j < NV; ++j)
                asm volatile("" : "+r"(raw[j].x), "+r"(raw[j].y), "+r"(raw[j].z), "+r"(raw[j].w));
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                float pj[8];
                sm_row_exp(raw[j], mxs, pj);
                float* q = reinterpret_cast<float*>(a.arena) + out_off + ((int64_t)j * T + t) * 8;
                __stcs(reinterpret_cast<float4*>(q), make_float4(pj[0] * inv, pj[1] * inv, pj[2] * inv, pj[3] * inv));
                __stcs(reinterpret_cast<float4*>(q + 4), make_float4(pj[4] * inv, pj[5] * inv, pj[6] * inv, pj[7] * inv));
            }
        }
    }
}

template <int NV>
static void launch_softmax(ktb_ctx* ctx, const ktb_softmax_args& a, int T, int64_t total_rows) {
    const int groups = 256 / T;
    const int64_t n_iter = (total_rows + groups - 1) / groups;
    int64_t blocks = (int64_t)ctx->sm_count * 8;
    if (blocks > n_iter) blocks = n_iter;
    const bool mn = a.max_is_maxnum != 0, r16 = a.f16_arith != 0;
    if (a.in_dtype == KTB_F16 && !r16) {
        blocks = n_iter < (int64_t)ctx->sm_count * 8 ? n_iter : (int64_t)ctx->sm_count * 8;
        if (mn) ktb_row_softmax_fast_kernel<NV, true><<<(unsigned)blocks, 256, 0, ctx->stream>>>(a, T, total_rows);
        else ktb_row_softmax_fast_kernel<NV, false><<<(unsigned)blocks, 256, 0, ctx->stream>>>(a, T, total_rows);
        return;
    }
    if constexpr (NV <= 8) {
#define KTB_SM_LAUNCH(MN, R) ktb_row_softmax_kernel<NV, MN, R><<<(unsigned)blocks, 256, 0, ctx->stream>>>(a, T, total_rows)
        if (mn && r16) KTB_SM_LAUNCH(true, true);
        else if (mn) KTB_SM_LAUNCH(true, false);
        else if (r16) KTB_SM_LAUNCH(false, true);
        else KTB_SM_LAUNCH(false, false);
#undef KTB_SM_LAUNCH
    }
}

extern "C" int ktb_launch_row_softmax(ktb_ctx* ctx, const ktb_softmax_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    const ktb_softmax_args& a = *args;
    if (a.n_items <= 0 || a.rows_per_item <= 0) return KTB_OK;
    if (a.cols < 8 || a.cols > 16384 || (a.cols & (a.cols - 1)) != 0)
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_softmax", "cols must be a power of two in [8, 16384]");
    if ((a.in_dtype != KTB_F16 && a.in_dtype != KTB_F32) || (a.out_dtype != KTB_F16 && a.out_dtype != KTB_F32))
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_softmax", "dtype must be f16 or f32");
    if ((a.in_row_stride % 8) || (a.out_row_stride % 8))
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_softmax", "row strides must be multiples of 8 elements");
    const int vecs = a.cols / 8;
    const int per_thread = 8;         // 16-byte vectors per thread
    int T = vecs / per_thread;
    if (T < 1) T = 1;
    if (T > 256) T = 256;             // ... unless the row is wider than 16384 elements
    const int NV = vecs / T;
    const int64_t total_rows = a.n_items * (int64_t)a.rows_per_item;
    if (total_rows >= (1ll << 31)) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_softmax", "more than 2^31 rows");
    switch (NV) {
        case 1: launch_softmax<1>(ctx, a, T, total_rows); break;
        case 2: launch_softmax<2>(ctx, a, T, total_rows); break;
        case 4: launch_softmax<4>(ctx, a, T, total_rows); break;
        case 8: launch_softmax<8>(ctx, a, T, total_rows); break;
        case 16:
            if (a.in_dtype == KTB_F16 && !a.f16_arith) { launch_softmax<16>(ctx, a, T, total_rows); break; }
            return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_softmax", "unsupported row width");
        default: return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_softmax", "unsupported row width");
    }
    KTB_CHECK_LAUNCH(ctx, "ktb_row_softmax_kernel");
    return KTB_OK;
}
