// Fused row softmax: one pass over HBM (read the row once, write it once).
// A row of `cols` elements is held in registers by T = min(256, cols/8) threads,
// thread t owning 16-byte vectors j*T + t, so global accesses are unit-stride
// and 128-bit.  Both reductions fold x[i] (op) x[i + h] for h = cols/2 ... 1 —
// the halving order of the reference's linalg.reduce
// (ktir_cpu/dialects/linalg_ops.py:86-133) — first across a thread's own
// vectors, then across warps through shared memory, then by warp shuffle, then
// across the 8 lanes of the remaining vector.
#include "common.cuh"

template <bool MAXNUM>
static __device__ __forceinline__ float sm_max(float a, float b) {
    if (!MAXNUM && (a != a || b != b)) return __int_as_float(0x7fc00000);
    return fmaxf(a, b);
}

// OP 0: max, 1: add.  Returns the fold of the T*8*NV values in every thread of the row group.
template <int NV, int OP, bool MAXNUM, bool R16>
static __device__ __forceinline__ float row_fold(float (&x)[NV][8], int T, int t, int group,
                                                 float* xchg /* [groups][T][8] */, float* bcast /* [groups] */) {
    auto comb = [](float a, float b) -> float {
        float r = OP == 0 ? sm_max<MAXNUM>(a, b) : a + b;
        return (R16 && OP == 1) ? ktb_round16(r) : r;
    };
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = x[0][k];
    if (NV > 1) {
        float w[NV][8];
#pragma unroll
        for (int j = 0; j < NV; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) w[j][k] = x[j][k];
#pragma unroll
        for (int m = NV / 2; m >= 1; m >>= 1)
#pragma unroll
            for (int j = 0; j < m; ++j)
#pragma unroll
                for (int k = 0; k < 8; ++k) w[j][k] = comb(w[j][k], w[j + m][k]);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = w[0][k];
    }
    float* mine = xchg + ((size_t)group * T + t) * 8;
    for (int d = T / 2; d >= 32; d >>= 1) {
#pragma unroll
        for (int k = 0; k < 8; ++k) mine[k] = v[k];
        __syncthreads();
        if (t < d) {
            const float* other = mine + (size_t)d * 8;
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = comb(v[k], other[k]);
        }
        __syncthreads();
    }
    const int w = T < 32 ? T : 32;
    for (int d = w / 2; d >= 1; d >>= 1) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float o = __shfl_down_sync(0xffffffffu, v[k], d, w);
            v[k] = comb(v[k], o);
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = comb(v[k], v[k + 4]);
    v[0] = comb(v[0], v[2]);
    v[1] = comb(v[1], v[3]);
    v[0] = comb(v[0], v[1]);
    if (t == 0) bcast[group] = v[0];
    __syncthreads();
    float r = bcast[group];
    __syncthreads();
    return r;
}

template <int NV, bool MAXNUM, bool R16>
__global__ void __launch_bounds__(256) ktb_row_softmax_kernel(const ktb_softmax_args a, int T, int64_t total_rows) {
    extern __shared__ float smem[];
    const int groups = 256 / T;
    float* xchg = smem;
    float* bcast = smem + 256 * 8;
    const int group = threadIdx.x / T;
    const int t = threadIdx.x - group * T;
    const int64_t n_iter = (total_rows + groups - 1) / groups;

    for (int64_t it = blockIdx.x; it < n_iter; it += gridDim.x) {
        const int64_t row = it * groups + group;
        const bool live = row < total_rows;
        const int64_t item = live ? row / a.rows_per_item : 0;
        const int64_t r = live ? row - item * a.rows_per_item : 0;
        const int64_t in_off = a.dev_item_offsets[item * 2] + r * a.in_row_stride;
        const int64_t out_off = a.dev_item_offsets[item * 2 + 1] + r * a.out_row_stride;

        float x[NV][8];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int64_t e = in_off + ((int64_t)j * T + t) * 8;
            if (!live) {
#pragma unroll
                for (int k = 0; k < 8; ++k) x[j][k] = 0.f;
            } else if (a.in_dtype == KTB_F16) {
                uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(a.arena) + e);
                const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 f = __half22float2(h[i]);
                    x[j][2 * i] = f.x;
                    x[j][2 * i + 1] = f.y;
                }
            } else {
                const float* p = reinterpret_cast<const float*>(a.arena) + e;
                float4 lo = *reinterpret_cast<const float4*>(p);
                float4 hi = *reinterpret_cast<const float4*>(p + 4);
                x[j][0] = lo.x; x[j][1] = lo.y; x[j][2] = lo.z; x[j][3] = lo.w;
                x[j][4] = hi.x; x[j][5] = hi.y; x[j][6] = hi.z; x[j][7] = hi.w;
            }
        }

        float mx = row_fold<NV, 0, MAXNUM, R16>(x, T, t, group, xchg, bcast);
        mx = sm_max<MAXNUM>(mx, a.max_init);
#pragma unroll
        for (int j = 0; j < NV; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float d = x[j][k] - mx;
                if (R16) d = ktb_round16(d);
                float e = expf(d);
                x[j][k] = R16 ? ktb_round16(e) : e;
            }
        float sum = row_fold<NV, 1, MAXNUM, R16>(x, T, t, group, xchg, bcast);
        sum = sum + a.sum_init;
        if (R16) sum = ktb_round16(sum);

        if (live) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int64_t e = out_off + ((int64_t)j * T + t) * 8;
                float y[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) y[k] = x[j][k] / sum;
                if (a.out_dtype == KTB_F16) {
                    uint4 raw;
                    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
                    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
                    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.arena) + e) = raw;
                } else {
                    float* p = reinterpret_cast<float*>(a.arena) + e;
                    *reinterpret_cast<float4*>(p) = make_float4(y[0], y[1], y[2], y[3]);
                    *reinterpret_cast<float4*>(p + 4) = make_float4(y[4], y[5], y[6], y[7]);
                }
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
    const size_t smem = (256 * 8 + 256) * sizeof(float);
    const bool mn = a.max_is_maxnum != 0, r16 = a.f16_arith != 0;
#define KTB_SM_LAUNCH(MN, R)                                                                       \
    ktb_row_softmax_kernel<NV, MN, R><<<(unsigned)blocks, 256, smem, ctx->stream>>>(a, T, total_rows)
    if (mn && r16) KTB_SM_LAUNCH(true, true);
    else if (mn) KTB_SM_LAUNCH(true, false);
    else if (r16) KTB_SM_LAUNCH(false, true);
    else KTB_SM_LAUNCH(false, false);
#undef KTB_SM_LAUNCH
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
    const int T = vecs < 256 ? vecs : 256;
    const int NV = vecs / T;
    const int64_t total_rows = a.n_items * (int64_t)a.rows_per_item;
    switch (NV) {
        case 1: launch_softmax<1>(ctx, a, T, total_rows); break;
        case 2: launch_softmax<2>(ctx, a, T, total_rows); break;
        case 4: launch_softmax<4>(ctx, a, T, total_rows); break;
        case 8: launch_softmax<8>(ctx, a, T, total_rows); break;
        default: return ktb_fail(ctx, KTB_E_UNSUPPORTED, "row_softmax", "unsupported row width");
    }
    KTB_CHECK_LAUNCH(ctx, "ktb_row_softmax_kernel");
    return KTB_OK;
}
