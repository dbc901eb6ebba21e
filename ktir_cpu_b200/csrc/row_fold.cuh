// Row reductions in the pairing order of the reference's linalg.reduce, shared by the row kernels.
//
// A row of cols = T * 8 * NV elements is held by a group of T threads (thread t owns the 16-byte vectors
// j * T + t, j < NV).  row_fold combines x[i] (op) x[i + h] for h = cols/2 ... 1 — the halving order of
// _tree_fold (ktir_cpu/dialects/linalg_ops.py:86-133) when cols is a power of two: first across a thread's
// own vectors, then across the warps of the group (one shared-memory exchange, combined in the same
// pairing), then by warp shuffle, then across the 8 elements of the remaining vector.
#pragma once
#include "common.cuh"

template <bool MAXNUM>
static __device__ __forceinline__ float sm_max(float a, float b) {
    if (!MAXNUM && (a != a || b != b)) return __int_as_float(0x7fc00000);
    return fmaxf(a, b);
}

template <int OP, bool MAXNUM, bool R16>
static __device__ __forceinline__ float sm_comb(float a, float b) {
    if (OP == 0) return sm_max<MAXNUM>(a, b);
    const float r = a + b;
    return R16 ? ktb_round16(r) : r;
}

// Named barrier of one row group (ids 1..4 as literals so only those are reserved).
static __device__ __forceinline__ void group_barrier(int id, int threads) {
    switch (id) {
        case 1: asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); break;
        case 2: asm volatile("bar.sync 2, %0;" ::"r"(threads) : "memory"); break;
        case 3: asm volatile("bar.sync 3, %0;" ::"r"(threads) : "memory"); break;
        default: asm volatile("bar.sync 4, %0;" ::"r"(threads) : "memory"); break;
    }
}

// Pairing of the cross-warp levels: value(base, stride, n) = value(base, 2*stride, n/2)
// (op) value(base + stride, 2*stride, n/2), leaves are the per-warp partials.
template <int OP, bool MAXNUM, bool R16>
static __device__ __forceinline__ float warp_tree(const float* p, int n_warps, int lane_slot_stride) {
    // p[w * lane_slot_stride] is the partial of warp w for this (lane, slot)
    float o[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) o[w] = w < n_warps ? p[w * lane_slot_stride] : 0.f;
    if (n_warps == 8) {
        const float a = sm_comb<OP, MAXNUM, R16>(sm_comb<OP, MAXNUM, R16>(o[0], o[4]), sm_comb<OP, MAXNUM, R16>(o[2], o[6]));
        const float b = sm_comb<OP, MAXNUM, R16>(sm_comb<OP, MAXNUM, R16>(o[1], o[5]), sm_comb<OP, MAXNUM, R16>(o[3], o[7]));
        return sm_comb<OP, MAXNUM, R16>(a, b);
    }
    if (n_warps == 4)
        return sm_comb<OP, MAXNUM, R16>(sm_comb<OP, MAXNUM, R16>(o[0], o[2]), sm_comb<OP, MAXNUM, R16>(o[1], o[3]));
    return sm_comb<OP, MAXNUM, R16>(o[0], o[1]);
}

// Fold of the T*8*NV values of a row; every thread of the group gets the result.
template <int NV, int OP, bool MAXNUM, bool R16>
static __device__ __forceinline__ float row_fold(const float (&x)[NV][8], int T, int t, int group,
                                                 float* xchg /* [256][8] */, float* bcast /* [256/32] */) {
    float v[8];
    if (NV == 1) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = x[0][k];
    } else {
        constexpr int H = NV / 2 > 0 ? NV / 2 : 1;
        float w[H][8];
#pragma unroll
        for (int j = 0; j < H; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) w[j][k] = sm_comb<OP, MAXNUM, R16>(x[j][k], x[j + H][k]);
#pragma unroll
        for (int m = H / 2; m >= 1; m >>= 1)
#pragma unroll
            for (int j = 0; j < m; ++j)
#pragma unroll
                for (int k = 0; k < 8; ++k) w[j][k] = sm_comb<OP, MAXNUM, R16>(w[j][k], w[j + m][k]);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = w[0][k];
    }
    if (T > 32) {
        const int n_warps = T >> 5;
        float* mine = xchg + (size_t)threadIdx.x * 8;
#pragma unroll
        for (int k = 0; k < 8; ++k) mine[k] = v[k];
        group_barrier(1 + group, T);
        if (t < 32) {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = warp_tree<OP, MAXNUM, R16>(mine + k, n_warps, 32 * 8);
        }
    }
    const int w = T < 32 ? T : 32;
    for (int d = w >> 1; d >= 1; d >>= 1) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float o = __shfl_down_sync(0xffffffffu, v[k], d, w);
            v[k] = sm_comb<OP, MAXNUM, R16>(v[k], o);
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = sm_comb<OP, MAXNUM, R16>(v[k], v[k + 4]);
    v[0] = sm_comb<OP, MAXNUM, R16>(v[0], v[2]);
    v[1] = sm_comb<OP, MAXNUM, R16>(v[1], v[3]);
    v[0] = sm_comb<OP, MAXNUM, R16>(v[0], v[1]);
    if (T > 32) {
        if (t == 0) bcast[group] = v[0];
        group_barrier(1 + group, T);
        return bcast[group];
    }
    return __shfl_sync(0xffffffffu, v[0], 0, w);
}


// The same fold of a sum whose every add rounds to f16, on packed halves: an f16 add of two f16 values is
// the f32 add rounded to f16 (24 >= 2 * 11 + 2 significand bits: the double rounding cannot show), so the
// results are those of row_fold<NV, 1, false, true> at an eighth of the conversions.  x[j][q] holds elements
// 2q, 2q + 1 of vector j.
static __device__ __forceinline__ __half2 warp_tree_h(const __half2* p, int n_warps, int stride) {
    __half2 o[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) o[w] = w < n_warps ? p[w * stride] : __half2();
    if (n_warps == 8)
        return __hadd2_rn(__hadd2_rn(__hadd2_rn(o[0], o[4]), __hadd2_rn(o[2], o[6])),
                          __hadd2_rn(__hadd2_rn(o[1], o[5]), __hadd2_rn(o[3], o[7])));
    if (n_warps == 4) return __hadd2_rn(__hadd2_rn(o[0], o[2]), __hadd2_rn(o[1], o[3]));
    return __hadd2_rn(o[0], o[1]);
}

template <int NV>
static __device__ __forceinline__ float row_fold_h(const __half2 (&x)[NV][4], int T, int t, int group,
                                                   float* xchg /* [256][8] */, float* bcast /* [256/32] */) {
    __half2 v[4];
    if (NV == 1) {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = x[0][k];
    } else {
        constexpr int H = NV / 2 > 0 ? NV / 2 : 1;
        __half2 w[H][4];
#pragma unroll
        for (int j = 0; j < H; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) w[j][k] = __hadd2_rn(x[j][k], x[j + H][k]);
#pragma unroll
        for (int m = H / 2; m >= 1; m >>= 1)
#pragma unroll
            for (int j = 0; j < m; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k) w[j][k] = __hadd2_rn(w[j][k], w[j + m][k]);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = w[0][k];
    }
    if (T > 32) {
        const int n_warps = T >> 5;
        __half2* mine = reinterpret_cast<__half2*>(xchg) + (size_t)threadIdx.x * 4;
#pragma unroll
        for (int k = 0; k < 4; ++k) mine[k] = v[k];
        group_barrier(1 + group, T);
        if (t < 32) {
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = warp_tree_h(mine + k, n_warps, 32 * 4);
        }
    }
    const int w = T < 32 ? T : 32;
    for (int d = w >> 1; d >= 1; d >>= 1) {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __hadd2_rn(v[k], __shfl_down_sync(0xffffffffu, v[k], d, w));
    }
    v[0] = __hadd2_rn(v[0], v[2]);                       // elements k and k + 4
    v[1] = __hadd2_rn(v[1], v[3]);
    v[0] = __hadd2_rn(v[0], v[1]);                       // 0 + 2, 1 + 3
    const float r = __half2float(__hadd_rn(__low2half(v[0]), __high2half(v[0])));
    if (T > 32) {
        if (t == 0) bcast[group] = r;
        group_barrier(1 + group, T);
        return bcast[group];
    }
    return __shfl_sync(0xffffffffu, r, 0, w);
}
