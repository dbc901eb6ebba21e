// Row gather / ordered read-modify-write row scatter.
//
// A statement processes E = n_tiles * tile_rows "entries"; entry e = (tile t, row
// pos) moves one row of `cols` elements per operand.  A row's address is
//     base[t] + IDX[idx_off[t] + pos * idx_stride] * idx_mult + pos * pos_stride
// for an indirect operand (IDX read from an index tensor in the arena) or
//     base[t] + pos * pos_stride
// for a direct one.  Replaces MemoryOps.indirect_load / indirect_store
// (ktir_cpu/ops/memory_ops.py:867-964) and the per-point coordinate resolution
// behind them (:330-386, :488-576).
//
// Ordering.  The reference applies tiles one after another; inside a tile all
// loads happen before the store and duplicate destination rows keep the LAST
// writer (ktir_cpu/memory.py:281-291).  The scatter kernels reproduce exactly
// that without atomics:
//   1. ktb_scatter_prepare: per tile, resolve destination row ids and drop every
//      entry that a later entry of the same tile overwrites.
//   2. ktb_scatter_apply: destination rows are partitioned over CTAs (owner
//      computes).  Each CTA scans the row-id list in order, keeps the entries it
//      owns (ordered compaction), ranks entries of the same row by tile order,
//      and applies rank 0, 1, 2, ... in rounds: inside a round all rows are
//      distinct, so warps run in parallel; rounds are separated by a barrier.
// HBM-bound: per entry one index, one row per input, one row written.
#include "vm.cuh"

#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)
#define SC_LCAP 4096            // entries buffered per CTA before a batch is applied
#define SC_MAX_OWN_ROWS 4096    // destination rows owned by one CTA (smem counters)

static __device__ __forceinline__ int64_t sc_read_index(const void* arena, int idx_dtype, int64_t off) {
    return idx_dtype == KTB_I64 ? reinterpret_cast<const int64_t*>(arena)[off]
                                : (int64_t) reinterpret_cast<const int32_t*>(arena)[off];
}

// Element offset of the row entry (t, pos) addresses through `op`; -1 if the index is negative.
static __device__ __forceinline__ int64_t sc_row_addr(const void* arena, const ktb_row_operand& op, int64_t t,
                                                      int pos, ktb_status* st) {
    int64_t a = op.dev_base[t] + (int64_t)pos * op.pos_stride;
    if (op.indirect) {
        const int64_t iv = sc_read_index(arena, op.idx_dtype, op.dev_idx_off[t] + (int64_t)pos * op.idx_stride);
        if (iv < 0) {
            if (atomicExch(&st->negative_index, 1) == 0) st->bad_index_value = (int32_t)iv;
            return -1;
        }
        a += iv * op.idx_mult;
    }
    return a;
}

template <int V>
static __device__ __forceinline__ void sc_load_row(const void* arena, const ktb_row_operand& op, int64_t addr, int col,
                                                   int cols, float (&x)[V]) {
    const bool inside = addr >= op.lo && addr + cols <= op.hi;
    if (inside && V == 4 && col + 4 <= cols) {
        if (op.dtype == KTB_F16) {
            uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(arena) + addr + col);
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
            float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
            x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
        } else {
            float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(arena) + addr + col);
            x[0] = f.x; x[1] = f.y; x[2] = f.z; x[3] = f.w;
        }
        return;
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int64_t e = addr + col + v;
        float val = 0.f;
        if (col + v < cols && e >= op.lo && e < op.hi)
            val = op.dtype == KTB_F16 ? __half2float(reinterpret_cast<const __half*>(arena)[e])
                                      : reinterpret_cast<const float*>(arena)[e];
        x[v] = val;
    }
}

template <int V>
static __device__ __forceinline__ void sc_store_row(void* arena, const ktb_row_operand& op, int64_t addr, int col,
                                                    int cols, const float (&x)[V]) {
    const bool inside = addr >= op.lo && addr + cols <= op.hi;
    if (inside && V == 4 && col + 4 <= cols) {
        if (op.dtype == KTB_F16) {
            uint2 raw;
            __half2* h = reinterpret_cast<__half2*>(&raw);
            h[0] = __floats2half2_rn(x[0], x[1]);
            h[1] = __floats2half2_rn(x[2], x[3]);
            *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(arena) + addr + col) = raw;
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(arena) + addr + col) = make_float4(x[0], x[1], x[2], x[3]);
        }
        return;
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int64_t e = addr + col + v;
        if (col + v < cols && e >= op.lo && e < op.hi) {
            if (op.dtype == KTB_F16) reinterpret_cast<__half*>(arena)[e] = __float2half_rn(x[v]);
            else reinterpret_cast<float*>(arena)[e] = x[v];
        }
    }
}

// One warp moves one entry: gathers every input row, runs the program, writes the output row.
template <int V>
static __device__ __forceinline__ void sc_do_entry(const ktb_rows_args& a, int64_t e, int64_t dst_addr, int lane,
                                                   ktb_status* st) {
    const int64_t t = e / a.tile_rows;
    const int pos = (int)(e - t * a.tile_rows);
    int64_t in_addr[KTB_ROWS_MAX_IN];
    bool ok = dst_addr >= 0;
    for (int k = 0; k < a.n_in; ++k) {
        in_addr[k] = a.in[k].alias_dst ? dst_addr : sc_row_addr(a.arena, a.in[k], t, pos, st);
        ok = ok && in_addr[k] >= 0;
    }
    if (!ok) return;
    for (int col = lane * V; col < a.cols; col += 32 * V) {
        float regs[KTB_VM_REGS][V];
        for (int k = 0; k < a.n_in; ++k) {
            float x[V];
            sc_load_row<V>(a.arena, a.in[k], in_addr[k], col, a.cols, x);
#pragma unroll
            for (int v = 0; v < V; ++v) regs[k][v] = x[v];
        }
        float out[V];
        ktb_vm_run<V>(a.program, regs, out);
        sc_store_row<V>(a.arena, a.out, dst_addr, col, a.cols, out);
    }
}

// ---- direct destination: every entry is independent ------------------------------------------
template <int V>
__global__ void __launch_bounds__(256) ktb_rows_program_kernel(const ktb_rows_args a, ktb_status* st) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t E = a.n_tiles * a.tile_rows;
    for (int64_t e = warp; e < E; e += n_warps) {
        const int64_t t = e / a.tile_rows;
        const int pos = (int)(e - t * a.tile_rows);
        sc_do_entry<V>(a, e, sc_row_addr(a.arena, a.out, t, pos, st), lane, st);
    }
}

// ---- indirect destination, step 1: row ids + last-writer-wins inside each tile -----------------
__global__ void __launch_bounds__(128) ktb_scatter_prepare_kernel(const ktb_rows_args a, ktb_status* st) {
    extern __shared__ int64_t s_addr[];      // [tile_rows]
    for (int64_t t = blockIdx.x; t < a.n_tiles; t += gridDim.x) {
        for (int pos = threadIdx.x; pos < a.tile_rows; pos += blockDim.x) {
            int64_t addr = sc_row_addr(a.arena, a.out, t, pos, st);
            if (addr >= 0) {
                const int64_t rel = addr - a.dst_row0;
                // rows that do not start on a row boundary of the destination cannot be ordered by id
                addr = (rel >= 0 && rel % a.out.idx_mult == 0 && rel / a.out.idx_mult < a.dst_rows)
                           ? rel / a.out.idx_mult : -1;
            }
            s_addr[pos] = addr;
        }
        __syncthreads();
        for (int pos = threadIdx.x; pos < a.tile_rows; pos += blockDim.x) {
            const int64_t mine = s_addr[pos];
            bool win = mine >= 0;
            for (int q = pos + 1; win && q < a.tile_rows; ++q) win = s_addr[q] != mine;
            a.dev_rowid_scratch[t * a.tile_rows + pos] = win ? (int32_t)mine : -1;
        }
        __syncthreads();
    }
}

// ---- step 2: owner-computes ordered apply ------------------------------------------------------
template <int V>
__global__ void __launch_bounds__(SC_THREADS) ktb_scatter_apply_kernel(const ktb_rows_args a, int rows_per_owner,
                                                                        ktb_status* st) {
    __shared__ int32_t list_e[SC_LCAP];
    __shared__ uint16_t list_r[SC_LCAP];
    __shared__ uint16_t list_k[SC_LCAP];     // rank among entries of the same row in this batch
    __shared__ uint16_t cnt[SC_MAX_OWN_ROWS];
    __shared__ int32_t warp_tot[SC_WARPS];
    __shared__ int32_t s_len, s_maxrank;

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int64_t E = a.n_tiles * a.tile_rows;
    const int32_t own_lo = blockIdx.x * rows_per_owner;
    const int32_t own_hi = own_lo + rows_per_owner;
    for (int i = tid; i < rows_per_owner; i += SC_THREADS) cnt[i] = 0;
    if (tid == 0) { s_len = 0; s_maxrank = 0; }
    __syncthreads();

    auto apply_batch = [&]() {
        const int len = s_len;
        // ranks in list order (warp 0): entries of one row get 0, 1, 2, ... in tile order
        if (wid == 0) {
            int mr = 0;
            for (int i0 = 0; i0 < len; i0 += 32) {
                const int i = i0 + lane;
                const bool act = i < len;
                const unsigned amask = __ballot_sync(0xffffffffu, act);
                if (act) {
                    const int r = list_r[i];
                    const unsigned m = __match_any_sync(amask, r);
                    const int k = cnt[r] + __popc(m & ((1u << lane) - 1));
                    list_k[i] = (uint16_t)k;
                    mr = max(mr, k);
                    __syncwarp(amask);
                    if ((m >> lane) == 1u) cnt[r] = (uint16_t)(cnt[r] + __popc(m));
                }
                __syncwarp();
            }
            for (int d = 16; d; d >>= 1) mr = max(mr, __shfl_xor_sync(0xffffffffu, mr, d));
            if (lane == 0) s_maxrank = mr;
        }
        __syncthreads();
        const int maxrank = s_maxrank;
        for (int round = 0; round <= maxrank; ++round) {
            for (int i = wid; i < len; i += SC_WARPS) {
                if (list_k[i] != round) continue;
                const int64_t row = (int64_t)own_lo + list_r[i];
                sc_do_entry<V>(a, list_e[i], a.dst_row0 + row * a.out.idx_mult, lane, st);
            }
            __syncthreads();
        }
        for (int i = tid; i < len; i += SC_THREADS) cnt[list_r[i]] = 0;
        if (tid == 0) s_len = 0;
        __syncthreads();
    };

    for (int64_t base = 0; base < E; base += SC_THREADS * 4) {
        // each thread looks at 4 consecutive entries; matches are appended in entry order
        int32_t rid[4];
        const int64_t e0 = base + (int64_t)tid * 4;
        if (e0 + 4 <= E && (E % 4 == 0)) {
            int4 v = *reinterpret_cast<const int4*>(a.dev_rowid_scratch + e0);
            rid[0] = v.x; rid[1] = v.y; rid[2] = v.z; rid[3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) rid[j] = e0 + j < E ? a.dev_rowid_scratch[e0 + j] : -1;
        }
        int m = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) m += (rid[j] >= own_lo && rid[j] < own_hi) ? 1 : 0;
        int incl = m;
        for (int d = 1; d < 32; d <<= 1) {
            int o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < SC_WARPS; ++w) {
            const int x = warp_tot[w];
            if (w < wid) before += x;
            total += x;
        }
        if (s_len + total > SC_LCAP) apply_batch();      // uniform: s_len and total are block-wide values
        int at = s_len + before + incl - m;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (rid[j] >= own_lo && rid[j] < own_hi) {
                list_e[at] = (int32_t)(e0 + j);
                list_r[at] = (uint16_t)(rid[j] - own_lo);
                ++at;
            }
        __syncthreads();
        if (tid == 0) s_len += total;
        __syncthreads();
    }
    if (s_len > 0) apply_batch();
}

static int check_rows_args(ktb_ctx* ctx, const ktb_rows_args& a, const char* who) {
    const ktb_vm_program& p = a.program;
    if (a.n_in < 1 || a.n_in > KTB_ROWS_MAX_IN || p.n_in != a.n_in || p.n_ops < 0 || p.n_ops > KTB_VM_MAX_OPS ||
        p.result_reg < 0 || p.result_reg >= KTB_VM_REGS)
        return ktb_fail(ctx, KTB_E_ARG, who, "bad program header");
    for (int i = 0; i < p.n_ops; ++i) {
        const ktb_vm_op& o = p.ops[i];
        if ((o.opcode & 0xff) >= KTB_VM_NOPS || o.dst < 0 || o.dst >= KTB_VM_REGS || o.a < 0 || o.a >= KTB_VM_REGS ||
            o.b < 0 || o.b >= KTB_VM_REGS || o.c < 0 || o.c >= KTB_VM_REGS)
            return ktb_fail(ctx, KTB_E_ARG, who, "bad program op");
    }
    for (int k = 0; k <= a.n_in; ++k) {
        const ktb_row_operand& op = k < a.n_in ? a.in[k] : a.out;
        if (op.dtype != KTB_F16 && op.dtype != KTB_F32) return ktb_fail(ctx, KTB_E_UNSUPPORTED, who, "row dtype must be f16 or f32");
        if (op.indirect && op.idx_dtype != KTB_I32 && op.idx_dtype != KTB_I64)
            return ktb_fail(ctx, KTB_E_UNSUPPORTED, who, "index dtype must be i32 or i64");
    }
    if (a.tile_rows <= 0 || a.cols <= 0 || a.n_tiles < 0) return ktb_fail(ctx, KTB_E_ARG, who, "bad tile geometry");
    if (a.n_tiles * (int64_t)a.tile_rows >= (1ll << 31)) return ktb_fail(ctx, KTB_E_UNSUPPORTED, who, "too many entries");
    return KTB_OK;
}

extern "C" int ktb_launch_rows_program(ktb_ctx* ctx, const ktb_rows_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    const ktb_rows_args& a = *args;
    int rc = check_rows_args(ctx, a, "rows_program");
    if (rc) return rc;
    if (a.n_tiles == 0) return KTB_OK;
    const int64_t E = a.n_tiles * a.tile_rows;
    int64_t blocks = (E + 7) / 8;
    const int64_t cap = (int64_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (a.vector_ok) ktb_rows_program_kernel<4><<<(unsigned)blocks, 256, 0, ctx->stream>>>(a, ctx->dev_status);
    else ktb_rows_program_kernel<1><<<(unsigned)blocks, 256, 0, ctx->stream>>>(a, ctx->dev_status);
    KTB_CHECK_LAUNCH(ctx, "ktb_rows_program_kernel");
    return KTB_OK;
}

// Shared by the two scatter entry points: `scratch` is the row-id list the launches use.
int ktb_scatter_rows_impl(ktb_ctx* ctx, const ktb_rows_args& a_in, int32_t* scratch) {
    ktb_rows_args a = a_in;
    a.dev_rowid_scratch = scratch;
    int rc = check_rows_args(ctx, a, "scatter_rows");
    if (rc) return rc;
    if (!a.out.indirect || !scratch) return ktb_fail(ctx, KTB_E_ARG, "scatter_rows", "destination must be indirect and scratch non-null");
    if (a.out.idx_mult <= 0 || a.dst_rows <= 0) return ktb_fail(ctx, KTB_E_ARG, "scatter_rows", "bad destination row geometry");
    if (a.dst_rows >= (1ll << 31)) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "scatter_rows", "too many destination rows");
    if (a.n_tiles == 0) return KTB_OK;
    int64_t prep_blocks = a.n_tiles < (int64_t)ctx->sm_count * 16 ? a.n_tiles : (int64_t)ctx->sm_count * 16;
    const size_t smem = (size_t)a.tile_rows * sizeof(int64_t);
    if (smem > 48 * 1024) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "scatter_rows", "tile has too many rows");
    ktb_scatter_prepare_kernel<<<(unsigned)prep_blocks, 128, smem, ctx->stream>>>(a, ctx->dev_status);
    KTB_CHECK_LAUNCH(ctx, "ktb_scatter_prepare_kernel");
    int64_t owners = (int64_t)ctx->sm_count * 2;
    int64_t rpo = (a.dst_rows + owners - 1) / owners;
    if (rpo > SC_MAX_OWN_ROWS) rpo = SC_MAX_OWN_ROWS;
    if (rpo < 1) rpo = 1;
    owners = (a.dst_rows + rpo - 1) / rpo;
    if (a.vector_ok) ktb_scatter_apply_kernel<4><<<(unsigned)owners, SC_THREADS, 0, ctx->stream>>>(a, (int)rpo, ctx->dev_status);
    else ktb_scatter_apply_kernel<1><<<(unsigned)owners, SC_THREADS, 0, ctx->stream>>>(a, (int)rpo, ctx->dev_status);
    KTB_CHECK_LAUNCH(ctx, "ktb_scatter_apply_kernel");
    return KTB_OK;
}

extern "C" int ktb_launch_scatter_rows(ktb_ctx* ctx, const ktb_rows_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    return ktb_scatter_rows_impl(ctx, *args, args->dev_rowid_scratch);
}
