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

// A warp handles up to 32 entries at a time.  The scalar work of an entry — decoding (tile, row),
// reading its index, forming the row addresses — is done by ONE lane per entry, all lanes in
// parallel (sc_resolve); the rows themselves are then moved by the whole warp, G entries in
// flight at once (sc_move_group), with the addresses broadcast by shuffle.  This keeps the
// per-entry instruction count low and overlaps the dependent index -> row chains of many entries.
// PROG selects how the row program is evaluated: the general register program, a plain copy of
// input 0, or out = round16(in[acc] + round16(in[1 - acc] * c)) with acc = 0 / 1 (the f16
// scaled-accumulate of a read-modify-write scatter), the latter two without any decoding.
enum { SC_PROG_VM = 0, SC_PROG_COPY = 1, SC_PROG_AXPY0 = 2, SC_PROG_AXPY1 = 3 };

static __device__ __forceinline__ int64_t sc_shfl64(int64_t v, int src) {
    const int lo = __shfl_sync(0xffffffffu, (int)(v & 0xffffffffll), src);
    const int hi = __shfl_sync(0xffffffffu, (int)(v >> 32), src);
    return ((int64_t)hi << 32) | (uint32_t)lo;
}

// Row addresses of the non-aliasing inputs of entry e (this lane's entry); -1 marks a bad index.
static __device__ __forceinline__ void sc_resolve(const ktb_rows_args& a, uint32_t e, ktb_status* st,
                                                  int64_t (&addr)[KTB_ROWS_MAX_IN]) {
    const uint32_t t = e / (uint32_t)a.tile_rows;
    const int pos = (int)(e - t * (uint32_t)a.tile_rows);
#pragma unroll
    for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) {
        addr[k] = 0;
        if (k < a.n_in && !a.in[k].alias_dst) addr[k] = sc_row_addr(a.arena, a.in[k], t, pos, st);
    }
}

template <int V, int G, int PROG>
static __device__ __forceinline__ void sc_move_group(const ktb_rows_args& a, const int64_t (&in_addr)[G][KTB_ROWS_MAX_IN],
                                                     const int64_t (&dst)[G], const bool (&ok)[G], int lane,
                                                     float4* vm, int vm_stride) {
    for (int col = lane * V; col < a.cols; col += 32 * V) {
        float x[G][KTB_ROWS_MAX_IN][V];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) {
#pragma unroll
                for (int v = 0; v < V; ++v) x[g][k][v] = 0.f;
                if (ok[g] && k < a.n_in) sc_load_row<V>(a.arena, a.in[k], in_addr[g][k], col, a.cols, x[g][k]);
            }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (!ok[g]) continue;
            float out[V];
            if (PROG == SC_PROG_COPY) {
#pragma unroll
                for (int v = 0; v < V; ++v) out[v] = x[g][0][v];
            } else if (PROG == SC_PROG_AXPY0 || PROG == SC_PROG_AXPY1) {
                constexpr int ACC = PROG == SC_PROG_AXPY0 ? 0 : 1;
                const float c = a.program.ops[0].imm;
#pragma unroll
                for (int v = 0; v < V; ++v) out[v] = ktb_round16(x[g][ACC][v] + ktb_round16(x[g][1 - ACC][v] * c));
            } else {
#pragma unroll
                for (int k = 0; k < KTB_ROWS_MAX_IN; ++k)
                    vm[k * vm_stride] = make_float4(x[g][k][0], V > 1 ? x[g][k][1 % V] : 0.f,
                                                    V > 1 ? x[g][k][2 % V] : 0.f, V > 1 ? x[g][k][3 % V] : 0.f);
                const float4 res = ktb_vm_run_smem4(a.program, vm, vm_stride);
                const float rv[4] = {res.x, res.y, res.z, res.w};
#pragma unroll
                for (int v = 0; v < V; ++v) out[v] = rv[v];
            }
            sc_store_row<V>(a.arena, a.out, dst[g], col, a.cols, out);
        }
    }
}

// ---- direct destination: every entry is independent ------------------------------------------
template <int V, int PROG>
__global__ void __launch_bounds__(256) ktb_rows_program_kernel(const __grid_constant__ ktb_rows_args a, ktb_status* st) {
    constexpr int G = 4;
    extern __shared__ float4 rp_vm[];                 // [KTB_VM_REGS][blockDim.x] register file
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t E = a.n_tiles * a.tile_rows;
    for (int64_t e0 = warp * 32; e0 < E; e0 += n_warps * 32) {
        const bool have = e0 + lane < E;
        const uint32_t e = (uint32_t)(have ? e0 + lane : 0);
        int64_t my_in[KTB_ROWS_MAX_IN];
        int64_t my_dst = -1;
        sc_resolve(a, e, st, my_in);
        if (have) {
            const uint32_t t = e / (uint32_t)a.tile_rows;
            my_dst = sc_row_addr(a.arena, a.out, t, (int)(e - t * (uint32_t)a.tile_rows), st);
        }
        const int cnt = (int)((E - e0) < 32 ? (E - e0) : 32);
        for (int b0 = 0; b0 < cnt; b0 += G) {
            int64_t in_addr[G][KTB_ROWS_MAX_IN], dst[G];
            bool ok[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const int src = (b0 + g) & 31;
                dst[g] = sc_shfl64(my_dst, src);
                ok[g] = b0 + g < cnt && dst[g] >= 0;
#pragma unroll
                for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) {
                    in_addr[g][k] = sc_shfl64(my_in[k], src);
                    if (k < a.n_in) ok[g] = ok[g] && in_addr[g][k] >= 0;
                }
            }
            sc_move_group<V, G, PROG>(a, in_addr, dst, ok, lane, rp_vm + threadIdx.x, blockDim.x);
        }
    }
}

// ---- indirect destination, step 1: row ids + last-writer-wins inside each tile -----------------
// Scratch layout: int32 row id per entry (-1 = dropped), then one owner byte per entry (255 = none).
#define SC_NO_OWNER 255

__global__ void __launch_bounds__(128) ktb_scatter_prepare_kernel(const __grid_constant__ ktb_rows_args a, int rows_per_owner,
                                                                  ktb_status* st) {
    extern __shared__ int64_t s_addr[];      // [tile_rows]
    const int64_t E = a.n_tiles * a.tile_rows;
    uint8_t* owner = reinterpret_cast<uint8_t*>(a.dev_rowid_scratch + E);
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
            const int64_t e = t * a.tile_rows + pos;
            a.dev_rowid_scratch[e] = win ? (int32_t)mine : -1;
            owner[e] = win ? (uint8_t)(mine / rows_per_owner) : (uint8_t)SC_NO_OWNER;
        }
        __syncthreads();
    }
}

// ---- step 2: owner-computes ordered apply ------------------------------------------------------
// Destination rows are partitioned over CTAs; inside a CTA a row belongs to warp (row % 32).  A
// CTA scans the owner bytes of all entries in order and appends its own entries to a list
// (ordered compaction).  Each warp then walks the list in order and applies the entries of its
// rows: updates of one row are applied by one warp in tile order, different rows never interact,
// so no barrier and no atomic is needed while applying.
#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)
#define SC_STEP (SC_THREADS * 16)   // entries examined per scan step (16 owner bytes per thread)
#define SC_LCAP SC_STEP             // entries buffered per CTA before the batch is applied
#define SC_GROUP 4
#define SC_PRIV 512                // entries in a warp's private list

template <int V, int PROG>
__global__ void __launch_bounds__(SC_THREADS, 1) ktb_scatter_apply_kernel(const __grid_constant__ ktb_rows_args a, int rows_per_owner,
                                                                           ktb_status* st) {
    extern __shared__ uint8_t sc_smem[];
    int32_t* list_e = reinterpret_cast<int32_t*>(sc_smem);                  // [SC_LCAP] entry ids
    int32_t* list_r = list_e + SC_LCAP;                                     // [SC_LCAP] destination row ids
    int32_t* my_e = list_r + SC_LCAP + (threadIdx.x >> 5) * (2 * SC_PRIV);   // this warp's private list
    int32_t* my_r = my_e + SC_PRIV;
    float4* vm = reinterpret_cast<float4*>(list_r + SC_LCAP + SC_WARPS * 2 * SC_PRIV) + threadIdx.x;  // [KTB_VM_REGS][SC_THREADS]
    __shared__ int32_t warp_tot[SC_WARPS];
    __shared__ int32_t s_len;

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int64_t E = a.n_tiles * a.tile_rows;
    const uint8_t* owner = reinterpret_cast<const uint8_t*>(a.dev_rowid_scratch + E);
    const uint32_t me4 = (uint32_t)blockIdx.x * 0x01010101u;
    if (tid == 0) s_len = 0;
    __syncthreads();

    // One warp applies a dense run of its own entries: lane l resolves entry l, then the rows move
    // SC_GROUP at a time in list order (an update of a row waits for the previous one of that row).
    auto apply_private = [&](int cnt) {
        for (int j0 = 0; j0 < cnt; j0 += 32) {
            const bool have = j0 + lane < cnt;
            const int32_t e = have ? my_e[j0 + lane] : 0;
            const int32_t r = have ? my_r[j0 + lane] : -1;
            int64_t my_in[KTB_ROWS_MAX_IN];
            sc_resolve(a, (uint32_t)e, st, my_in);
            const int64_t my_dst = a.dst_row0 + (int64_t)(r < 0 ? 0 : r) * a.out.idx_mult;
            const int m = cnt - j0 < 32 ? cnt - j0 : 32;
            int next = 0;
            while (next < m) {
                int64_t in_addr[SC_GROUP][KTB_ROWS_MAX_IN], dst[SC_GROUP];
                int32_t rows[SC_GROUP];
                bool ok[SC_GROUP];
                int n = 0;
#pragma unroll
                for (int g = 0; g < SC_GROUP; ++g) {
                    rows[g] = -1;
                    dst[g] = -1;
                    ok[g] = false;
#pragma unroll
                    for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) in_addr[g][k] = 0;
                    if (next < m && n == g) {
                        const int src = next;
                        const int32_t rr = __shfl_sync(0xffffffffu, r, src);
                        bool clash = false;
#pragma unroll
                        for (int h = 0; h < SC_GROUP; ++h) clash = clash || (h < g && rows[h] == rr);
                        if (!clash) {
                            rows[g] = rr;
                            dst[g] = sc_shfl64(my_dst, src);
                            ok[g] = true;
#pragma unroll
                            for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) {
                                const int64_t v = sc_shfl64(my_in[k], src);
                                if (k < a.n_in) {
                                    in_addr[g][k] = a.in[k].alias_dst ? dst[g] : v;
                                    ok[g] = ok[g] && in_addr[g][k] >= 0;
                                }
                            }
                            ++next;
                            n = g + 1;
                        }
                    }
                }
                sc_move_group<V, SC_GROUP, PROG>(a, in_addr, dst, ok, lane, vm, SC_THREADS);
            }
        }
    };

    // Entries of the CTA list are dealt to warps by destination row (row % SC_WARPS); each warp
    // packs its entries, in list order, into a private list and applies them in dense runs.
    auto apply_batch = [&]() {
        const int len = s_len;
        int cnt = 0;
        for (int i0 = 0; i0 < len; i0 += 32) {
            const int i = i0 + lane;
            const int32_t r = i < len ? list_r[i] : -1;
            const int32_t e = i < len ? list_e[i] : 0;
            const bool mine = r >= 0 && (r & (SC_WARPS - 1)) == wid;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int at = cnt + __popc(mask & ((1u << lane) - 1));
                my_e[at] = e;
                my_r[at] = r;
            }
            cnt += __popc(mask);
            __syncwarp();
            if (cnt > SC_PRIV - 32) {
                apply_private(cnt);
                cnt = 0;
                __syncwarp();
            }
        }
        if (cnt) apply_private(cnt);
        __syncthreads();
        if (tid == 0) s_len = 0;
        __syncthreads();
    };

    const int64_t n_steps = (E + SC_STEP - 1) / SC_STEP;
    auto load_bytes = [&](int64_t step) -> uint4 {
        const int64_t e0 = step * SC_STEP + (int64_t)tid * 16;
        if (e0 + 16 <= E && ((reinterpret_cast<uintptr_t>(owner) & 15) == 0))
            return __ldg(reinterpret_cast<const uint4*>(owner + e0));
        uint32_t w[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        for (int j = 0; j < 16; ++j)
            if (e0 + j < E) w[j >> 2] = (w[j >> 2] & ~(0xffu << (8 * (j & 3)))) | ((uint32_t)owner[e0 + j] << (8 * (j & 3)));
        return make_uint4(w[0], w[1], w[2], w[3]);
    };
    uint4 cur = n_steps > 0 ? load_bytes(0) : make_uint4(~0u, ~0u, ~0u, ~0u);
    for (int64_t step = 0; step < n_steps; ++step) {
        const uint4 nxt = step + 1 < n_steps ? load_bytes(step + 1) : make_uint4(~0u, ~0u, ~0u, ~0u);
        const int64_t e0 = step * SC_STEP + (int64_t)tid * 16;
        const uint32_t w[4] = {cur.x, cur.y, cur.z, cur.w};
        uint32_t hit[4];
        int m = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            hit[j] = __vcmpeq4(w[j], me4);          // 0xff in every byte that names this CTA
            m += __popc(hit[j]) >> 3;
        }
        int incl = m;
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        int before = 0, total = 0;
        for (int wv = 0; wv < SC_WARPS; ++wv) {
            const int x = warp_tot[wv];
            if (wv < wid) before += x;
            total += x;
        }
        if (s_len + total > SC_LCAP) apply_batch();      // uniform: s_len and total are block-wide values
        int at = s_len + before + incl - m;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (hit[j >> 2] & (0xffu << (8 * (j & 3)))) {
                list_e[at] = (int32_t)(e0 + j);
                list_r[at] = a.dev_rowid_scratch[e0 + j];
                ++at;
            }
        __syncthreads();
        if (tid == 0) s_len += total;
        __syncthreads();
        cur = nxt;
    }
    if (s_len > 0) apply_batch();
}

// Recognise the two row programs that have a decoded fast path.
static int sc_classify(const ktb_rows_args& a) {
    const ktb_vm_program& p = a.program;
    if (p.n_ops == 0 && p.result_reg == 0) return SC_PROG_COPY;
    if (a.n_in == 2 && p.n_ops == 3 && (p.ops[0].opcode & 0xff) == KTB_VM_CONST &&
        p.ops[1].opcode == (KTB_VM_MUL | KTB_VM_ROUND16) && p.ops[2].opcode == (KTB_VM_ADD | KTB_VM_ROUND16) &&
        p.result_reg == p.ops[2].dst) {
        const int creg = p.ops[0].dst, mreg = p.ops[1].dst;
        int scaled = -1;
        if (p.ops[1].a == creg && p.ops[1].b < 2) scaled = p.ops[1].b;
        if (p.ops[1].b == creg && p.ops[1].a < 2) scaled = p.ops[1].a;
        int acc = -1;
        if (p.ops[2].a == mreg && p.ops[2].b < 2) acc = p.ops[2].b;
        if (p.ops[2].b == mreg && p.ops[2].a < 2) acc = p.ops[2].a;
        if (scaled >= 0 && acc >= 0 && scaled != acc) return acc == 0 ? SC_PROG_AXPY0 : SC_PROG_AXPY1;
    }
    return SC_PROG_VM;
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
    const size_t vsmem = (size_t)KTB_VM_REGS * 256 * sizeof(float4);
#define KTB_RP(V, P) ktb_rows_program_kernel<V, P><<<(unsigned)blocks, 256, vsmem, ctx->stream>>>(a, ctx->dev_status)
    switch (sc_classify(a) * 2 + (a.vector_ok ? 1 : 0)) {
        case SC_PROG_COPY * 2 + 1: KTB_RP(4, SC_PROG_COPY); break;
        case SC_PROG_COPY * 2: KTB_RP(1, SC_PROG_COPY); break;
        case SC_PROG_AXPY0 * 2 + 1: KTB_RP(4, SC_PROG_AXPY0); break;
        case SC_PROG_AXPY1 * 2 + 1: KTB_RP(4, SC_PROG_AXPY1); break;
        default:
            if (a.vector_ok) KTB_RP(4, SC_PROG_VM);
            else KTB_RP(1, SC_PROG_VM);
    }
#undef KTB_RP
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
    // destination rows are split evenly over one owner CTA per SM (at most 254 owners)
    int64_t n_own = ctx->sm_count < 254 ? ctx->sm_count : 254;
    int64_t rpo = (a.dst_rows + n_own - 1) / n_own;
    if (rpo < 1) rpo = 1;
    const int64_t owners = (a.dst_rows + rpo - 1) / rpo;
    int64_t prep_blocks = a.n_tiles < (int64_t)ctx->sm_count * 16 ? a.n_tiles : (int64_t)ctx->sm_count * 16;
    const size_t smem = (size_t)a.tile_rows * sizeof(int64_t);
    if (smem > 48 * 1024) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "scatter_rows", "tile has too many rows");
    ktb_scatter_prepare_kernel<<<(unsigned)prep_blocks, 128, smem, ctx->stream>>>(a, (int)rpo, ctx->dev_status);
    KTB_CHECK_LAUNCH(ctx, "ktb_scatter_prepare_kernel");
    const size_t asmem = (size_t)SC_LCAP * 8 + (size_t)SC_WARPS * SC_PRIV * 8 + (size_t)KTB_VM_REGS * SC_THREADS * sizeof(float4);
#define KTB_SA(V, P)                                                                                              \
    do {                                                                                                          \
        KTB_CUDA(ctx, cudaFuncSetAttribute(ktb_scatter_apply_kernel<V, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)asmem));                                                          \
        ktb_scatter_apply_kernel<V, P><<<(unsigned)owners, SC_THREADS, asmem, ctx->stream>>>(a, (int)rpo, ctx->dev_status); \
    } while (0)
    switch (sc_classify(a) * 2 + (a.vector_ok ? 1 : 0)) {
        case SC_PROG_COPY * 2 + 1: KTB_SA(4, SC_PROG_COPY); break;
        case SC_PROG_COPY * 2: KTB_SA(1, SC_PROG_COPY); break;
        case SC_PROG_AXPY0 * 2 + 1: KTB_SA(4, SC_PROG_AXPY0); break;
        case SC_PROG_AXPY1 * 2 + 1: KTB_SA(4, SC_PROG_AXPY1); break;
        default:
            if (a.vector_ok) KTB_SA(4, SC_PROG_VM);
            else KTB_SA(1, SC_PROG_VM);
    }
#undef KTB_SA
    KTB_CHECK_LAUNCH(ctx, "ktb_scatter_apply_kernel");
    return KTB_OK;
}

extern "C" int ktb_launch_scatter_rows(ktb_ctx* ctx, const ktb_rows_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    return ktb_scatter_rows_impl(ctx, *args, args->dev_rowid_scratch);
}
