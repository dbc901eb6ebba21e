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
// writer (ktir_cpu/memory.py:281-291).  The scatter path reproduces exactly that
// without sorting the whole index list and without floating-point atomics: the
// entries are bucketed by destination row (count, prefix sum, fill) and one warp
// per row replays that row's updates in tile order with the row in registers.
// HBM-bound: per entry one index and one row per gathered input; each touched
// destination row is read and written once.
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
        if (op.indirect > 1) {
            const int64_t jv = sc_read_index(arena, op.idx2_dtype, op.dev_idx2_off[t] + (int64_t)pos * op.idx2_stride);
            if (jv < 0) {
                if (atomicExch(&st->negative_index, 1) == 0) st->bad_index_value = (int32_t)jv;
                return -1;
            }
            a += jv * op.idx2_mult;
        }
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
// A warp resolves the addresses of `per_warp` entries at once (one per lane) and then moves their rows
// four at a time; with few entries per_warp is small, so that the rows spread over many warps
// instead of queueing behind one another in a few.
__global__ void __launch_bounds__(256) ktb_rows_program_kernel(const __grid_constant__ ktb_rows_args a, int per_warp,
                                                               ktb_status* st) {
    constexpr int G = 4;
    extern __shared__ float4 rp_vm[];                 // [KTB_VM_REGS][blockDim.x] register file
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t E = a.n_tiles * a.tile_rows;
    for (int64_t e0 = warp * per_warp; e0 < E; e0 += n_warps * per_warp) {
        const bool have = lane < per_warp && e0 + lane < E;
        const uint32_t e = (uint32_t)(have ? e0 + lane : 0);
        int64_t my_in[KTB_ROWS_MAX_IN];
        int64_t my_dst = -1;
        sc_resolve(a, e, st, my_in);
        if (have) {
            const uint32_t t = e / (uint32_t)a.tile_rows;
            my_dst = sc_row_addr(a.arena, a.out, t, (int)(e - t * (uint32_t)a.tile_rows), st);
        }
        const int cnt = (int)((E - e0) < per_warp ? (E - e0) : per_warp);
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

// ---- indirect destination -------------------------------------------------------------------------
// Entries are bucketed by destination row, then one warp per row replays that row's updates.
//   prepare: per tile, the destination row id of every entry; an entry that a later entry of the
//            same tile overwrites is dropped (last writer wins).  A surviving entry takes the next
//            slot of its row's bucket (atomic counter) and records its id and the resolved row
//            addresses of its gathered inputs; entries beyond the bucket capacity go to an
//            overflow list.
//   apply:   one warp per destination row orders its bucket by entry id — which is tile order —
//            and applies the updates one after another with the row held in registers: the row is
//            read once and written once however many tiles touch it.
// Scratch layout: int32 count[R + 2] (count[R] = overflow length, count[R + 1] = used part of `sorted`) |
// int32 bucket_e[R * C] | int64 bucket_addr[KTB_ROWS_MAX_IN][R * C] | int32 overflow[2 * E] (row, entry
// pairs) | int32 sorted[E] (per long row a segment with its entry ids in ascending order).
struct sc_scratch {
    int32_t* count;
    int32_t* bucket_e;
    int64_t* bucket_addr;     // [k][R * C]
    int32_t* overflow;
    int32_t* sorted;
    int32_t cap;              // C
    int64_t slots;            // R * C
};

static inline int sc_bucket_cap(int64_t E, int64_t R) {
    int64_t want = 2 * ((E + R - 1) / (R > 0 ? R : 1)) + 4;
    int c = 4;
    while (c < want && c < 32) c <<= 1;
    return c;
}

static inline size_t sc_scratch_bytes(int64_t E, int64_t R) {
    const int64_t slots = R * sc_bucket_cap(E, R);
    return (size_t)(4 * (R + 2) + 4 * slots + 8 + 8 * (int64_t)KTB_ROWS_MAX_IN * slots + 12 * E + 64);
}

static inline sc_scratch sc_carve(void* base, int64_t E, int64_t R) {
    sc_scratch s;
    s.cap = sc_bucket_cap(E, R);
    s.slots = R * s.cap;
    s.count = reinterpret_cast<int32_t*>(base);
    s.bucket_e = s.count + (R + 2);
    uintptr_t p = reinterpret_cast<uintptr_t>(s.bucket_e + s.slots);
    p = (p + 7) & ~(uintptr_t)7;
    s.bucket_addr = reinterpret_cast<int64_t*>(p);
    s.overflow = reinterpret_cast<int32_t*>(s.bucket_addr + (int64_t)KTB_ROWS_MAX_IN * s.slots);
    s.sorted = s.overflow + 2 * E;
    return s;
}

__global__ void __launch_bounds__(128) ktb_scatter_prepare_kernel(const __grid_constant__ ktb_rows_args a,
                                                                  const sc_scratch sc, ktb_status* st) {
    extern __shared__ int64_t s_addr[];      // [tile_rows]
    for (int64_t t = blockIdx.x; t < a.n_tiles; t += gridDim.x) {
        for (int pos = threadIdx.x; pos < a.tile_rows; pos += blockDim.x) {
            int64_t addr = sc_row_addr(a.arena, a.out, t, pos, st);
            if (addr >= 0) {
                const int64_t rel = addr - a.dst_row0;
                // rows that do not start on a row boundary of the destination cannot be ordered by id
                // (32-bit division when the operands fit: a 64-bit one costs more than the rest of the entry)
                int64_t q = -1, rem = 1;
                if (rel >= 0) {
                    if (((uint64_t)rel | (uint64_t)a.out.idx_mult) >> 32) {
                        q = rel / a.out.idx_mult;
                        rem = rel - q * a.out.idx_mult;
                    } else {
                        const uint32_t q32 = (uint32_t)rel / (uint32_t)a.out.idx_mult;
                        q = q32;
                        rem = (uint32_t)rel - q32 * (uint32_t)a.out.idx_mult;
                    }
                }
                addr = (rem == 0 && q < a.dst_rows) ? q : -1;
            }
            s_addr[pos] = addr;
        }
        __syncthreads();
        for (int pos = threadIdx.x; pos < a.tile_rows; pos += blockDim.x) {
            const int64_t mine = s_addr[pos];
            bool win = mine >= 0;
            for (int q = pos + 1; win && q < a.tile_rows; ++q) win = s_addr[q] != mine;
            if (!win) continue;
            const int32_t e = (int32_t)(t * a.tile_rows + pos);
            const int slot = atomicAdd(&sc.count[mine], 1);
            if (slot < sc.cap) {
                const int64_t at = mine * sc.cap + slot;
                sc.bucket_e[at] = e;
#pragma unroll
                for (int k = 0; k < KTB_ROWS_MAX_IN; ++k)
                    if (k < a.n_in && !a.in[k].alias_dst)
                        sc.bucket_addr[(int64_t)k * sc.slots + at] = sc_row_addr(a.arena, a.in[k], t, pos, st);
            } else {
                const int o = atomicAdd(&sc.count[a.dst_rows], 1);
                sc.overflow[2 * o] = (int32_t)mine;
                sc.overflow[2 * o + 1] = e;
            }
        }
        __syncthreads();
    }
}

template <int V, int PROG>
static __device__ __forceinline__ void sc_apply_one(const ktb_rows_args& a, const float (&x)[KTB_ROWS_MAX_IN][V],
                                                    float (&cur)[V], float4* vm, int vm_stride) {
    // inputs that alias the destination read the running value of the row
    float in[KTB_ROWS_MAX_IN][V];
#pragma unroll
    for (int k = 0; k < KTB_ROWS_MAX_IN; ++k)
#pragma unroll
        for (int v = 0; v < V; ++v) in[k][v] = (k < a.n_in && a.in[k].alias_dst) ? cur[v] : x[k][v];
    if (PROG == SC_PROG_COPY) {
#pragma unroll
        for (int v = 0; v < V; ++v) cur[v] = in[0][v];
    } else if (PROG == SC_PROG_AXPY0 || PROG == SC_PROG_AXPY1) {
        constexpr int ACC = PROG == SC_PROG_AXPY0 ? 0 : 1;
        const float c = a.program.ops[0].imm;
#pragma unroll
        for (int v = 0; v < V; ++v) cur[v] = ktb_round16(in[ACC][v] + ktb_round16(in[1 - ACC][v] * c));
    } else {
#pragma unroll
        for (int k = 0; k < KTB_ROWS_MAX_IN; ++k)
            vm[k * vm_stride] = make_float4(in[k][0], V > 1 ? in[k][1 % V] : 0.f, V > 1 ? in[k][2 % V] : 0.f,
                                            V > 1 ? in[k][3 % V] : 0.f);
        const float4 res = ktb_vm_run_smem4(a.program, vm, vm_stride);
        const float rv[4] = {res.x, res.y, res.z, res.w};
#pragma unroll
        for (int v = 0; v < V; ++v) cur[v] = rv[v];
    }
    // what is stored is rounded to the destination type, so the next update must see that value
    if (a.out.dtype == KTB_F16) {
#pragma unroll
        for (int v = 0; v < V; ++v) cur[v] = ktb_round16(cur[v]);
    }
}

template <int V, int PROG>
__global__ void __launch_bounds__(256, 4) ktb_scatter_apply_kernel(const __grid_constant__ ktb_rows_args a,
                                                                   const sc_scratch sc, ktb_status* st,
                                                                   const int only_long) {
    constexpr int G = 2;
    // only_long: the short chains were applied by the specialised kernel; without an overflow entry
    // no chain is long and there is nothing left to do
    if (only_long && sc.count[a.dst_rows] == 0) return;
    extern __shared__ float4 sa_vm[];                 // [KTB_VM_REGS][blockDim.x] register file
    float4* vm = sa_vm + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    bool rmw = false;
#pragma unroll
    for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) rmw = rmw || (k < a.n_in && a.in[k].alias_dst);

    // the count and the bucket of the NEXT row are fetched while the current row is applied, so only
    // the gathered rows themselves remain on the dependent-load path
    const int bl = lane < sc.cap ? lane : 0;
    int cnt_n = warp < a.dst_rows ? sc.count[warp] : 0;
    int32_t e_n = warp < a.dst_rows ? sc.bucket_e[warp * sc.cap + bl] : 0;
    int64_t in_n[KTB_ROWS_MAX_IN];
#pragma unroll
    for (int k = 0; k < KTB_ROWS_MAX_IN; ++k)
        in_n[k] = (warp < a.dst_rows && k < a.n_in && !a.in[k].alias_dst) ? sc.bucket_addr[(int64_t)k * sc.slots + warp * sc.cap + bl] : 0;

    for (int64_t row = warp; row < a.dst_rows; row += n_warps) {
        const int cnt = cnt_n;
        const int32_t e_cur = e_n;
        int64_t my_in[KTB_ROWS_MAX_IN];
#pragma unroll
        for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) my_in[k] = in_n[k];
        const int64_t nrow = row + n_warps;
        if (nrow < a.dst_rows) {
            cnt_n = sc.count[nrow];
            e_n = sc.bucket_e[nrow * sc.cap + bl];
#pragma unroll
            for (int k = 0; k < KTB_ROWS_MAX_IN; ++k)
                if (k < a.n_in && !a.in[k].alias_dst) in_n[k] = sc.bucket_addr[(int64_t)k * sc.slots + nrow * sc.cap + bl];
        }
        if (cnt == 0 || (only_long && cnt <= sc.cap)) continue;
        const int64_t dst = a.dst_row0 + row * a.out.idx_mult;
        if (cnt <= sc.cap) {
            const int32_t e = lane < cnt ? e_cur : 0x7fffffff;
            int rank = 0;
            for (int j = 0; j < cnt; ++j) rank += __shfl_sync(0xffffffffu, e, j) < e ? 1 : 0;
            const int first = rmw ? 0 : cnt - 1;      // a plain overwrite only keeps the last writer
            for (int c0 = 0; c0 < a.cols; c0 += 32 * V) {     // uniform trip count: the body shuffles
                const int col = c0 + lane * V;
                const bool act = col < a.cols;
                float cur[V];
#pragma unroll
                for (int v = 0; v < V; ++v) cur[v] = 0.f;
                if (rmw && act) sc_load_row<V>(a.arena, a.out, dst, col, a.cols, cur);
                for (int k0 = first; k0 < cnt; k0 += G) {
                    int64_t in_addr[G][KTB_ROWS_MAX_IN];
                    bool ok[G];
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const unsigned m = __ballot_sync(0xffffffffu, lane < cnt && rank == k0 + g);
                        const int src = m ? __ffs(m) - 1 : 0;
                        ok[g] = m != 0;
#pragma unroll
                        for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) {
                            in_addr[g][k] = 0;
                            if (k < a.n_in && !a.in[k].alias_dst) {
                                in_addr[g][k] = sc_shfl64(my_in[k], src);
                                ok[g] = ok[g] && in_addr[g][k] >= 0;
                            }
                        }
                    }
                    float x[G][KTB_ROWS_MAX_IN][V];
#pragma unroll
                    for (int g = 0; g < G; ++g)
#pragma unroll
                        for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) {
#pragma unroll
                            for (int v = 0; v < V; ++v) x[g][k][v] = 0.f;
                            if (act && ok[g] && k < a.n_in && !a.in[k].alias_dst)
                                sc_load_row<V>(a.arena, a.in[k], in_addr[g][k], col, a.cols, x[g][k]);
                        }
#pragma unroll
                    for (int g = 0; g < G; ++g)
                        if (ok[g]) sc_apply_one<V, PROG>(a, x[g], cur, vm, blockDim.x);
                }
                if (act) sc_store_row<V>(a.arena, a.out, dst, col, a.cols, cur);
            }
        } else {
            // long chain (more tiles hit this row than a bucket holds): its entries sit in the bucket and,
            // mixed with those of other rows, in the overflow list.  They are collected ONCE into a
            // segment of the `sorted` area, ordered there by entry id (= tile order), and then replayed
            // for every column chunk — cost O(list scan + n log^2 n + n * chunks) instead of a full
            // rescan of the lists for every single update.
            const int n_ovf = sc.count[a.dst_rows];
            int n = 0;
            int32_t* seg;
            {
                int seg0 = 0;
                if (lane == 0) seg0 = atomicAdd(&sc.count[a.dst_rows + 1], rmw ? cnt : 1);
                seg = sc.sorted + __shfl_sync(0xffffffffu, seg0, 0);
            }
            if (rmw) {
                for (int i0 = 0; i0 < sc.cap + n_ovf; i0 += 32) {
                    const int i = i0 + lane;
                    int32_t v = -1;
                    if (i < sc.cap) v = sc.bucket_e[row * sc.cap + i];
                    else if (i < sc.cap + n_ovf && sc.overflow[2 * (i - sc.cap)] == (int32_t)row) v = sc.overflow[2 * (i - sc.cap) + 1];
                    const unsigned m = __ballot_sync(0xffffffffu, v >= 0);
                    const int at = n + __popc(m & ((1u << lane) - 1u));
                    if (v >= 0 && at < cnt) seg[at] = v;
                    n += __popc(m);
                }
                if (n > cnt) n = cnt;
                __syncwarp();
                // bitonic network in which every comparator moves the smaller key to the lower index:
                // positions >= n behave like +infinity and never take part, so n need not be a power of two
                for (int k = 2; (k >> 1) < n; k <<= 1) {
                    for (int j = k >> 1; j > 0; j >>= 1) {
                        for (int i = lane; i < n; i += 32) {
                            const int p = (j == (k >> 1)) ? (i ^ (k - 1)) : (i ^ j);
                            if (p > i && p < n) {
                                const int32_t lo = seg[i], hi = seg[p];
                                if (lo > hi) { seg[i] = hi; seg[p] = lo; }
                            }
                        }
                        __syncwarp();
                    }
                }
            } else {
                // plain overwrite: only the last writer matters
                int32_t best = -1;
                for (int i = lane; i < sc.cap + n_ovf; i += 32) {
                    int32_t v = -1;
                    if (i < sc.cap) v = sc.bucket_e[row * sc.cap + i];
                    else if (sc.overflow[2 * (i - sc.cap)] == (int32_t)row) v = sc.overflow[2 * (i - sc.cap) + 1];
                    best = max(best, v);
                }
                for (int d = 16; d; d >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, d));
                if (lane == 0) seg[0] = best;
                n = best >= 0 ? 1 : 0;
                __syncwarp();
            }
            for (int c0 = 0; c0 < a.cols; c0 += 32 * V) {
                const int col = c0 + lane * V;
                const bool act = col < a.cols;
                float cur[V];
#pragma unroll
                for (int v = 0; v < V; ++v) cur[v] = 0.f;
                if (rmw && act) sc_load_row<V>(a.arena, a.out, dst, col, a.cols, cur);
                for (int step = 0; step < n; ++step) {
                    int64_t in_addr[KTB_ROWS_MAX_IN];
                    sc_resolve(a, (uint32_t)seg[step], st, in_addr);
                    bool ok = true;
                    float x[KTB_ROWS_MAX_IN][V];
#pragma unroll
                    for (int k = 0; k < KTB_ROWS_MAX_IN; ++k) {
#pragma unroll
                        for (int v = 0; v < V; ++v) x[k][v] = 0.f;
                        if (k < a.n_in && !a.in[k].alias_dst) ok = ok && in_addr[k] >= 0;
                    }
#pragma unroll
                    for (int k = 0; k < KTB_ROWS_MAX_IN; ++k)
                        if (act && ok && k < a.n_in && !a.in[k].alias_dst)
                            sc_load_row<V>(a.arena, a.in[k], in_addr[k], col, a.cols, x[k]);
                    if (ok) sc_apply_one<V, PROG>(a, x, cur, vm, blockDim.x);
                }
                if (act) sc_store_row<V>(a.arena, a.out, dst, col, a.cols, cur);
            }
        }
    }
}

// The common scatter of embedding-style updates, specialised: out[row] = out[row] (+) c * src[..] on
// rows of 128 f16 (a lane holds 4 elements), every chain no longer than a bucket.  Same order and
// rounding as the general kernel (one f16 rounding after the multiply, one after the add), about a
// quarter of its instructions: no operand descriptors, no per-element guards, rows loaded four at a
// time before the dependent adds.
template <int ACC>
__global__ void __launch_bounds__(256, 6) ktb_scatter_apply_axpy128_kernel(const __grid_constant__ ktb_rows_args a,
                                                                          const sc_scratch sc, ktb_status* st) {
    constexpr int K = 1 - ACC;                      // the gathered operand
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const __half* arena = reinterpret_cast<const __half*>(a.arena);
    __half* arena_w = reinterpret_cast<__half*>(a.arena);
    const __half2 c2 = __float2half2_rn(a.program.ops[0].imm);      // the scale is an f16 value (checked on the host)
    const int64_t in_lo = a.in[K].lo, in_hi = a.in[K].hi - 128;
    const int64_t* baddr = sc.bucket_addr + (int64_t)K * sc.slots;
    const int bl = lane < sc.cap ? lane : 0;
    int cnt_n = warp < a.dst_rows ? sc.count[warp] : 0;
    int32_t e_n = warp < a.dst_rows ? sc.bucket_e[warp * sc.cap + bl] : 0;
    int64_t ad_n = warp < a.dst_rows ? baddr[warp * sc.cap + bl] : 0;
    for (int64_t row = warp; row < a.dst_rows; row += n_warps) {
        const int cnt = cnt_n;
        const int32_t e = lane < cnt ? e_n : 0x7fffffff;
        const int64_t my_ad = ad_n;
        const int64_t nrow = row + n_warps;
        if (nrow < a.dst_rows) {
            cnt_n = sc.count[nrow];
            e_n = sc.bucket_e[nrow * sc.cap + bl];
            ad_n = baddr[nrow * sc.cap + bl];
        }
        if (cnt == 0 || cnt > sc.cap) continue;      // long chains are left to the general kernel
        int rank = 0;
        for (int j = 0; j < cnt; ++j) rank += __shfl_sync(0xffffffffu, e, j) < e ? 1 : 0;
        __half* drow = arena_w + a.dst_row0 + row * a.out.idx_mult + lane * 4;
        // f16 multiply and add with one rounding each are what NumPy's half ufuncs compute (f32
        // arithmetic on f16 inputs rounds to the same f16 value: 24 >= 2 * 11 + 2 bits); the _rn
        // forms are never contracted into a fused multiply-add
        uint2 raw = *reinterpret_cast<const uint2*>(drow);
        __half2 cur0 = *reinterpret_cast<const __half2*>(&raw.x), cur1 = *reinterpret_cast<const __half2*>(&raw.y);
        for (int j0 = 0; j0 < cnt; j0 += 4) {
            uint2 x[4];
            bool use[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                x[g] = make_uint2(0u, 0u);
                use[g] = false;
                if (j0 + g < cnt) {                  // uniform
                    const unsigned m = __ballot_sync(0xffffffffu, lane < cnt && rank == j0 + g);
                    const int64_t ad = sc_shfl64(my_ad, __ffs(m) - 1);
                    use[g] = ad >= 0;                // an unresolved (negative) index was reported by prepare
                    if (ad >= in_lo && ad <= in_hi) {
                        x[g] = __ldg(reinterpret_cast<const uint2*>(arena + ad + lane * 4));
                    } else if (ad >= 0 && ad + 128 > in_lo && ad < in_hi + 128) {
                        // a row that straddles the end of its allocation: elements outside read as 0
                        __half h[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int64_t el = ad + lane * 4 + i;
                            h[i] = (el >= in_lo && el < in_hi + 128) ? arena[el] : __float2half(0.f);
                        }
                        x[g] = *reinterpret_cast<const uint2*>(h);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                if (!use[g]) continue;
                cur0 = __hadd2_rn(cur0, __hmul2_rn(*reinterpret_cast<const __half2*>(&x[g].x), c2));
                cur1 = __hadd2_rn(cur1, __hmul2_rn(*reinterpret_cast<const __half2*>(&x[g].y), c2));
            }
        }
        raw.x = *reinterpret_cast<const uint32_t*>(&cur0);
        raw.y = *reinterpret_cast<const uint32_t*>(&cur1);
        *reinterpret_cast<uint2*>(drow) = raw;
    }
}

// The same with TWO destination rows per warp, one per half-warp (a lane holds 8 elements), for buckets of at
// most 16 entries: the rank and selection steps — shuffles, votes, address checks, the bulk of the
// instructions of a row in the one-row kernel, which is issue-bound — serve both rows at once.  Order
// and rounding are those of the kernel above.
template <int ACC>
#ifndef KTB_H_OCC
#define KTB_H_OCC 4
#endif
__global__ void __launch_bounds__(256, KTB_H_OCC) ktb_scatter_apply_axpy128h_kernel(const __grid_constant__ ktb_rows_args a,
                                                                           const sc_scratch sc, ktb_status* st) {
    constexpr int K = 1 - ACC;                      // the gathered operand
    const int lane = threadIdx.x & 31, hl = lane & 15, half = lane >> 4;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const __half* arena = reinterpret_cast<const __half*>(a.arena);
    __half* arena_w = reinterpret_cast<__half*>(a.arena);
    const __half2 c2 = __float2half2_rn(a.program.ops[0].imm);      // the scale is an f16 value (checked on the host)
    const int64_t in_lo = a.in[K].lo, in_hi = a.in[K].hi - 128;
    const int64_t* baddr = sc.bucket_addr + (int64_t)K * sc.slots;
    const int bl = hl < sc.cap ? hl : 0;
    int64_t row = warp * 2 + half;
    bool have = row < a.dst_rows;
    int cnt_n = have ? sc.count[row] : 0;
    int32_t e_n = have ? sc.bucket_e[row * sc.cap + bl] : 0;
    int64_t ad_n = have ? baddr[row * sc.cap + bl] : 0;
    for (; __any_sync(0xffffffffu, have); row += n_warps * 2) {
        have = row < a.dst_rows;
        int cnt = have ? cnt_n : 0;
        if (cnt > sc.cap) cnt = 0;                   // long chains are left to the general kernel
        const int32_t e = hl < cnt ? e_n : 0x7fffffff;
        const int64_t my_ad = ad_n;
        const int64_t nrow = row + n_warps * 2;
        if (nrow < a.dst_rows) {
            cnt_n = sc.count[nrow];
            e_n = sc.bucket_e[nrow * sc.cap + bl];
            ad_n = baddr[nrow * sc.cap + bl];
        }
        const int other = __shfl_xor_sync(0xffffffffu, cnt, 16);
        const int cmax = cnt > other ? cnt : other;  // the two halves walk their chains in step
        if (cmax == 0) continue;
        int rank = 0;
        for (int j = 0; j < cmax; ++j) rank += __shfl_sync(0xffffffffu, e, j, 16) < e ? 1 : 0;
        __half* drow = arena_w + a.dst_row0 + (have ? row : 0) * a.out.idx_mult + hl * 8;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (cnt > 0) raw = *reinterpret_cast<const uint4*>(drow);
        __half2* cur = reinterpret_cast<__half2*>(&raw);
        for (int j0 = 0; j0 < cmax; j0 += 4) {
            uint4 x[4];
            bool use[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                x[g] = make_uint4(0u, 0u, 0u, 0u);
                use[g] = false;
                if (j0 + g < cmax) {                 // uniform
                    const unsigned m = __ballot_sync(0xffffffffu, hl < cnt && rank == j0 + g);
                    const unsigned mine = (m >> (half * 16)) & 0xffffu;       // the entry of my half, if it has one left
                    const int64_t ad = sc_shfl64(my_ad, mine ? __ffs(mine) - 1 + half * 16 : lane);
                    use[g] = mine != 0 && ad >= 0;   // an unresolved (negative) index was reported by prepare
                    if (mine == 0) {
                    } else if (ad >= in_lo && ad <= in_hi) {
                        if ((ad & 7) == 0) {
                            x[g] = __ldg(reinterpret_cast<const uint4*>(arena + ad + hl * 8));
                        } else {                     // gathered rows start on multiples of 4 elements only
                            const uint2 p0 = __ldg(reinterpret_cast<const uint2*>(arena + ad + hl * 8));
                            const uint2 p1 = __ldg(reinterpret_cast<const uint2*>(arena + ad + hl * 8 + 4));
                            x[g] = make_uint4(p0.x, p0.y, p1.x, p1.y);
                        }
                    } else if (ad >= 0 && ad + 128 > in_lo && ad < in_hi + 128) {
                        // a row that straddles the end of its allocation: elements outside read as 0
                        __half h[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int64_t el = ad + hl * 8 + i;
                            h[i] = (el >= in_lo && el < in_hi + 128) ? arena[el] : __float2half(0.f);
                        }
                        x[g] = *reinterpret_cast<const uint4*>(h);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                if (!use[g]) continue;
                const __half2* xv = reinterpret_cast<const __half2*>(&x[g]);
#pragma unroll
                for (int i = 0; i < 4; ++i) cur[i] = __hadd2_rn(cur[i], __hmul2_rn(xv[i], c2));
            }
        }
        if (cnt > 0) *reinterpret_cast<uint4*>(drow) = raw;
    }
}

static bool sc_axpy128_ok(const ktb_rows_args& a, int acc) {
    if (a.n_in != 2 || !a.in[acc].alias_dst || a.in[1 - acc].alias_dst || !a.vector_ok || a.cols != 128) return false;
    if (a.in[0].dtype != KTB_F16 || a.in[1].dtype != KTB_F16 || a.out.dtype != KTB_F16) return false;
    const float c = a.program.ops[0].imm;
    if (!(__half2float(__float2half_rn(c)) == c)) return false;      // the scale must be exact in f16
    if (a.dst_rows <= 0 || a.dst_row0 < a.out.lo || a.dst_row0 + (a.dst_rows - 1) * a.out.idx_mult + 128 > a.out.hi) return false;
    return (a.dst_row0 % 4) == 0 && (a.out.idx_mult % 4) == 0;
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
        if (op.indirect < 0 || op.indirect > (k < a.n_in ? 2 : 1))
            return ktb_fail(ctx, KTB_E_UNSUPPORTED, who, "an input takes at most two index lookups, the destination one");
        if (op.indirect > 1 && (!op.dev_idx2_off || (op.idx2_dtype != KTB_I32 && op.idx2_dtype != KTB_I64)))
            return ktb_fail(ctx, KTB_E_ARG, who, "second index lookup needs offsets and an i32 or i64 dtype");
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
    const int64_t cap = (int64_t)ctx->sm_count * 16;                 // CTAs of 8 warps
    int per_warp = (int)((E + cap * 8 - 1) / (cap * 8));             // entries a warp takes when all warps are used
    per_warp = per_warp >= 32 ? 32 : (per_warp + 3) / 4 * 4;
    int64_t blocks = (E + (int64_t)per_warp * 8 - 1) / ((int64_t)per_warp * 8);
    if (blocks > cap) blocks = cap;
    const size_t vsmem = (size_t)KTB_VM_REGS * 256 * sizeof(float4);
#define KTB_RP(V, P) ktb_rows_program_kernel<V, P><<<(unsigned)blocks, 256, vsmem, ctx->stream>>>(a, per_warp, ctx->dev_status)
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
    const int64_t E = a.n_tiles * a.tile_rows, R = a.dst_rows;
    const sc_scratch sc = sc_carve(scratch, E, R);
    KTB_CUDA(ctx, cudaMemsetAsync(sc.count, 0, (size_t)(R + 2) * sizeof(int32_t), ctx->stream));
    int64_t prep_blocks = a.n_tiles < (1 << 20) ? a.n_tiles : (1 << 20);
    const size_t smem = (size_t)a.tile_rows * sizeof(int64_t);
    if (smem > 48 * 1024) return ktb_fail(ctx, KTB_E_UNSUPPORTED, "scatter_rows", "tile has too many rows");
    int prep_threads = (a.tile_rows + 31) / 32 * 32;
    if (prep_threads > 128) prep_threads = 128;
    ktb_scatter_prepare_kernel<<<(unsigned)prep_blocks, prep_threads, smem, ctx->stream>>>(a, sc, ctx->dev_status);
    KTB_CHECK_LAUNCH(ctx, "ktb_scatter_prepare_kernel");
    int64_t blocks = (R + 7) / 8;
    if (blocks > (int64_t)ctx->sm_count * 32) blocks = (int64_t)ctx->sm_count * 32;
    const size_t asmem = (size_t)KTB_VM_REGS * 256 * sizeof(float4);
    const int prog = sc_classify(a);
    int only_long = 0;
    if ((prog == SC_PROG_AXPY0 || prog == SC_PROG_AXPY1) && sc_axpy128_ok(a, prog == SC_PROG_AXPY0 ? 0 : 1)) {
        int64_t fb = (R + 7) / 8;
        if (fb > (int64_t)ctx->sm_count * 6) fb = (int64_t)ctx->sm_count * 6;      // resident CTAs; rows are strided over them
        const bool halves = sc.cap <= 16 && (a.dst_row0 % 8) == 0 && (a.out.idx_mult % 8) == 0;
#ifdef KTB_SCATTER_NO_HALVES
        const bool two_rows = false;
#else
        const bool two_rows = halves;
#endif
        if (two_rows) {
            fb = (R + 15) / 16;
            if (fb > (int64_t)ctx->sm_count * KTB_H_OCC) fb = (int64_t)ctx->sm_count * KTB_H_OCC;
            if (prog == SC_PROG_AXPY0) ktb_scatter_apply_axpy128h_kernel<0><<<(unsigned)fb, 256, 0, ctx->stream>>>(a, sc, ctx->dev_status);
            else ktb_scatter_apply_axpy128h_kernel<1><<<(unsigned)fb, 256, 0, ctx->stream>>>(a, sc, ctx->dev_status);
        } else if (prog == SC_PROG_AXPY0) ktb_scatter_apply_axpy128_kernel<0><<<(unsigned)fb, 256, 0, ctx->stream>>>(a, sc, ctx->dev_status);
        else ktb_scatter_apply_axpy128_kernel<1><<<(unsigned)fb, 256, 0, ctx->stream>>>(a, sc, ctx->dev_status);
        KTB_CHECK_LAUNCH(ctx, "ktb_scatter_apply_axpy128_kernel");
        only_long = 1;
        blocks = ctx->sm_count;          // the general kernel only sweeps for chains longer than a bucket
    }
#define KTB_SA(V, P) ktb_scatter_apply_kernel<V, P><<<(unsigned)blocks, 256, asmem, ctx->stream>>>(a, sc, ctx->dev_status, only_long)
    switch (prog * 2 + (a.vector_ok ? 1 : 0)) {
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

extern "C" size_t ktb_scatter_scratch_bytes(int64_t entries, int64_t dst_rows) {
    return sc_scratch_bytes(entries, dst_rows);
}

extern "C" int ktb_launch_scatter_rows(ktb_ctx* ctx, const ktb_rows_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    return ktb_scatter_rows_impl(ctx, *args, args->dev_rowid_scratch);
}

// ---- scatter without a caller-provided scratch buffer ---------------------------------------
// The same launches as ktb_launch_scatter_rows, with the bucket scratch taken from a fixed array
// in device global memory that is part of the loaded library image.  The entry point performs no
// device or host allocation of any kind, so it can be used by callers that must not allocate:
// code running while an allocator lock is held, a steady-state serving loop whose memory budget
// was fixed at start-up, or a host thread that may not synchronise with the device (cudaFree and
// some cudaMalloc calls do).
//
// The array's name in host code is only a handle of the symbol; the device address is looked up
// with cudaGetSymbolAddress once per device, on the first call for that device, with that device
// made current.  That first call should therefore come before any stream capture is started.
// All calls on a device share the one array: nothing in it needs to survive between calls (the
// per-row counters, the only part that must start at zero, are cleared on the stream at the start
// of every call), but two calls in flight at the same time on different streams would race on it.
static __device__ __align__(256) unsigned char ktb_scatter_static_scratch[KTB_SCATTER_STATIC_BYTES];

#define KTB_STATIC_MAX_DEVICES 64
static int32_t* sc_static_ptr[KTB_STATIC_MAX_DEVICES];   // device address of the array, per device

extern "C" int ktb_launch_scatter_rows_static(ktb_ctx* ctx, const ktb_rows_args* args) {
    if (!ctx || !args) return KTB_E_ARG;
    const ktb_rows_args& a = *args;
    if (a.n_tiles < 0 || a.tile_rows <= 0 || a.dst_rows <= 0)
        return ktb_fail(ctx, KTB_E_ARG, "scatter_rows_static", "bad tile or destination row geometry");
    if (a.n_tiles >= (1ll << 31) / a.tile_rows || a.dst_rows >= (1ll << 31))
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "scatter_rows_static", "too many entries or destination rows");
    const size_t need = sc_scratch_bytes(a.n_tiles * a.tile_rows, a.dst_rows);
    if (need > (size_t)KTB_SCATTER_STATIC_BYTES) {
        char msg[160];
        snprintf(msg, sizeof(msg), "needs %zu bytes of scratch, the built-in array holds %zu; use ktb_launch_scatter_rows",
                 need, (size_t)KTB_SCATTER_STATIC_BYTES);
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "scatter_rows_static", msg);
    }
    if (ctx->device < 0 || ctx->device >= KTB_STATIC_MAX_DEVICES)
        return ktb_fail(ctx, KTB_E_UNSUPPORTED, "scatter_rows_static", "device ordinal out of range");
    KTB_CUDA(ctx, cudaSetDevice(ctx->device));
    if (!sc_static_ptr[ctx->device]) {
        void* p = nullptr;
        KTB_CUDA(ctx, cudaGetSymbolAddress(&p, ktb_scatter_static_scratch));
        if (!p) return ktb_fail(ctx, KTB_E_CUDA, "scatter_rows_static", "symbol lookup returned a null address");
        sc_static_ptr[ctx->device] = reinterpret_cast<int32_t*>(p);
    }
    return ktb_scatter_rows_impl(ctx, a, sc_static_ptr[ctx->device]);
}
