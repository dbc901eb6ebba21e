/*
 * ktir_b200 — C ABI of the B200 execution backend for KTIR kernels.
 *
 * The reference interpreter is pure Python and has no foreign-function layer;
 * every entry point below names the Python routine whose work it takes over
 * (paths are relative to the reference project root).  All functions return 0
 * on success or a negative KTB_E_* code; ktb_last_error() gives the message.
 * Pointers named `dev*`/`arena` are device addresses, everything else is host
 * memory that the call copies before returning.  One context per (process,
 * device); a context is not thread-safe.
 */
#ifndef KTIR_B200_H
#define KTIR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ktb_ctx ktb_ctx;

enum { KTB_OK = 0, KTB_E_CUDA = -1, KTB_E_ARG = -2, KTB_E_UNSUPPORTED = -3, KTB_E_DEVICE_STATUS = -4 };

/* element type codes */
enum { KTB_F16 = 0, KTB_F32 = 1, KTB_I32 = 2, KTB_I64 = 3, KTB_I1 = 4 };

/* Device status word read back by ktb_sync(): kernels never trap; they record
 * what went wrong here and return (ktir_cpu/ops/memory_ops.py:378-382 raises
 * IndexError for a negative indirect index; ktir_cpu/grid.py:615-621 reports
 * deadlock). */
typedef struct {
    int32_t negative_index;   /* != 0: an indirect index was negative */
    int32_t bad_index_value;  /* the offending value */
    int32_t wait_timeout;     /* != 0: a bounded device-side wait ran out */
    int32_t wait_site;        /* which wait gave up */
    int32_t reserved[4];
} ktb_status;

/* ---- context, memory, transfers ------------------------------------------
 * Replaces SpyreMemoryHierarchy/HBMSimulator set-up, argument upload and
 * read-back in KTIRInterpreter.execute_function
 * (ktir_cpu/interpreter.py:95-120,156-194; ktir_cpu/memory.py:311-398). */
int ktb_init(int device, ktb_ctx** out);
int ktb_destroy(ktb_ctx* ctx);
const char* ktb_last_error(ktb_ctx* ctx);
int ktb_alloc(ktb_ctx* ctx, size_t bytes, void** dev_ptr);
int ktb_free(ktb_ctx* ctx, void* dev_ptr);
int ktb_alloc_host(ktb_ctx* ctx, size_t bytes, void** host_ptr);   /* pinned */
int ktb_free_host(ktb_ctx* ctx, void* host_ptr);
int ktb_memset(ktb_ctx* ctx, void* dev_ptr, int byte_value, size_t bytes);
int ktb_h2d(ktb_ctx* ctx, void* dev_dst, const void* host_src, size_t bytes);
int ktb_d2h(ktb_ctx* ctx, void* host_dst, const void* dev_src, size_t bytes);
int ktb_d2d(ktb_ctx* ctx, void* dev_dst, const void* dev_src, size_t bytes);
int ktb_sync(ktb_ctx* ctx, ktb_status* status_out);
/* Use an existing CUDA stream (e.g. torch's current stream) for all work. */
int ktb_set_stream(ktb_ctx* ctx, uint64_t cuda_stream);
/* CUDA-event timing on the context's stream; slot in [0, 64). */
int ktb_event_record(ktb_ctx* ctx, int slot);
int ktb_event_elapsed_ms(ktb_ctx* ctx, int slot_begin, int slot_end, float* ms_out);
/* Record an event slot on the launch stream (lane 0) or a copy lane (1, 2) and wait for one on the
 * host: several calls can be in flight and each is retired on its own, without ktb_sync. */
int ktb_event_record_on(ktb_ctx* ctx, int slot, int lane);
int ktb_event_sync(ktb_ctx* ctx, int slot);
/* Queue, on the launch stream, a copy of the device status word into page-locked host memory
 * followed by its reset: what the kernels queued so far reported, attributable to one call
 * (read it after an event recorded behind it has completed). */
int ktb_status_snapshot(ktb_ctx* ctx, ktb_status* host_pinned);
/* Write `bytes` (> L2 size) of scratch so the next kernel starts with a cold L2. */
int ktb_flush_l2(ktb_ctx* ctx);
/* Number of kernels this library has launched on the context so far. */
int64_t ktb_launch_count(ktb_ctx* ctx);
/* Record the launches issued between begin and end (they do not run) and replay them with one
 * ktb_graph_launch — the per-op dispatch loop of the reference (ktir_cpu/interpreter.py:343-395)
 * collapses into a single submission.  The recorded calls must not allocate; arguments and
 * device pointers are frozen at capture time. */
int ktb_graph_begin(ktb_ctx* ctx);
int ktb_graph_end(ktb_ctx* ctx, void** graph_out);
int ktb_graph_launch(ktb_ctx* ctx, void* graph);
int ktb_graph_destroy(ktb_ctx* ctx, void* graph);

/* ---- pipelined transfers ---------------------------------------------------------------
 * Two copy lanes (streams) beside the launch stream: lane 1 uploads, lane 2 reads back; 0 names
 * the launch stream.  ktb_lane_fence(from, to) makes everything queued later on `to` wait for
 * what is queued on `from` so far; ktb_lane_d2h queues a read-back of `height` rows of `width`
 * bytes, `pitch` bytes apart on both sides, on lane 2 (host_dst page-locked).  ktb_sync also
 * waits for both lanes.
 *
 * ktb_run_pipeline is KTIRInterpreter.execute_function's data movement
 * (ktir_cpu/interpreter.py:156-194: a flatten() copy of every ndarray argument into simulated
 * memory, the run, a read-back of every argument into a new array) as one overlapped pass.  Per
 * tensor t the caller gives src[t], its own array, and pinned[t], a page-locked array of the same
 * layout that it will hand back.  A chunk lists the regions it needs on the device (`up`), an
 * optional launch and the regions to read back (`down`).  Host threads copy the `up` regions
 * src -> pinned for all chunks, in order; the calling thread follows behind: when a chunk's
 * copies have landed it queues their DMAs pinned -> arena on lane 1, fences, calls
 * launch(ctx, launch_args) (any ktb_launch_* with its argument struct), fences and queues the
 * `down` DMAs arena -> pinned on lane 2.  So one host copy yields the upload and the caller's
 * fresh array, and upload, kernels and read-back of neighbouring chunks overlap.  A region with
 * dev_off == KTB_NO_DEVICE is copied on the host only; src[t] == pinned[t] skips the host copy.
 * Returns once everything is queued (ktb_sync waits for it).  ktb_set_copy_threads sizes the
 * process-wide pool of copy threads (default: half the hardware threads, at most 8). */
#define KTB_NO_DEVICE UINT64_MAX
typedef struct {
    int32_t tensor;            /* index into pinned[] / src[] */
    int32_t reserved;
    uint64_t dev_off;          /* byte offset in the arena, or KTB_NO_DEVICE */
    uint64_t rel;              /* byte offset inside the tensor */
    uint64_t width, height, pitch;   /* rows of `width` bytes, `pitch` apart (height 1: one run) */
} ktb_region;
typedef struct {
    int (*launch)(ktb_ctx*, const void*);   /* may be NULL */
    const void* launch_args;
    int32_t n_up, n_down;
    const ktb_region* up;
    const ktb_region* down;
} ktb_pipe_chunk;
int ktb_run_pipeline(ktb_ctx* ctx, void* arena, const ktb_pipe_chunk* chunks, int n_chunks, void* const* pinned,
                     const void* const* src, int n_tensors);
/* ktb_run_pipeline handed to the context's submission thread: the call copies its arguments (not
 * the tensors), returns at once with a sequence number, and the thread stages, queues and — when
 * given — snapshots the status word into `snapshot` (page-locked) and records event `event_slot`
 * behind the job's last device work.  Jobs are issued in submission order.  While jobs are
 * pending the caller must not queue other work on the context; ktb_wait_submitted(seq) returns
 * once job `seq` has been issued (its event can then be waited for) and reports the first
 * error of the jobs up to it; ktb_sync waits for all of them.  This is how a batch of
 * candidate kernels keeps the host preparing call i+1 while call i is being staged
 * (notebooks/demo_helpers.py:32-46 runs them one after the other). */
int ktb_submit_pipeline(ktb_ctx* ctx, void* arena, const ktb_pipe_chunk* chunks, int n_chunks, void* const* pinned,
                        const void* const* src, int n_tensors, ktb_status* snapshot, int event_slot, uint64_t* seq_out);
int ktb_wait_submitted(ktb_ctx* ctx, uint64_t seq);
int ktb_lane_fence(ktb_ctx* ctx, int from, int to);
int ktb_lane_d2h(ktb_ctx* ctx, void* host_dst, const void* dev_src, size_t width, size_t height, size_t pitch);
int ktb_set_copy_threads(int n);
int ktb_copy_threads(void);

/* ---- elementwise register programs ---------------------------------------
 * A short straight-line program over f32 registers; inputs are loaded into
 * registers 0..n_in-1.  Replaces per-op NumPy dispatch of the arith/math
 * dialects (ktir_cpu/dialects/_helpers.py:39-72, ktir_cpu/dialects/arith_ops.py:49-308,
 * ktir_cpu/ops/math_ops.py:27-138).  Setting KTB_VM_ROUND16 on an op rounds its
 * result to f16 (round-to-nearest-even), which is how NumPy evaluates f16 tiles. */
enum {
    KTB_VM_MOV = 0, KTB_VM_CONST, KTB_VM_ADD, KTB_VM_SUB, KTB_VM_MUL, KTB_VM_DIV,
    KTB_VM_MAX, KTB_VM_MAXNUM, KTB_VM_MIN, KTB_VM_MINNUM, KTB_VM_NEG, KTB_VM_ABS,
    KTB_VM_EXP, KTB_VM_LOG, KTB_VM_LOG2, KTB_VM_SQRT, KTB_VM_RSQRT, KTB_VM_TANH,
    KTB_VM_SIN, KTB_VM_COS, KTB_VM_FMA, KTB_VM_NOPS,
    KTB_VM_ROUND16 = 0x100,
    /* row-value programs of ktb_launch_row_program only (row scalars, per-row and side results): operand a / b of
       the op is `imm` instead of a register, which saves the KTB_VM_CONST op in front of it */
    KTB_VM_IMM_A = 0x200, KTB_VM_IMM_B = 0x400
};
#define KTB_VM_MAX_OPS 12
#define KTB_VM_MAX_IN 4
#define KTB_VM_REGS 8

typedef struct {
    int32_t opcode;      /* KTB_VM_* | optional KTB_VM_ROUND16 | (row-value programs) KTB_VM_IMM_A / _B */
    int32_t dst, a, b, c;
    float imm;
} ktb_vm_op;

typedef struct {
    int32_t n_in;
    int32_t n_ops;
    int32_t result_reg;
    int32_t reserved;
    ktb_vm_op ops[KTB_VM_MAX_OPS];
} ktb_vm_program;

/* ---- fused load -> elementwise -> store over all grid cores ----------------
 * One launch covers every (core, loop iteration) work item of a statement:
 * ktdp.load of each operand tile (ktir_cpu/dialects/ktdp_ops.py:200-227,
 * ktir_cpu/ops/memory_ops.py:723-800), the elementwise ops between, and the
 * ktdp.store (ktdp_ops.py:230-260, memory_ops.py:802-865).  Tiles are rows x
 * cols with unit column stride; item_offsets holds, per item, the element
 * offset of each input and then of the output, relative to `arena`. */
typedef struct {
    void* arena;
    const int64_t* dev_item_offsets;   /* [n_items][n_in + 1] */
    int64_t n_items;
    int32_t rows, cols;
    int64_t row_stride[KTB_VM_MAX_IN + 1];   /* elements; inputs then output */
    int32_t dtype[KTB_VM_MAX_IN + 1];        /* KTB_F16 / KTB_F32 */
    int32_t vector_ok;   /* 1: cols, every item offset and row stride are multiples of 8 elements */
    ktb_vm_program program;
} ktb_ew_args;
int ktb_launch_ew_stream(ktb_ctx* ctx, const ktb_ew_args* args);

/* ---- fused row softmax --------------------------------------------------------
 * load -> [extf] -> reduce(max) -> sub -> exp -> reduce(add) -> div -> [truncf]
 * -> store, one row per CTA.  Replaces the op sequence a softmax kernel runs per
 * row through linalg.reduce's pairwise fold (ktir_cpu/dialects/linalg_ops.py:86-246),
 * math.exp (ktir_cpu/ops/_helpers.py:50-60) and the arith binops.  The reduction
 * follows the same halving order (x[i] op x[i+h]) when cols is a power of two. */
typedef struct {
    void* arena;
    const int64_t* dev_item_offsets;   /* [n_items][2]: input, output element offsets */
    int64_t n_items;
    int32_t rows_per_item, cols;
    int64_t in_row_stride, out_row_stride;   /* elements */
    int32_t in_dtype, out_dtype;             /* KTB_F16 / KTB_F32 */
    int32_t f16_arith;      /* 1: every op rounds to f16 (tile dtype f16 throughout) */
    int32_t max_is_maxnum;  /* 1: arith.maxnumf (NaN ignored), 0: maximumf */
    float max_init, sum_init;   /* the `outs` initial values of the two reductions */
} ktb_softmax_args;
int ktb_launch_row_softmax(ktb_ctx* ctx, const ktb_softmax_args* args);

/* ---- fused row programs: elementwise ops and row reductions in one pass over HBM ----------
 * A statement whose value mixes elementwise ops with reductions along the last tile dimension — layer
 * norm, RMS norm, softmax variants the softmax kernel does not take — runs as up to KTB_RP_MAX_RED
 * reduction phases and one output phase per row.  Phase p evaluates a register program on every
 * 8-element vector of the row (inputs: the operand tiles, then the row scalars known so far) and
 * folds the results with `op` in the pairing order of the reference's linalg.reduce
 * (ktir_cpu/dialects/linalg_ops.py:86-246); row scalars (mean, 1/sqrt(var + eps), ...) are register
 * programs over the reduction results, evaluated once per row; the output phase stores its
 * program's result.  A row is read from HBM once: later phases find it in L1/L2.  Replaces the op
 * sequence linalg.reduce -> arith/math ops on the reduced tile -> broadcast -> elementwise ops
 * (ktir_cpu/dialects/linalg_ops.py:136-246, 349-465; ktir_cpu/dialects/arith_ops.py:49-308) with the
 * same rounding points.  cols: power of two in [8, 16384]; offsets and strides multiples of 8. */
#define KTB_RP_MAX_RED 3
#define KTB_RP_MAX_SCAL 4
#define KTB_RP_MAX_SIDE 2
enum { KTB_RP_ADD = 0, KTB_RP_MAX = 1, KTB_RP_MAXNUM = 2 };
typedef struct {
    ktb_vm_program prog;      /* vector program; registers 0..n_in-1 = operand tiles, n_in..n_in+n_scal-1 = row scalars */
    int32_t op;               /* KTB_RP_* */
    int32_t round16;          /* 1: the fold rounds to f16 after every combine (an f16 tile is reduced) */
    int32_t load_mask;        /* bit k: the program reads operand k */
    int32_t blocked;          /* 1: a row is `n_blocks` column blocks of `cols` elements (operand k's blocks are
                                 blk_stride[k] elements apart).  A reduction phase evaluates its program on every block
                                 and adds the results up elementwise, block after block, starting from acc_init — the
                                 accumulator tile a column-blocked kernel carries through its scf.for
                                 (examples/triton-ktir/layernorm_fwd_ktir.mlir:58-75) — before the fold over the `cols`
                                 sums; the output phase stores one block after the other */
    int32_t acc_round16;      /* blocked reduction: the elementwise adds round to f16 */
    float acc_init;           /* blocked reduction: initial value of the accumulator */
} ktb_rp_phase;
typedef struct {
    ktb_vm_program prog;      /* one value per row; registers 0..n_red-1 = the reduction results */
    int32_t ready_after;      /* index of the last reduction it reads, -1 for none; entries sorted by it */
    int32_t reserved;
} ktb_rp_scalar;
typedef struct {
    ktb_vm_program prog;      /* one value per row; registers 0..n_red-1 = the reduction results */
    int64_t row_stride;       /* elements between the values of consecutive rows of an item */
    int32_t dtype;            /* KTB_F16 / KTB_F32 */
    int32_t reserved;
} ktb_rp_side;
typedef struct {
    void* arena;
    const int64_t* dev_item_offsets;   /* [n_items][n_in + 1 + n_side]: operand tiles, the output, the side results */
    int64_t n_items;
    int32_t rows_per_item, cols;
    int32_t n_in, n_red, n_scal;
    int32_t out_per_row;      /* 1: the statement stores ONE value per row (a row mean, say): `out.prog` is a program over the
                                 reduction results like a row scalar, and row_stride[n_in] is the element distance between the
                                 values of consecutive rows of an item */
    int64_t row_stride[KTB_VM_MAX_IN + 1];   /* elements; inputs then output */
    int32_t dtype[KTB_VM_MAX_IN + 1];        /* KTB_F16 / KTB_F32 */
    int64_t blk_stride[KTB_VM_MAX_IN + 1];   /* elements between the column blocks of a row (blocked phases); inputs then output */
    int32_t n_blocks;                        /* column blocks per row, 1 if no phase is blocked */
    int32_t n_side;                          /* per-row results stored beside the output tile (the Mean and Rstd vectors a
                                                layer norm keeps for its backward pass,
                                                examples/triton-ktir/layernorm_fwd_ktir.mlir:127-128): programs over the
                                                reduction results, evaluated once all reductions of the row are done; 0 when
                                                out_per_row is set */
    ktb_rp_phase red[KTB_RP_MAX_RED];
    ktb_rp_scalar scal[KTB_RP_MAX_SCAL];
    ktb_rp_phase out;                        /* op unused */
    ktb_rp_side side[KTB_RP_MAX_SIDE];
} ktb_rowprog_args;
int ktb_launch_row_program(ktb_ctx* ctx, const ktb_rowprog_args* args);

/* ---- row gather / ordered row scatter ---------------------------------------------
 * A statement moves E = n_tiles * tile_rows rows ("entries") of `cols` elements per
 * operand; entry (t, pos) of an operand lives at element offset
 *     base[t] + IDX[idx_off[t] + pos * idx_stride] * idx_mult + pos * pos_stride   (indirect)
 *     base[t] + pos * pos_stride                                                    (direct)
 * and an input with two index subscripts (X[P[p], T[t], :]) adds a second term
 * IDX2[idx2_off[t] + pos * idx2_stride] * idx2_mult.
 * Replaces MemoryOps.indirect_load / indirect_store and the per-point index
 * resolution behind them (ktir_cpu/ops/memory_ops.py:330-386, 488-576, 867-964) plus
 * the fancy-index gather/scatter of the memory simulator (ktir_cpu/memory.py:243-251,
 * 281-291): reads outside [lo, hi) give 0, writes outside are dropped, a negative
 * index sets ktb_status.negative_index. */
#define KTB_ROWS_MAX_IN 3
typedef struct {
    int32_t indirect;             /* number of index lookups in the row address: 0, 1, or (inputs only) 2 */
    int32_t dtype;                /* KTB_F16 / KTB_F32 */
    int32_t idx_dtype;            /* KTB_I32 / KTB_I64 */
    int32_t alias_dst;            /* inputs only: 1 = reads the destination row (read-modify-write) */
    const int64_t* dev_base;      /* [n_tiles] element offset of the tile's direct part */
    const int64_t* dev_idx_off;   /* [n_tiles] element offset (index units) of the tile's first index */
    int64_t idx_stride;           /* index elements between consecutive tile rows (0: one index per tile) */
    int64_t idx_mult;             /* data elements per unit of index value */
    int64_t pos_stride;           /* data elements between consecutive tile rows (direct part) */
    int64_t lo, hi;               /* allocation bounds in data elements */
    const int64_t* dev_idx2_off;  /* second lookup (indirect == 2): as dev_idx_off / idx_stride / idx_mult */
    int64_t idx2_stride;
    int64_t idx2_mult;
    int32_t idx2_dtype;           /* KTB_I32 / KTB_I64 */
    int32_t reserved;
} ktb_row_operand;

typedef struct {
    void* arena;
    int64_t n_tiles;
    int32_t tile_rows, cols;
    int32_t n_in;
    int32_t vector_ok;            /* 1: cols and every row address are multiples of 4 elements */
    ktb_row_operand in[KTB_ROWS_MAX_IN];
    ktb_row_operand out;
    ktb_vm_program program;
    int32_t* dev_rowid_scratch;   /* scatter only: ktb_scatter_scratch_bytes(n_tiles * tile_rows, dst_rows) bytes, 16-byte aligned */
    int64_t dst_row0;             /* scatter only: element offset of destination row id 0 */
    int64_t dst_rows;             /* scatter only: number of destination rows */
} ktb_rows_args;

/* out (direct) = program(inputs); inputs may be gathered.  ktdp.load through an
 * indirect access tile followed by elementwise ops and a direct ktdp.store. */
int ktb_launch_rows_program(ktb_ctx* ctx, const ktb_rows_args* args);
/* out (indirect) = program(inputs), tiles applied in order, last writer of a row
 * within a tile wins — ktdp.store through an indirect access tile, including the
 * load/modify/store-back form. */
int ktb_launch_scatter_rows(ktb_ctx* ctx, const ktb_rows_args* args);
/* Bytes of device scratch ktb_launch_scatter_rows needs for this many entries and destination rows. */
size_t ktb_scatter_scratch_bytes(int64_t entries, int64_t dst_rows);
/* ktb_launch_scatter_rows for callers that may not allocate: `dev_rowid_scratch` is ignored and
 * the scratch is a fixed KTB_SCATTER_STATIC_BYTES array inside the library, so the call makes no
 * device or host allocation.  A statement whose ktb_scatter_scratch_bytes() exceeds the array
 * is rejected with KTB_E_UNSUPPORTED.  The first call on a device looks the array's address up
 * and should come before any stream capture; all calls on a device share the array, so they
 * must not overlap in time.  No counterpart in the reference, whose allocator is a Python dict
 * (ktir_cpu/memory.py:311-345). */
#define KTB_SCATTER_STATIC_BYTES (8u << 20)
int ktb_launch_scatter_rows_static(ktb_ctx* ctx, const ktb_rows_args* args);

/* ---- generic whole-grid steps ---------------------------------------------------------
 * The op-by-op path for tile programs no fused kernel covers: one call performs one step on
 * buffers of [points][elems] in caller-provided device scratch.  Replaces the per-op
 * handlers the reference dispatches (ktir_cpu/dialects/arith_ops.py, math_ops via
 * ktir_cpu/ops/math_ops.py:27-138, linalg_ops.py:61-347, tensor_ops.py:47-359,
 * ktir_cpu/ops/memory_ops.py:723-964) with the same rounding points: float tiles compute in
 * f32 and round to the destination type per step, integer tiles wrap in their width.
 * KTB_G_RING is ktdp.inter_tile_reduce (ktir_cpu/dialects/ktdp_ops.py:1160-1240 with
 * RingReduceBackend, ktir_cpu/ops/comm_ops.py:229-345): per point the fold of its own partial with
 * its group's other partials in ring arrival order; a group of at most 8 cores runs as one
 * thread-block cluster that reads the partials out of its members' shared memory.
 * KTB_G_TABLE fills dst from a [points][elems] host-computed table — the element addresses of a tile
 * that several partitions of a distributed memory view back (MemoryOps.distributed_tile_access,
 * ktir_cpu/ops/memory_ops.py:985-1098); KTB_G_GATHER / KTB_G_SCATTER then move the data.
 * KTB_G_CONCAT joins two tiles along one axis (dst [outer][n + h][inner] = a [outer][n][inner] followed by
 * b [outer][h][inner]): the carried odd slice of a pairwise reduction level
 * (_tree_fold, ktir_cpu/dialects/linalg_ops.py:86-133). */
enum { KTB_G_LOAD = 0, KTB_G_ADDR, KTB_G_IDXADD, KTB_G_GATHER, KTB_G_CONSTV, KTB_G_FILL, KTB_G_PARAM,
       KTB_G_IOTA, KTB_G_MAP, KTB_G_EW, KTB_G_REDL, KTB_G_MATMUL, KTB_G_STORE, KTB_G_SCATTER, KTB_G_RING, KTB_G_TABLE,
       KTB_G_CONCAT };
#define KTB_G_MAXDIM 6
typedef struct {
    int32_t kind;                 /* KTB_G_* */
    int32_t op;                   /* KTB_G_EW / KTB_G_REDL: opcode (order of lower_generic.EW_OPS) */
    int32_t dt_dst, dt_a, dt_b, dt_c;   /* KTB_F16 .. KTB_I1 */
    int32_t flags;                /* bit 0: compare as integers; bit 1 (RING): combiner takes (received, accumulator);
                                     bit 2 (SCATTER): the addresses are all different, elements may be written in any order */
    int32_t ndim;                 /* KTB_G_MAP / KTB_G_IOTA: rank of `shape` */
    int64_t points, elems;        /* extent of dst (of the stored tile for STORE / SCATTER) */
    int64_t ea, eb, ec;           /* elems of the sources; 1 = one value per point, broadcast */
    void* dst;
    const void* a;
    const void* b;
    const void* c;
    void* arena;
    const int64_t* dev_base;      /* [points] element address of the tile origin (LOAD / ADDR / STORE); RING: sources per point */
    const int64_t* dev_rel;       /* [elems] element offset of each element from the origin; RING with a cluster: point of each CTA */
    const void* dev_table;        /* CONSTV: [elems] values of dt_dst; PARAM: [points] values of dt_dst; TABLE: [points][elems];
                                     RING: int64 [points][n] sources in fold order (cluster ranks with h > 1, else points) */
    int64_t lo, hi;               /* allocation bounds in elements: reads outside give 0, writes are dropped */
    int64_t shape[KTB_G_MAXDIM];  /* MAP: dst shape; IOTA: tile shape */
    int64_t strides[KTB_G_MAXDIM];/* MAP: source element stride per dst dim */
    int64_t offset;               /* MAP: source element offset; IOTA: dimension */
    int64_t outer, n, inner, h;   /* REDL: src viewed as [outer][n][inner], pairs (i, i + h), odd tail carried;
                                     RING: n = row length of dev_table, h = cores per cluster (<= 1: no cluster) */
    int64_t batch, M, N, K;       /* MATMUL */
    double fimm;                  /* FILL value for float destinations */
    int64_t iimm;                 /* FILL value for integer destinations; IDXADD: stride */
} ktb_gen_op;
int ktb_launch_generic(ktb_ctx* ctx, const ktb_gen_op* op);

/* ---- dense f16 GEMM on tensor cores -------------------------------------------------
 * C[M,N] = A[M,K] * B[K,N] + c_init, row-major operands in the arena, f32 accumulation
 * (tcgen05.mma into TMEM), C rounded once to c_dtype.  What a tiled KTIR matmul kernel
 * computes when its per-core tile loop — ktdp.load of an A and a B tile per K-step,
 * linalg.matmul into the loop-carried accumulator (ktir_cpu/ops/arith_ops.py:323-340,
 * ktir_cpu/dialects/linalg_ops.py:307-347), ktdp.store of the C tile — covers a dense
 * grid of tiles.  N multiple of 32; K, leading dimensions and offsets multiples of 8. */
typedef struct {
    void* arena;
    int64_t a_off, b_off, c_off;   /* element offsets: A and B in f16 units, C in c_dtype units */
    int32_t M, N, K;
    int32_t c_dtype;               /* KTB_F16 / KTB_F32 */
    int64_t lda, ldb, ldc;         /* elements */
    float c_init;                  /* constant initial value of the accumulator (usually 0) */
    int32_t reserved;
} ktb_gemm_args;
int ktb_launch_gemm_f16(ktb_ctx* ctx, const ktb_gemm_args* args);

/* ---- causal attention forward, paged K/V ----------------------------------------------
 * O[R, h, :] = softmax_p( scale * Q[R, h, :] . K[p, h, :] ) V[p, h, :] over the KV positions
 * p <= R + causal_delta (all positions when causal == 0), f32 scores / statistics, f16 in
 * and out, head_dim 128.  K and V live in pages of `page` rows reached through a block
 * table: page j of the walk is cache page block_table[j].  This is the loop a KTIR
 * attention kernel carries out per KV page — indirect ktdp.load of K and V
 * (ktir_cpu/ops/memory_ops.py:867-915), two linalg.matmul, mask, running max / sum and
 * rescale (examples/triton-ktir/paged_attention.mlir:183-396 of the reference).
 * m_init / l_init are the initial running max and sum the kernel carries (-inf and 1.0
 * there).  kv_group query heads share one K/V head (query head h reads K/V head
 * h / kv_group, paged_attention.mlir:163-181; 0 or 1 = one K/V head per query head).
 * All offsets and strides are in elements and must be multiples of 8. */
typedef struct {
    void* arena;
    int64_t q_off, o_off, k_off, v_off;        /* f16 element offsets of query, output, K cache, V cache */
    int64_t bt_off;                            /* element offset (bt_dtype units) of the first block-table entry */
    int32_t bt_dtype;                          /* KTB_I32 / KTB_I64 */
    int32_t seq_q, heads, head_dim;
    int32_t page, n_pages_total, num_tiles;    /* rows per page, pages in the cache, pages to walk */
    int32_t causal, causal_delta;
    int64_t q_row_stride, q_head_stride, o_row_stride, o_head_stride;
    int64_t kv_page_stride, kv_row_stride, kv_head_stride;
    float scale, m_init, l_init;
    int32_t kv_group;                          /* query heads per K/V head */
} ktb_attn_args;
int ktb_launch_attention_fwd(ktb_ctx* ctx, const ktb_attn_args* args);

#ifdef __cplusplus
}
#endif
#endif /* KTIR_B200_H */
