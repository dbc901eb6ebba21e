// Context, memory, transfers, events — the part of the C ABI that replaces the
// reference's simulated memory hierarchy set-up and argument upload/read-back
// (ktir_cpu/interpreter.py:95-120,156-194).
#include "common.cuh"

// Streams `n` 16-byte words through the cache; the result is stored only if it is non-zero
// (the buffer holds zeros), which keeps the loads alive without dirtying a line.
__global__ void __launch_bounds__(256) ktb_flush_read_kernel(const uint4* __restrict__ src, size_t n, unsigned* sink) {
    unsigned acc = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        acc |= v.x | v.y | v.z | v.w;
    }
    if (acc) *sink = acc;
}

extern "C" {

int ktb_init(int device, ktb_ctx** out) {
    if (!out) return KTB_E_ARG;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || device < 0 || device >= n) return KTB_E_CUDA;
    ktb_ctx* ctx = new ktb_ctx();
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    if (cudaSetDevice(device) != cudaSuccess) { delete ctx; return KTB_E_CUDA; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete ctx; return KTB_E_CUDA; }
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return KTB_E_CUDA;
    }
    ctx->own_stream = true;
    for (int i = 0; i < KTB_NUM_EVENTS; ++i) cudaEventCreate(&ctx->events[i]);
    if (cudaMalloc(&ctx->dev_status, sizeof(ktb_status)) != cudaSuccess) { delete ctx; return KTB_E_CUDA; }
    cudaMemset(ctx->dev_status, 0, sizeof(ktb_status));
    *out = ctx;
    return KTB_OK;
}

int ktb_destroy(ktb_ctx* ctx) {
    if (!ctx) return KTB_E_ARG;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    ktb_transfer_destroy(ctx);
    for (int i = 0; i < KTB_NUM_EVENTS; ++i) cudaEventDestroy(ctx->events[i]);
    if (ctx->flush_buf) cudaFree(ctx->flush_buf);
    cudaFree(ctx->dev_status);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return KTB_OK;
}

const char* ktb_last_error(ktb_ctx* ctx) { return ctx ? ctx->err : "null context"; }

int ktb_set_stream(ktb_ctx* ctx, uint64_t cuda_stream) {
    if (!ctx) return KTB_E_ARG;
    if (ctx->own_stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
    }
    ctx->stream = (cudaStream_t)cuda_stream;
    ctx->own_stream = false;
    return KTB_OK;
}

int ktb_alloc(ktb_ctx* ctx, size_t bytes, void** dev_ptr) {
    if (!ctx || !dev_ptr) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaSetDevice(ctx->device));
    KTB_CUDA(ctx, cudaMalloc(dev_ptr, bytes ? bytes : 1));
    return KTB_OK;
}

int ktb_free(ktb_ctx* ctx, void* dev_ptr) {
    if (!ctx) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    KTB_CUDA(ctx, cudaFree(dev_ptr));
    return KTB_OK;
}

int ktb_alloc_host(ktb_ctx* ctx, size_t bytes, void** host_ptr) {
    if (!ctx || !host_ptr) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaMallocHost(host_ptr, bytes ? bytes : 1));
    return KTB_OK;
}

int ktb_free_host(ktb_ctx* ctx, void* host_ptr) {
    if (!ctx) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaFreeHost(host_ptr));
    return KTB_OK;
}

int ktb_memset(ktb_ctx* ctx, void* dev_ptr, int byte_value, size_t bytes) {
    if (!ctx) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaMemsetAsync(dev_ptr, byte_value, bytes, ctx->stream));
    return KTB_OK;
}

int ktb_h2d(ktb_ctx* ctx, void* dev_dst, const void* host_src, size_t bytes) {
    if (!ctx) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return KTB_OK;
}

int ktb_d2h(ktb_ctx* ctx, void* host_dst, const void* dev_src, size_t bytes) {
    if (!ctx) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return KTB_OK;
}

int ktb_d2d(ktb_ctx* ctx, void* dev_dst, const void* dev_src, size_t bytes) {
    if (!ctx) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaMemcpyAsync(dev_dst, dev_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return KTB_OK;
}

int ktb_sync(ktb_ctx* ctx, ktb_status* status_out) {
    if (!ctx) return KTB_E_ARG;
    if (int rc = ktb_transfer_drain(ctx, 0)) return rc;   // jobs still queued for the submission thread
    ktb_status st;
    KTB_CUDA(ctx, cudaMemcpyAsync(&st, ctx->dev_status, sizeof(st), cudaMemcpyDeviceToHost, ctx->stream));
    KTB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (int rc = ktb_transfer_sync(ctx)) return rc;      // the copy lanes, when a pipelined call used them
    if (status_out) *status_out = st;
    if (st.negative_index || st.wait_timeout) {
        KTB_CUDA(ctx, cudaMemsetAsync(ctx->dev_status, 0, sizeof(st), ctx->stream));
        if (st.negative_index) {
            char buf[64];
            snprintf(buf, sizeof(buf), "%d is negative", st.bad_index_value);
            return ktb_fail(ctx, KTB_E_DEVICE_STATUS, "indirect index", buf);
        }
        return ktb_fail(ctx, KTB_E_DEVICE_STATUS, "device wait", "bounded wait ran out");
    }
    return KTB_OK;
}

int ktb_event_record(ktb_ctx* ctx, int slot) {
    if (!ctx || slot < 0 || slot >= KTB_NUM_EVENTS) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaEventRecord(ctx->events[slot], ctx->stream));
    return KTB_OK;
}

int ktb_event_record_on(ktb_ctx* ctx, int slot, int lane) {
    if (!ctx || slot < 0 || slot >= KTB_NUM_EVENTS || lane < 0 || lane > 2) return KTB_E_ARG;
    if (lane > 0 && !ctx->lanes_ok) return ktb_fail(ctx, KTB_E_ARG, "ktb_event_record_on", "copy lanes not in use");
    KTB_CUDA(ctx, cudaEventRecord(ctx->events[slot], lane == 0 ? ctx->stream : ctx->lane[lane - 1]));
    return KTB_OK;
}

int ktb_event_sync(ktb_ctx* ctx, int slot) {
    if (!ctx || slot < 0 || slot >= KTB_NUM_EVENTS) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaEventSynchronize(ctx->events[slot]));
    return KTB_OK;
}

int ktb_status_snapshot(ktb_ctx* ctx, ktb_status* host_pinned) {
    if (!ctx || !host_pinned) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaMemcpyAsync(host_pinned, ctx->dev_status, sizeof(ktb_status), cudaMemcpyDeviceToHost, ctx->stream));
    KTB_CUDA(ctx, cudaMemsetAsync(ctx->dev_status, 0, sizeof(ktb_status), ctx->stream));
    return KTB_OK;
}

int ktb_event_elapsed_ms(ktb_ctx* ctx, int a, int b, float* ms_out) {
    if (!ctx || !ms_out || a < 0 || b < 0 || a >= KTB_NUM_EVENTS || b >= KTB_NUM_EVENTS) return KTB_E_ARG;
    KTB_CUDA(ctx, cudaEventSynchronize(ctx->events[b]));
    KTB_CUDA(ctx, cudaEventElapsedTime(ms_out, ctx->events[a], ctx->events[b]));
    return KTB_OK;
}

int ktb_flush_l2(ktb_ctx* ctx) {
    if (!ctx) return KTB_E_ARG;
    // first half is written (evicts everything cached), second half is then read, which pushes the
    // dirty lines of the write back to HBM now instead of during the next timed launch
    if (!ctx->flush_buf) {
        KTB_CUDA(ctx, cudaMalloc(&ctx->flush_buf, 2 * (size_t)KTB_FLUSH_BYTES));
        KTB_CUDA(ctx, cudaMemsetAsync(ctx->flush_buf, 0, 2 * (size_t)KTB_FLUSH_BYTES, ctx->stream));
    }
    KTB_CUDA(ctx, cudaMemsetAsync(ctx->flush_buf, 0, KTB_FLUSH_BYTES, ctx->stream));
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<char*>(ctx->flush_buf) + KTB_FLUSH_BYTES);
    ktb_flush_read_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(src, KTB_FLUSH_BYTES / sizeof(uint4),
                                                                    reinterpret_cast<unsigned*>(ctx->flush_buf));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ktb_fail(ctx, KTB_E_CUDA, "ktb_flush_read_kernel", cudaGetErrorString(e));
    return KTB_OK;
}

int64_t ktb_launch_count(ktb_ctx* ctx) { return ctx ? ctx->launches : -1; }

// ---- replaying a launch sequence as a CUDA graph -------------------------------------------
struct ktb_graph {
    cudaGraphExec_t exec;
    int64_t launches;           // kernel launches the sequence contains
};

int ktb_graph_begin(ktb_ctx* ctx) {
    if (!ctx) return KTB_E_ARG;
    ctx->capture_base = ctx->launches;
    KTB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    return KTB_OK;
}

int ktb_graph_end(ktb_ctx* ctx, void** graph_out) {
    if (!ctx || !graph_out) return KTB_E_ARG;
    *graph_out = nullptr;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    const int64_t n = ctx->launches - ctx->capture_base;
    ctx->launches = ctx->capture_base;            // captured launches have not run
    if (e != cudaSuccess || !g) {
        cudaGetLastError();
        return ktb_fail(ctx, KTB_E_CUDA, "cudaStreamEndCapture", cudaGetErrorString(e));
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return ktb_fail(ctx, KTB_E_CUDA, "cudaGraphInstantiate", cudaGetErrorString(e));
    ktb_graph* out = new ktb_graph{exec, n};
    *graph_out = out;
    return KTB_OK;
}

int ktb_graph_launch(ktb_ctx* ctx, void* graph) {
    if (!ctx || !graph) return KTB_E_ARG;
    ktb_graph* g = static_cast<ktb_graph*>(graph);
    KTB_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
    ctx->launches += g->launches;
    return KTB_OK;
}

int ktb_graph_destroy(ktb_ctx* ctx, void* graph) {
    if (!graph) return KTB_OK;
    ktb_graph* g = static_cast<ktb_graph*>(graph);
    cudaGraphExecDestroy(g->exec);
    delete g;
    return KTB_OK;
}

}  // extern "C"
