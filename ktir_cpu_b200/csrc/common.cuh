// Shared internals of libktir_b200: context layout, error helpers, status word.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/ktir_b200.h"

#define KTB_NUM_EVENTS 64
#define KTB_MAX_DEVICES 64            // power of two; per-device launch state is indexed by device & (this - 1)
#define KTB_FLUSH_BYTES (256u << 20)   // > 126 MB L2
#define KTB_NUM_FENCES 64             // rotating events that order the copy lanes against the launch stream

struct ktb_submitter;          // transfer.cu: the thread that issues queued pipeline jobs

struct ktb_ctx {
    int device;
    int sm_count;
    cudaStream_t stream;
    bool own_stream;
    cudaEvent_t events[KTB_NUM_EVENTS];
    ktb_status* dev_status;     // device copy of the status word
    void* flush_buf;            // lazily allocated L2 flush scratch
    int64_t launches;
    int64_t capture_base;       // launch count when a graph capture began
    cudaStream_t lane[2];       // upload lane, read-back lane (created on first use)
    cudaEvent_t fences[KTB_NUM_FENCES];
    unsigned next_fence;
    bool lanes_ok, lanes_used;
    ktb_submitter* submitter;   // created by the first ktb_submit_pipeline
    char err[512];
};

void ktb_transfer_destroy(ktb_ctx* ctx);   // transfer.cu
int ktb_transfer_sync(ktb_ctx* ctx);
int ktb_transfer_drain(ktb_ctx* ctx, uint64_t seq);

static inline int ktb_fail(ktb_ctx* ctx, int code, const char* what, const char* detail) {
    if (ctx) snprintf(ctx->err, sizeof(ctx->err), "%s: %s", what, detail ? detail : "");
    return code;
}

#define KTB_CUDA(ctx, call)                                                        \
    do {                                                                           \
        cudaError_t e__ = (call);                                                  \
        if (e__ != cudaSuccess)                                                    \
            return ktb_fail((ctx), KTB_E_CUDA, #call, cudaGetErrorString(e__));   \
    } while (0)

#define KTB_CHECK_LAUNCH(ctx, name)                                                \
    do {                                                                           \
        cudaError_t e__ = cudaGetLastError();                                      \
        if (e__ != cudaSuccess)                                                    \
            return ktb_fail((ctx), KTB_E_CUDA, name, cudaGetErrorString(e__));    \
        (ctx)->launches++;                                                         \
    } while (0)

static __device__ __forceinline__ float ktb_round16(float x) {
    return __half2float(__float2half_rn(x));
}
