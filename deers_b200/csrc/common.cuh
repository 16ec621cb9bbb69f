// Shared internals of the deers_b200 library: the context object, status helpers
// and the launch prototypes each kernel file exports to the C-ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/deers_b200.h"

struct deers_ctx {
    int device;
    cudaStream_t stream;
    bool owns_stream;
    int sm_count;
    // Error word the kernels write when a bounded wait gives up.  Pinned, mapped
    // host memory: the kernels use dev_err, the host reads host_err after a sync.
    unsigned int* host_err;
    unsigned int* dev_err;
    uint64_t launches;
    char last_error[256];
    // cuTensorMapEncodeTiled, fetched through the runtime so that the library
    // does not link against the driver.
    void* encode_tiled;
};

#define DEERS_CUDA_TRY(ctx, expr)                                                            \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess) {                                                              \
            snprintf((ctx)->last_error, sizeof((ctx)->last_error), "%s: %s", #expr,           \
                     cudaGetErrorString(_e));                                                 \
            return DEERS_ERR_CUDA;                                                            \
        }                                                                                     \
    } while (0)

// Device-side error codes (upper byte: which kernel, lower bits: which wait).
enum {
    DEERS_KERR_FWD_F16 = 0x100,
    DEERS_KERR_BWD_F16 = 0x200,
    DEERS_KERR_SELFTEST = 0x300,
};

// f32 FFMA path (attn_f32.cu)
int launch_attn_fwd_f32(deers_ctx* ctx, const deers_attn_desc* d, const float* q, const float* k,
                        const float* v, float* o, float* lse);
int launch_attn_bwd_f32(deers_ctx* ctx, const deers_attn_desc* d, const float* q, const float* k,
                        const float* v, const float* o, const float* lse, const float* d_o, float* dq,
                        float* dk, float* dv, float* delta);

// f16 tcgen05 path (attn_f16_sm100.cu)
int launch_attn_fwd_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k,
                        const void* v, void* o, float* lse);
int launch_attn_bwd_f16(deers_ctx* ctx, const deers_attn_desc* d, const void* q, const void* k,
                        const void* v, const void* o, const float* lse, const void* d_o, void* dq,
                        void* dk, void* dv, void* workspace);
size_t attn_bwd_f16_workspace_bytes(const deers_attn_desc* d);
int run_selftest_umma(deers_ctx* ctx, float* max_abs_err);
