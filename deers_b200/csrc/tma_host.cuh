// Host-side construction of TMA tensor maps for [B,H,T,D] f16 tensors.
#pragma once
#include "common.cuh"

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

// Tensor map over a [B,H,T,D] f16 tensor (strides in elements, inner stride 1),
// dimensions ordered {D, T, H, B}, box {64 columns, box_rows rows, 1, 1}, 128-byte
// swizzle, out-of-range rows read as zero.  Returns DEERS_ERR_LAYOUT when the
// driver rejects the strides or the alignment.
static inline int make_tmap_bhtd_f16(deers_ctx* ctx, CUtensorMap* out, const void* base, int B, int H, int T,
                                     int D, const int64_t* strides, int box_rows) {
    if (!ctx->encode_tiled) {
        snprintf(ctx->last_error, sizeof(ctx->last_error), "cuTensorMapEncodeTiled not available");
        return DEERS_ERR_CUDA;
    }
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
    // A dimension of extent 1 never advances: give it any legal stride.
    const int64_t st_t = T > 1 ? strides[2] : D;
    const int64_t st_h = H > 1 ? strides[1] : st_t * T;
    const int64_t st_b = B > 1 ? strides[0] : (st_h * H > 0 ? st_h * H : st_t * T);
    const cuuint64_t gstr[3] = {(cuuint64_t)st_t * 2, (cuuint64_t)st_h * 2, (cuuint64_t)st_b * 2};
    const cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1u, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = ((PFN_encodeTiled)ctx->encode_tiled)(
        out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, gstr, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(ctx->last_error, sizeof(ctx->last_error), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return DEERS_ERR_LAYOUT;
    }
    return DEERS_OK;
}
