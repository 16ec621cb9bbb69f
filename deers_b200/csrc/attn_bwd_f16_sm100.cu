#include "common.cuh"
size_t attn_bwd_f16_dqacc_bytes(const deers_attn_desc* d) {
    return (size_t)d->B * d->H * (size_t)((d->T + 127) / 128 * 128) * d->D * sizeof(float);
}
int launch_attn_bwd_f16(deers_ctx*, const deers_attn_desc*, const void*, const void*, const void*, const void*,
                        const float*, const void*, void*, void*, void*, float*, float*) {
    return DEERS_ERR_UNSUPPORTED;
}
