// Variant selection for the packed paged decode attention (the kernels live in rq_attention_impl.cuh, instantiated
// once per head dimension).  Mirrors the reference's registry lookup (dispatch/kernel_registry.h:48-75): an
// unknown key is an error, never a slow path.
#include "rq_kernels.h"

namespace rq {

cudaError_t launch_attention_d128(const AttentionVariant& v, const AttentionParams& p, cudaStream_t stream);
cudaError_t launch_attention_d96(const AttentionVariant& v, const AttentionParams& p, cudaStream_t stream);

bool attention_variant_available(const AttentionVariant& v) {
    if (v.head_dim != 128 && v.head_dim != 96) return false;
    if (v.page_tokens != 16 && v.page_tokens != 32) return false;
    if (v.adjacent) return true;  // record types are checked by the caller (INT4 g32, INT2 g16/g32; at most 4 records)
    const int ab = v.anchor_bits, ag = v.anchor_group, rb = v.residual_bits, rg = v.residual_group;
    if (ab == 4 && ag == 32) return rb == 0 || (rb == 2 && (rg == 16 || rg == 32)) || (rb == 4 && rg == 32);
    if (ab == 2 && ag == 32) return rb == 0 || (rb == 2 && rg == 32) || (rb == 4 && rg == 32);
    if (ab == 2 && ag == 16) return rb == 0 || (rb == 2 && rg == 16) || (rb == 4 && rg == 32);
    return false;
}

cudaError_t launch_attention(const AttentionVariant& v, const AttentionParams& p, cudaStream_t stream) {
    if (!attention_variant_available(v)) return cudaErrorInvalidDeviceFunction;
    return v.head_dim == 128 ? launch_attention_d128(v, p, stream) : launch_attention_d96(v, p, stream);
}

}  // namespace rq
