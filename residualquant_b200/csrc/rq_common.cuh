// Shared device helpers for the packed-KV kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/rq_b200.h"

namespace rq {

constexpr unsigned kFullMask = 0xffffffffu;

// ---- FP8 e4m3 <-> float (exact decode; RNE + saturate-to-finite encode) -------------------------------
__device__ __forceinline__ uint8_t fp8_encode(float v) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float fp8_decode(uint8_t b) {
    const __half_raw raw = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
    return __half2float(__half(raw));
}
// Two FP8 bytes (low 16 bits of `pair`) -> half2, one hardware conversion.
__device__ __forceinline__ __half2 fp8x2_to_half2(uint32_t pair) {
    const __half2_raw raw = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(pair & 0xffffu), __NV_E4M3);
    return __half2(raw);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits) { return __uint_as_float(bits << 16); }

// ---- programmatic dependent launch ---------------------------------------------------------------------
// launch_dependents: the next kernel of the stream (if it was launched as a programmatic dependent) may be scheduled
// once every CTA of this grid has said so or exited.  wait: returns when the previous kernel of the stream has
// completed and its writes are visible.  Both are no-ops in a kernel launched with plain stream order.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- Walsh-Hadamard helpers ---------------------------------------------------------------------------
// In-register butterflies with strides 1, 2, ..., N/2 over x[0..N), (a, b) -> (a + b, a - b).
template <int N>
__device__ __forceinline__ void butterflies_in_lane(float (&x)[N]) {
#pragma unroll
    for (int h = 1; h < N; h <<= 1) {
#pragma unroll
        for (int i = 0; i < N; ++i) {
            if ((i & h) == 0) {
                const float a = x[i], b = x[i + h];
                x[i] = __fadd_rn(a, b);
                x[i + h] = __fsub_rn(a, b);
            }
        }
    }
}

// One butterfly stage between lanes `lane` and `lane ^ mask`; the lane whose `bit` is set holds b.
template <int N>
__device__ __forceinline__ void butterfly_across_lanes(float (&x)[N], int mask, bool upper) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float other = __shfl_xor_sync(kFullMask, x[i], mask);
        x[i] = __fmaf_rn(upper ? -1.f : 1.f, x[i], other);  // other - x or x + other, one rounding either way
    }
}

// Row i of the 12x12 Paley matrix as a bit mask: bit j set when P[i][j] == -1
// (scripts/calibration/rotation_math.py:7-15: first row and column +1, P[i+1][j+1] = -1 on the diagonal,
// +1 when (i - j) mod 11 is a quadratic residue, else -1).
__device__ __forceinline__ uint32_t paley12_negative_mask(int i) {
    if (i == 0) return 0u;
    uint32_t mask = 0u;
#pragma unroll
    for (int j = 1; j < 12; ++j) {
        const int d = ((i - 1) - (j - 1) + 11) % 11;
        // quadratic residues mod 11: 1, 3, 4, 5, 9
        const bool residue = d == 1 || d == 3 || d == 4 || d == 5 || d == 9;
        const bool negative = (i == j) || !residue;
        mask |= (negative ? 1u : 0u) << j;
    }
    return mask;
}

}  // namespace rq
