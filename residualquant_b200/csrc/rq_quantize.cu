// KV-write quantizer: rotate (fused signed Walsh-Hadamard), quantize the anchor record, then the
// coefficient-scaled residual records against the reconstructed anchor, and bit-pack everything into the
// paged uint8 cache.  One launch per call.
//
// Replaces quantize_kernel / quantize_token / commit_record of the reference
// (plugins/residual_quantization/csrc/quantize/kernel.cuh:33-228, 236-355) and its TF32-MMA rotation
// (quantize/rotation.cuh:25-150).  Every operation that feeds a rounding decision is an explicit
// round-to-nearest binary32 intrinsic in a fixed order, so a CPU restatement reproduces the packed bytes
// bit for bit.  This file must be compiled with -fmad=false and without --use_fast_math.
//
// Work split: a row = one (token, head, plane); 8 lanes own a row, each lane 16 consecutive channels, so a
// warp owns 4 consecutive tokens of one head and a 128-thread CTA 16 consecutive tokens (one vLLM block when
// the slots are contiguous).  Grid = (ceil(tokens/16), heads, 2 planes).
#include <atomic>
#include <type_traits>

#include "rq_common.cuh"
#include "rq_kernels.h"

namespace rq {
namespace {

// P[i][j] == -1  <=>  bit j of kPaleyRow[i]  <=>  bit i of kPaleyCol[j]   (12x12 Paley matrix)
__constant__ uint32_t kPaleyRow[16] = {0x0, 0x476, 0x8ec, 0x1da, 0x3b4, 0x768, 0xed0, 0xda2,
                                       0xb46, 0x68e, 0xd1c, 0xa3a, 0, 0, 0, 0};
__constant__ uint32_t kPaleyCol[16] = {0x0, 0xb8a, 0x716, 0xe2c, 0xc5a, 0x8b6, 0x16e, 0x2dc,
                                       0x5b8, 0xb70, 0x6e2, 0xdc4, 0, 0, 0, 0};

// The same masks for code whose indices are compile-time constants (the unrolled 12-point stage of a row in shared memory).
__host__ __device__ constexpr uint32_t paley_row_mask(int i) {
    constexpr uint32_t rows[12] = {0x0, 0x476, 0x8ec, 0x1da, 0x3b4, 0x768, 0xed0, 0xda2, 0xb46, 0x68e, 0xd1c, 0xa3a};
    return rows[i];
}
__host__ __device__ constexpr uint32_t paley_col_mask(int j) {
    constexpr uint32_t cols[12] = {0x0, 0xb8a, 0x716, 0xe2c, 0xc5a, 0x8b6, 0x16e, 0x2dc, 0x5b8, 0xb70, 0x6e2, 0xdc4};
    return cols[j];
}
// head_dim 96: the 12-point stage runs through shared memory, one scratch row of 96 floats per row of the warp.  The
// stride keeps the four rows of a warp on different banks when 32 lanes read (row, position) columns.
constexpr int kPaleyStride = 104;
constexpr int kPaleyWarpFloats = 4 * kPaleyStride;

// ---- packed binary32 pairs ------------------------------------------------------------------------------------------
// sm_100 issues add / mul / fma on PAIRS of binary32 values (add.f32x2, mul.f32x2, fma.f32x2): two IEEE operations with
// round-to-nearest-even each -- the same results as two scalar instructions -- in one issue slot.  A lane's 16 channels
// are paired as (channel i, channel i + 8), i = 0..7; every helper below keeps that pairing so that values stay in
// the same register pairs from one operation to the next.
__device__ __forceinline__ float2 pair_of(const float (&values)[16], int i) { return make_float2(values[i], values[i + 8]); }
__device__ __forceinline__ void unpair(float (&values)[16], int i, float2 pair) {
    values[i] = pair.x;
    values[i + 8] = pair.y;
}
#define RQ_PAIR(array, index) pair_of(array, index)
#define RQ_UNPAIR(array, index, pair) unpair(array, index, pair)
// Written as PTX with an explicit rounding mode on every instruction: an instruction that names its rounding is never
// merged with a neighbour into a fused multiply-add, which is what keeps the packed bytes reproducible.
__device__ __forceinline__ unsigned long long pack2(float2 v) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(v.x), "f"(v.y));
    return r;
}
__device__ __forceinline__ float2 unpack2(unsigned long long r) {
    float2 v;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(v.x), "=f"(v.y) : "l"(r));
    return v;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long c;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(c) : "l"(pack2(a)), "l"(pack2(b)));
    return unpack2(c);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long c;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(c) : "l"(pack2(a)), "l"(pack2(b)));
    return unpack2(c);
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack2(a)), "l"(pack2(b)), "l"(pack2(c)));
    return unpack2(d);
}
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return fma2(b, make_float2(-1.f, -1.f), a); }  // RN(a - b)
__device__ __forceinline__ float2 add2_round_up(float2 a, float2 b) {
    unsigned long long c;
    asm("add.rp.f32x2 %0, %1, %2;" : "=l"(c) : "l"(pack2(a)), "l"(pack2(b)));
    return unpack2(c);
}

// Butterflies with strides 1, 2, 4, 8 over the lane's 16 values, in that order, (a, b) -> (a + b, a - b): the first three
// stages act on both halves alike (packed), the last one crosses the halves.
__device__ __forceinline__ void butterflies_16(float (&x)[16], bool with_stride_8) {
#pragma unroll
    for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((i & h) == 0) {
                const float2 a = RQ_PAIR(x, i), b = RQ_PAIR(x, i + h);
                const float2 sum = add2(a, b), difference = sub2(a, b);
                RQ_UNPAIR(x, i, sum);
                RQ_UNPAIR(x, i + h, difference);
            }
        }
    }
    if (with_stride_8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a = x[i], b = x[i + 8];
            x[i] = __fadd_rn(a, b);
            x[i + 8] = __fsub_rn(a, b);
        }
    }
}

// One butterfly stage between lanes `lane` and `lane ^ mask`: x <- other + x, or other - x in the lane that holds b.
__device__ __forceinline__ void butterfly_across_lanes_16(float (&x)[16], int mask, bool upper) {
    const float sign = upper ? -1.f : 1.f;
    const float2 signs = make_float2(sign, sign);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 other = make_float2(__shfl_xor_sync(kFullMask, x[i], mask), __shfl_xor_sync(kFullMask, x[i + 8], mask));
        const float2 v = fma2(signs, RQ_PAIR(x, i), other);  // one rounding either way
        RQ_UNPAIR(x, i, v);
    }
}

// Forward: y = ((sign * x) H) * rscale.  Inverse: x = ((y H^T) * rscale) * sign.
// `j` is the lane's slice (channels 16j .. 16j+15) inside its 8-lane row group.
// `scratch`: head_dim 96 only, kPaleyWarpFloats floats of shared memory owned by the calling warp.
template <int D, bool INVERSE>
__device__ __forceinline__ void rotate_row(float (&x)[16], int j, uint32_t sign16, float rscale, float* scratch) {
    // forward: the sign diagonal has already been applied when the row was loaded
    if (D == 128) {
        butterflies_16(x, true);
        butterfly_across_lanes_16(x, 1, (j & 1) != 0);
        butterfly_across_lanes_16(x, 2, (j & 2) != 0);
        butterfly_across_lanes_16(x, 4, (j & 4) != 0);
    } else {
        // Sylvester-8 inside each block of 8 channels (two blocks per lane) ...
        butterflies_16(x, false);
        // ... then the 12-point Paley transform across the row's 12 blocks: out[a'] = sum_a s(a, a') t[a], a = 0..11, added
        // in that order.  The warp's four rows go to shared memory; lane (row, b) then owns position b of every block of
        // its row -- one column of 12 values -- and forms the 12 outputs from registers with compile-time signs: 12 loads
        // and 132 additions per lane and record instead of 96 shuffles and 192 additions with run-time signs.
        const int lane = threadIdx.x & 31;
        float* row = scratch + (lane >> 3) * kPaleyStride;
        __syncwarp();  // the previous record's readers are done with the scratch rows
        if (j < 6) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<float4*>(row + 16 * j + 4 * i) = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
        }
        __syncwarp();
        float t[12], out[12];
#pragma unroll
        for (int a = 0; a < 12; ++a) t[a] = row[8 * a + j];   // j = lane & 7 is the position inside a block here
#pragma unroll
        for (int to = 0; to < 12; ++to) {
            const uint32_t mask = INVERSE ? paley_row_mask(to) : paley_col_mask(to);
            out[to] = (mask & 1u) ? -t[0] : t[0];
#pragma unroll
            for (int a = 1; a < 12; ++a) out[to] = ((mask >> a) & 1u) ? __fsub_rn(out[to], t[a]) : __fadd_rn(out[to], t[a]);
        }
#pragma unroll
        for (int to = 0; to < 12; ++to) row[8 * to + j] = out[to];   // only this lane reads or writes its column
        __syncwarp();
        // lanes 6 and 7 of a row group own no channels: keep them at zero so that row sums ignore them
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = j < 6 ? *reinterpret_cast<const float4*>(row + 16 * j + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
        }
    }
    const float2 rscale2 = make_float2(rscale, rscale);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 v = mul2(RQ_PAIR(x, i), rscale2);
        RQ_UNPAIR(x, i, v);
    }
    if (INVERSE) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if ((sign16 >> i) & 1u) x[i] = -x[i];
    }
}

// sum over the row of a[c]*b[c]: 16 sequential (product rounded, then added) terms per lane, then the
// lanes combine as ((s0+s1)+(s2+s3)) + ((s4+s5)+(s6+s7)).  Scalar on purpose: a packed multiply feeding a packed add
// was observed to come out as one fused multiply-add (a single rounding), which no longer is the stated arithmetic.
__device__ __forceinline__ float row_dot(const float (&a)[16], const float (&b)[16]) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc = __fadd_rn(acc, __fmul_rn(a[i], b[i]));
    acc = __fadd_rn(acc, __shfl_xor_sync(kFullMask, acc, 1));
    acc = __fadd_rn(acc, __shfl_xor_sync(kFullMask, acc, 2));
    acc = __fadd_rn(acc, __shfl_xor_sync(kFullMask, acc, 4));
    return acc;
}

// A quantized 16-channel slice.  magic[i] = bit pattern of the float 2^23 + code[i], i.e. 0x4B000000 + code[i]:
// the form the codes come out of the rounding step in, cheap to pack and to turn back into a float.
struct GroupCode {
    uint32_t magic[16];
    uint8_t scale8, offset8;
};
constexpr uint32_t kMagicBits = 0x4B000000u;  // 8388608.0f
__device__ __forceinline__ float code_value(uint32_t magic) { return __fsub_rn(__uint_as_float(magic), 8388608.f); }

// sum_i magic[i] << (BITS * i) (mod 2^32) carries this constant on top of the packed codes.
template <int BITS, int COUNT>
__host__ __device__ constexpr uint32_t packed_magic_bias() {
    uint32_t bias = 0;
    for (int i = 0; i < COUNT; ++i) bias += kMagicBits << (BITS * i);
    return bias;
}
// COUNT codes of BITS bits each, code i at bit BITS*i: one shift-add per code.
template <int BITS, int COUNT>
__device__ __forceinline__ uint32_t pack_codes(const uint32_t* magic) {
    uint32_t word = 0;
#pragma unroll
    for (int i = COUNT - 1; i >= 0; --i) word = (word << BITS) + magic[i];
    constexpr uint32_t kBias = packed_magic_bias<BITS, COUNT>();
    return word - kBias;
}

// Asymmetric group quantizer (reference: quantize/kernel.cuh:111-158; scripts/calibration/quantization.py:40-53).
template <int BITS>
__device__ __forceinline__ GroupCode group_quantize(const float (&z)[16], int group) {
    GroupCode out;
    float low = z[0], high = z[0];
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        low = fminf(low, z[i]);
        high = fmaxf(high, z[i]);
    }
    if (group == 32) {
        low = fminf(low, __shfl_xor_sync(kFullMask, low, 1));
        high = fmaxf(high, __shfl_xor_sync(kFullMask, high, 1));
    }
    constexpr float kLevels = BITS == 2 ? 3.f : 15.f;
    const float center = __fmul_rn(__fadd_rn(low, high), 0.5f);
    const float width = __fsub_rn(high, low);
    const float radius = BITS == 2 ? __fmul_rn(__fmul_rn(width, 0.9f), 0.5f) : __fmul_rn(width, 0.5f);
    // "+ 0.0f" turns a -0.0 lower bound into +0.0 so the stored byte never depends on which signed zero won a min/max.
    out.offset8 = fp8_encode(__fadd_rn(__fsub_rn(center, radius), 0.0f));
    out.scale8 = fp8_encode(__fdiv_rn(__fmul_rn(2.f, radius), kLevels));
    const float offset = fp8_decode(out.offset8), scale = fp8_decode(out.scale8);
    // n = (z - offset) / scale, correctly rounded, without a division per channel: with r = RN(1/scale),
    // q0 = RN(d*r), e = d - q0*scale (exact in one fma), n = RN(q0 + e*r) is the IEEE quotient (the divisor has a
    // 4-bit significand; checked against exact rational arithmetic for every FP8 scale).
    // code = floor(n) + (n - floor(n) > 0.5)  ==  ceil(n - 0.5): a half rounds down, n - 0.5 is exact for n >= 0.5.
    // The clamp to [0, levels] commutes with the ceiling (integer bounds), so it is done first, in floating point;
    // adding 2^23 rounding upwards then leaves ceil(t) in the low significand bits.  A zero scale gives r = 0,
    // n = 0 and code 0, as the reference stores; a NaN loses the first max() and also becomes code 0.
    const float r = scale > 0.f ? __frcp_rn(scale) : 0.f;
    const float2 offset2 = make_float2(offset, offset), minus_scale = make_float2(-scale, -scale);
    const float2 r2 = make_float2(r, r), minus_half = make_float2(-0.5f, -0.5f), magic = make_float2(8388608.f, 8388608.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        // z - offset as a fused multiply-add with multiplier -1: z may itself be the product that ended a rotation, and a
        // plain packed add behind a packed multiply is liable to be merged with it into one rounding
        const float2 d = sub2(RQ_PAIR(z, i), offset2);
        const float2 q0 = mul2(d, r2);
        const float2 e = fma2(q0, minus_scale, d);            // d - q0 * scale, exact
        const float2 n = fma2(e, r2, q0);
        float2 t = add2(n, minus_half);
        t.x = fminf(fmaxf(t.x, 0.f), kLevels);
        t.y = fminf(fmaxf(t.y, 0.f), kLevels);
        const float2 rounded = add2_round_up(t, magic);
        out.magic[i] = __float_as_uint(rounded.x);
        out.magic[i + 8] = __float_as_uint(rounded.y);
    }
    return out;
}

// bf16( code * bf16(scale) + bf16(offset) ) with a single rounding (reference: kernel.cuh:161-186).
__device__ __forceinline__ float restore_bf16(uint32_t magic, float scale, float offset) {
    return __bfloat162float(__hfma(__float2bfloat16_rn(code_value(magic)),
                                   __float2bfloat16_rn(scale), __float2bfloat16_rn(offset)));
}
__device__ __forceinline__ float bf16_add(float a, float b) {
    return __bfloat162float(__hadd(__float2bfloat16_rn(a), __float2bfloat16_rn(b)));
}
__device__ __forceinline__ float bf16_round(float a) { return __bfloat162float(__float2bfloat16_rn(a)); }

// What the kernel knows at compile time about the group's records.  The general kernel reads everything from its
// parameters; the headline schedule (three INT2 residual loops predicted from an INT4 g32 anchor in the last loop, least
// squares coefficient, kernel chain) is also compiled with these values as constants, which unrolls the record loop
// and drops every other chain's code.  Same arithmetic, same packed bytes.
struct AnySchedule {
    static constexpr bool kFixed = false;
};
template <int RESIDUAL_GROUP>
struct Anchor2224 {
    static constexpr bool kFixed = true;
    static constexpr int kRecords = 4, kAnchor = 3, kResidualGroup = RESIDUAL_GROUP;
};

// Row stride (floats) of a tile of rotated rows in shared memory: conflict-free for the MMA fragment loads.
template <int D>
constexpr int kTileStride = D + 8;

// Everything that happens to the rows of one (token, head, plane): the anchor record, then the residual records.
// Eight lanes own the row (lane j: channels 16j .. 16j+15); `token` is the lane group's token.  SHARED_ROWS: the rows
// were rotated by a dense matrix into `tile` (shared memory, fp32 [record * 16 + token % 16][kTileStride]) by
// quantize_dense_kernel; otherwise they are read from the caller's bf16 tensors and rotated here if the plane has a
// signed-Hadamard rotation.
template <int D, class S, bool SHARED_ROWS>
__device__ __forceinline__ void quantize_rows(const QuantizeParams& p, int token, int head, int plane, const float* tile,
                                              float* scratch) {
    // run-time values, or the schedule's constants
    const int num_records = [&] { if constexpr (S::kFixed) return S::kRecords; else return p.num_records; }();
    const int anchor = [&] { if constexpr (S::kFixed) return S::kAnchor; else return p.anchor; }();
    const int chain = S::kFixed ? static_cast<int>(RQ_CHAIN_KERNEL) : p.chain;
    const int coefficient_kind = S::kFixed ? static_cast<int>(RQ_COEFF_LS) : p.coefficient;
    const int mode = S::kFixed ? static_cast<int>(RQ_REFERENCE_ANCHOR) : p.mode;
    auto record_bits = [&](int r) { if constexpr (S::kFixed) return r == S::kAnchor ? 4 : 2; else return p.bits[r]; };
    auto record_group = [&](int r) {
        if constexpr (S::kFixed) return r == S::kAnchor ? 32 : S::kResidualGroup; else return p.group[r];
    };
    constexpr int kSlices = D / 16;
    const int lane = threadIdx.x & 31;
    const int j = lane & 7;

    int64_t slot = -1;
    if (token < p.num_tokens) slot = p.slots[token];
    if (__ballot_sync(kFullMask, slot >= 0) == 0u) return;  // padding only: nothing to read or write
    const bool active = slot >= 0 && j < kSlices;

    const __nv_bfloat16* const* sources = plane == 0 ? p.key : p.value;
    const int64_t* strides = plane == 0 ? p.key_stride : p.value_stride;
    const bool rotated = !SHARED_ROWS && p.rotation[plane] == RQ_ROTATION_SIGNED_HADAMARD;
    const float rscale = p.rscale[plane];
    uint32_t sign16 = 0;
    if (rotated && j < kSlices)
        sign16 = (p.sign[plane][head * (D / 32) + (j >> 1)] >> (16 * (j & 1))) & 0xffffu;
    // bit 15 / bit 31 of word i flips channel 2i / 2i+1 of the lane (rows are loaded as pairs of bf16)
    uint32_t sign_words[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        sign_words[i] = (((sign16 >> (2 * i)) & 1u) << 15) | (((sign16 >> (2 * i + 1)) & 1u) << 31);
    const bool centered = plane == 0 && p.mean != nullptr;

    const int P = p.page_tokens;
    const int tok = active ? static_cast<int>(slot % P) : 0;
    uint8_t* page = p.cache + plane * p.plane_stride +
                    (active ? (slot / P * p.heads + head) * static_cast<int64_t>(P) * p.page_width : 0);

    // Rows of 16-byte aligned bf16 tensors are fetched as two 16-byte words per lane, one record ahead of their use.
    const bool packed_rows = p.vector_loads && !SHARED_ROWS;
    auto fetch_packed = [&](int r, uint32_t (&w)[8]) {
        uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
        if (active) {
            const uint4* src = reinterpret_cast<const uint4*>(sources[r] + static_cast<int64_t>(token) * strides[r] +
                                                              head * D + 16 * j);
            lo = __ldg(src);
            hi = __ldg(src + 1);
        }
        w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w;
        w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
    };
    // flip = apply the rotation's sign diagonal (rows that go straight into the forward rotation)
    auto unpack = [&](const uint32_t (&w)[8], float (&x)[16], bool flip) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t flipped = flip ? w[i] ^ sign_words[i] : w[i];  // sign diagonal on the raw bf16 pair
            x[2 * i] = __uint_as_float(flipped << 16);
            x[2 * i + 1] = __uint_as_float(flipped & 0xffff0000u);
        }
    };
    // the other two sources: fp32 rows rotated by the dense path (shared memory), and bf16 rows without 16-byte alignment
    auto load_unpacked = [&](int r, float (&x)[16], bool flip) {
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = 0.f;
        if (!active) return;
        if constexpr (SHARED_ROWS) {
            const float4* src4 = reinterpret_cast<const float4*>(tile + (r * 16 + (threadIdx.x >> 3)) * kTileStride<D> + 16 * j);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = src4[i];
                x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
            }
            return;
        }
        const __nv_bfloat16* src = sources[r] + static_cast<int64_t>(token) * strides[r] + head * D + 16 * j;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float v = __bfloat162float(src[i]);
            x[i] = (flip && ((sign16 >> i) & 1u)) ? -v : v;
        }
    };
    auto load_mean = [&](int r, float (&m)[16]) {
#pragma unroll
        for (int i = 0; i < 16; ++i) m[i] = 0.f;
        if (centered && j < kSlices) {
            const float4* src = reinterpret_cast<const float4*>(p.mean + (static_cast<int64_t>(r) * p.heads + head) * D + 16 * j);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = __ldg(src + i);
                m[4 * i] = v.x; m[4 * i + 1] = v.y; m[4 * i + 2] = v.z; m[4 * i + 3] = v.w;
            }
        }
    };
    // Quantize z (already centered) as record r, store it, return the codes and parameters.
    auto commit_as = [&](auto bits_tag, int r, const float (&z)[16], uint16_t alpha_bits) -> GroupCode {
        constexpr int kBits = decltype(bits_tag)::value;
        const int group = record_group(r);
        const GroupCode q = group_quantize<kBits>(z, group);
        if (active) {
            constexpr int kCodeBytes = D * kBits / 8;
            const int groups = D / group;
            uint8_t* record = page + static_cast<int64_t>(P) * p.record_offset[r];
            if (kBits == 2) {
                *reinterpret_cast<uint32_t*>(record + tok * kCodeBytes + 4 * j) = pack_codes<2, 16>(q.magic);
            } else {
                *reinterpret_cast<uint2*>(record + tok * kCodeBytes + 8 * j) =
                    make_uint2(pack_codes<4, 8>(q.magic), pack_codes<4, 8>(q.magic + 8));
            }
            uint8_t* scales = record + P * kCodeBytes;
            uint8_t* offsets = scales + P * groups;
            if (group == 16) {
                scales[tok * groups + j] = q.scale8;
                offsets[tok * groups + j] = q.offset8;
            } else if ((j & 1) == 0) {
                scales[tok * groups + (j >> 1)] = q.scale8;
                offsets[tok * groups + (j >> 1)] = q.offset8;
            }
            if (j == 0)
                *reinterpret_cast<uint16_t*>(record + P * (kCodeBytes + 2 * groups) + tok * 2) = alpha_bits;
        }
        return q;
    };
    auto commit = [&](int r, const float (&z)[16], uint16_t alpha_bits) -> GroupCode {
        if (record_bits(r) == 2) return commit_as(std::integral_constant<int, 2>{}, r, z, alpha_bits);
        return commit_as(std::integral_constant<int, 4>{}, r, z, alpha_bits);
    };
    // den = row_dot(ref, ref) is passed in: in anchor mode every residual record divides by the same sum.
    auto coefficient = [&](const float (&x)[16], const float (&ref)[16], float den) -> float {
        if (coefficient_kind == RQ_COEFF_UNIT) return 1.f;
        if (coefficient_kind == RQ_COEFF_NORM) {
            const float num = row_dot(x, x);
            return den > 0.f ? __fdiv_rn(__fsqrt_rn(num), fmaxf(__fsqrt_rn(den), 1e-6f)) : 0.f;
        }
        return __fdiv_rn(row_dot(x, ref), fmaxf(den, 1e-12f));
    };
    // records in processing order: the anchor, then the others in loop order
    auto record_at = [&](int k) { return k == 0 ? anchor : (k - 1 < anchor ? k - 1 : k); };

    uint32_t words[8], ahead[8];
    if (packed_rows) {
        fetch_packed(anchor, words);
        if (num_records > 1) fetch_packed(record_at(1), ahead);
    }

    float ref[16];  // bf16-valued reconstruction that residuals predict from
    {
        float y[16], mean[16];
        if (packed_rows) unpack(words, y, true); else load_unpacked(anchor, y, true);
        if (rotated) rotate_row<D, false>(y, j, sign16, rscale, scratch);
        if (centered) {
            load_mean(anchor, mean);
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] = __fsub_rn(y[i], mean[i]);
        }
        const GroupCode q = commit(anchor, y, 0x3F80u);
        const float scale = fp8_decode(q.scale8), offset = fp8_decode(q.offset8);
        if (chain == RQ_CHAIN_KERNEL) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                ref[i] = restore_bf16(q.magic[i], scale, offset);
                if (centered) ref[i] = bf16_add(ref[i], bf16_round(mean[i]));
            }
        } else {
            // decoded value (+ mean) back in original coordinates, rounded to bf16 there
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                ref[i] = __fmaf_rn(code_value(q.magic[i]), scale, offset);
                if (centered) ref[i] = __fadd_rn(ref[i], mean[i]);
            }
            if (rotated) rotate_row<D, true>(ref, j, sign16, rscale, scratch);
#pragma unroll
            for (int i = 0; i < 16; ++i) ref[i] = bf16_round(ref[i]);
        }
    }
    float den = 0.f;
    if (coefficient_kind != RQ_COEFF_UNIT && num_records > 1) den = row_dot(ref, ref);

#pragma unroll(S::kFixed ? 4 : 1)
    for (int k = 1; k < num_records; ++k) {
        const int r = record_at(k);
        float y[16], mean[16];
        if (packed_rows) {
#pragma unroll
            for (int i = 0; i < 8; ++i) words[i] = ahead[i];
            if (k + 1 < num_records) fetch_packed(record_at(k + 1), ahead);
            unpack(words, y, chain == RQ_CHAIN_KERNEL);
        } else {
            load_unpacked(r, y, chain == RQ_CHAIN_KERNEL);
        }
        uint16_t alpha_bits;
        if (chain == RQ_CHAIN_KERNEL) {
            if (rotated) rotate_row<D, false>(y, j, sign16, rscale, scratch);
            const __nv_bfloat16 stored = __float2bfloat16_rn(coefficient(y, ref, den));
            alpha_bits = __bfloat16_as_ushort(stored);
            const float alpha = __bfloat162float(stored);
            const float2 minus_alpha = make_float2(-alpha, -alpha);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 v = fma2(RQ_PAIR(ref, i), minus_alpha, RQ_PAIR(y, i));  // y - ref * alpha, one rounding
                RQ_UNPAIR(y, i, v);
            }
        } else {
            const __nv_bfloat16 stored = __float2bfloat16_rn(coefficient(y, ref, den));
            alpha_bits = __bfloat16_as_ushort(stored);
            const float alpha = __bfloat162float(stored);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float prediction = bf16_round(__fmul_rn(ref[i], alpha));
                const float target = bf16_round(__fsub_rn(y[i], prediction));
                y[i] = ((sign16 >> i) & 1u) ? -target : target;  // sign diagonal of the forward rotation
            }
            if (rotated) rotate_row<D, false>(y, j, sign16, rscale, scratch);
        }
        if (centered) {
            load_mean(r, mean);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 v = sub2(RQ_PAIR(y, i), RQ_PAIR(mean, i));
                RQ_UNPAIR(y, i, v);
            }
        }
        const GroupCode q = commit(r, y, alpha_bits);
        if (mode == RQ_REFERENCE_ADJACENT) {
            // the next record predicts from this record's reconstruction (reference: kernel.cuh:195-201)
            const float scale = fp8_decode(q.scale8), offset = fp8_decode(q.offset8);
            const __nv_bfloat16 alpha_bf = __ushort_as_bfloat16(alpha_bits);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float restored = restore_bf16(q.magic[i], scale, offset);
                if (centered) restored = bf16_add(restored, bf16_round(mean[i]));
                ref[i] = __bfloat162float(
                    __hfma(__float2bfloat16_rn(ref[i]), alpha_bf, __float2bfloat16_rn(restored)));
            }
            if (coefficient_kind != RQ_COEFF_UNIT && k + 1 < num_records) den = row_dot(ref, ref);
        }
    }
}

template <int D, class S>
__global__ void __launch_bounds__(128, 5) quantize_kernel(const __grid_constant__ QuantizeParams p) {
    // Launched as a programmatic dependent of the previous kernel of the stream: the launch itself overlaps that kernel;
    // nothing is read or written before it has completed.  After that the next kernel may be scheduled.
    pdl_wait();
    pdl_launch_dependents();
    __shared__ __align__(16) float paley[D == 96 ? 4 * kPaleyWarpFloats : 4];  // head_dim 96: the rotation's 12-point stage
    const int token = blockIdx.x * 16 + (threadIdx.x >> 3);  // a warp owns 4 consecutive tokens of one head
    quantize_rows<D, S, false>(p, token, blockIdx.y, p.plane_first + blockIdx.z, nullptr,
                               paley + (D == 96 ? (threadIdx.x >> 5) * kPaleyWarpFloats : 0));
}

// ---- dense (learned) rotation fused into the quantizer ------------------------------------------------------------
// y = x @ R[h] for every record's row, on the tensor cores, inside the CTA that quantizes the rows: R[h] is staged once
// per CTA in shared memory (fp32: bf16 inputs and fp16 matrix entries are exact in TF32, fp32 accumulation, like the
// reference's rotation, plugins/residual_quantization/csrc/quantize/rotation.cuh:25-150), the CTA then walks over
// kDenseTiles tiles of 16 tokens: stage the tile's records x 16 rows, rotate them in place (one 16-row MMA tile per
// warp and record), quantize them from shared memory.  Nothing goes through global memory in between.
constexpr int kDenseTiles = 4;  // long writes: 64 (or 128) tokens per CTA, the matrix is staged once per CTA

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// The staged matrix is stored in the order the MMA's B fragments are consumed, so that a lane fetches the fragments of
// two adjacent 8-column tiles with one 8-byte load: entry ((k / 8) * (D / 16) + n / 2) * 32 + lane holds the four halves
// {R[k0][8n+g], R[k0+1][8n+g], R[k0][8(n+1)+g], R[k0+1][8(n+1)+g]} with k0 = k - k % 8 + 2 * (lane % 4), g = lane / 4.
// (Rows k0, k0 + 1 are the k-indices "t" and "t + 4" of the MMA: the product does not care which physical row carries
// which index as long as the A fragment uses the same assignment.)  It stays fp16 in shared memory -- half the bytes of
// a binary32 copy, which is what lets three CTAs share an SM instead of two -- and is widened (exactly) when a fragment
// is loaded: two conversions per MMA on a kernel whose issue slots are two thirds idle.
template <int D>
constexpr int kMatrixFloats = D * D;   // entries

template <int D>
size_t dense_shared_bytes(int num_records) {
    return static_cast<size_t>(kMatrixFloats<D>) * sizeof(__half) + static_cast<size_t>(num_records) * 16 * kTileStride<D> * sizeof(float);
}

template <int D, class S>
__global__ void __launch_bounds__(128, 3) quantize_dense_kernel(const __grid_constant__ QuantizeParams p) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float dense_shared[];
    uint2* matrix = reinterpret_cast<uint2*>(dense_shared);   // fp16, fragment order, see kMatrixFloats
    float* tile = dense_shared + kMatrixFloats<D> / 2;        // [records * 16][kTileStride]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.y, plane = p.plane_first + blockIdx.z;
    const int num_records = [&] { if constexpr (S::kFixed) return S::kRecords; else return p.num_records; }();
    const int tiles = p.dense_tiles;
    if (p.dense_matrix[plane] == nullptr) {
        // the other plane of the same call has no dense rotation: same launch, plain path
        for (int step = 0; step < tiles; ++step)   // the tile area is free here: it serves as the rotation's scratch
            quantize_rows<D, S, false>(p, (blockIdx.x * tiles + step) * 16 + (tid >> 3), head, plane, nullptr,
                                       tile + warp * kPaleyWarpFloats);
        return;
    }

    // R[h]: fp16 [D][D] -> shared memory, in fragment order.  A warp fills one block of 32 entries (the B fragments of one
    // k-step and one pair of 8-column tiles) per round: every lane gathers its own four halves -- two rows, two column
    // tiles -- and stores them as 8 bytes, so the stores are contiguous over the warp (no bank conflict); the 2-byte
    // gathers hit L1/L2, every CTA of the head reads the same 2 D^2 bytes.
    {
        const unsigned short* r = reinterpret_cast<const unsigned short*>(p.dense_matrix[plane]) + static_cast<int64_t>(head) * D * D;
        const int g = lane >> 2, t = lane & 3;
        constexpr int kBlocks = (D / 8) * (D / 16);
#pragma unroll 4
        for (int block = warp; block < kBlocks; block += 4) {
            const int ks = block / (D / 16), pair = block % (D / 16);
            const unsigned short* from = r + (8 * ks + 2 * t) * D + 16 * pair + g;
            const unsigned short a0 = __ldg(from), a1 = __ldg(from + D), b0 = __ldg(from + 8), b1 = __ldg(from + D + 8);
            matrix[block * 32 + lane] = make_uint2(a0 | (static_cast<uint32_t>(a1) << 16), b0 | (static_cast<uint32_t>(b1) << 16));
        }
    }
    const __nv_bfloat16* const* sources = plane == 0 ? p.key : p.value;
    const int64_t* strides = plane == 0 ? p.key_stride : p.value_stride;

    // A thread's share of a tile: chunk i = tid + 128 u is eight channels (16 bytes) of row i / (D/8) of the tile.  The
    // rows of the NEXT tile are fetched into registers before the current tile is rotated and quantized, so that their
    // latency is covered by that work instead of standing in front of the next staging step.
    constexpr int kChunks = 4 * 16 * (D / 8) / 128;   // per thread, for the largest group (four records)
    uint4 fetched[kChunks];
    auto fetch = [&](int first) {
        const int chunks = num_records * 16 * (D / 8);
#pragma unroll
        for (int u = 0; u < kChunks; ++u) {
            const int i = tid + 128 * u;
            const int row = i / (D / 8), c8 = i % (D / 8);
            const int record = row >> 4, token = first + (row & 15);
            fetched[u] = make_uint4(0u, 0u, 0u, 0u);   // rows of padding slots or beyond the call stay zero
            if (i < chunks && token < p.num_tokens && p.slots[token] >= 0) {
                const __nv_bfloat16* x = sources[record] + static_cast<int64_t>(token) * strides[record] + head * D + 8 * c8;
                if (p.vector_loads) {
                    fetched[u] = __ldg(reinterpret_cast<const uint4*>(x));
                } else {
                    const unsigned short* h = reinterpret_cast<const unsigned short*>(x);
                    fetched[u] = make_uint4(h[0] | (static_cast<uint32_t>(h[1]) << 16), h[2] | (static_cast<uint32_t>(h[3]) << 16),
                                            h[4] | (static_cast<uint32_t>(h[5]) << 16), h[6] | (static_cast<uint32_t>(h[7]) << 16));
                }
            }
        }
    };
    const int first_tile = blockIdx.x * tiles * 16;
    if (first_tile < p.num_tokens) fetch(first_tile);

    for (int step = 0; step < tiles; ++step) {
        const int first = (blockIdx.x * tiles + step) * 16;
        if (first >= p.num_tokens) break;  // uniform over the CTA
        __syncthreads();  // the previous tile has been quantized (and, the first time, the matrix is staged below the next barrier)
        // stage: the fetched bf16 rows -> fp32
        {
            const int chunks = num_records * 16 * (D / 8);
#pragma unroll
            for (int u = 0; u < kChunks; ++u) {
                const int i = tid + 128 * u;
                if (i < chunks) {
                    const int row = i / (D / 8), c8 = i % (D / 8);
                    const uint32_t words[4] = {fetched[u].x, fetched[u].y, fetched[u].z, fetched[u].w};
                    float4* dst = reinterpret_cast<float4*>(tile + row * kTileStride<D> + 8 * c8);
                    dst[0] = make_float4(__uint_as_float(words[0] << 16), __uint_as_float(words[0] & 0xffff0000u),
                                         __uint_as_float(words[1] << 16), __uint_as_float(words[1] & 0xffff0000u));
                    dst[1] = make_float4(__uint_as_float(words[2] << 16), __uint_as_float(words[2] & 0xffff0000u),
                                         __uint_as_float(words[3] << 16), __uint_as_float(words[3] & 0xffff0000u));
                }
            }
        }
        if (step + 1 < tiles && first + 16 < p.num_tokens) fetch(first + 16);
        __syncthreads();
        // rotate in place: warp w takes the 16-row tiles w, w + 4, ... (one per record in a four-record group)
        const int g = lane >> 2, t = lane & 3;
        for (int block = warp; block < num_records; block += 4) {
            float* rows = tile + block * 16 * kTileStride<D>;
            float acc[D / 8][4];
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
            const uint2* fragments = matrix + lane;
#pragma unroll 2
            for (int k = 0; k < D; k += 8) {
                // physical columns k + 2t, k + 2t + 1 of the rows play the k-indices t, t + 4
                const float2 upper = *reinterpret_cast<const float2*>(rows + g * kTileStride<D> + k + 2 * t);
                const float2 lower = *reinterpret_cast<const float2*>(rows + (g + 8) * kTileStride<D> + k + 2 * t);
                const uint32_t a[4] = {__float_as_uint(upper.x), __float_as_uint(lower.x), __float_as_uint(upper.y),
                                       __float_as_uint(lower.y)};
#pragma unroll
                for (int n = 0; n < D / 8; n += 2) {
                    const uint2 packed = fragments[((k >> 3) * (D / 16) + (n >> 1)) * 32];
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&packed.x));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&packed.y));
                    const uint32_t b0[2] = {__float_as_uint(f0.x), __float_as_uint(f0.y)};
                    const uint32_t b1[2] = {__float_as_uint(f1.x), __float_as_uint(f1.y)};
                    mma_tf32(acc[n], a, b0);
                    mma_tf32(acc[n + 1], a, b1);
                }
            }
            __syncwarp();  // every lane has read the rows it needs before they are overwritten
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                *reinterpret_cast<float2*>(rows + g * kTileStride<D> + 8 * n + 2 * t) = make_float2(acc[n][0], acc[n][1]);
                *reinterpret_cast<float2*>(rows + (g + 8) * kTileStride<D> + 8 * n + 2 * t) = make_float2(acc[n][2], acc[n][3]);
            }
        }
        __syncthreads();
        quantize_rows<D, S, true>(p, first + (tid >> 3), head, plane, tile, nullptr);
    }
}

// Decode-sized writes of the headline schedule: a handful of tokens, so latency is what counts.  One warp per
// (token, head, plane); its four 8-lane groups take the four records of the token side by side: every group loads
// and rotates its own record at the same time, the last group's anchor is quantized and its bf16 reconstruction is
// handed to the other three by shuffles, which then form their coefficients and quantize together.  Each row sees the
// same operations in the same order as in quantize_kernel (8 lanes per row, 16 channels per lane), so the packed bytes
// are identical; only the four records of a token no longer wait for one another.
template <int D, int RESIDUAL_GROUP>
__global__ void __launch_bounds__(128) quantize_token_kernel(const __grid_constant__ QuantizeParams p) {
    constexpr int kSlices = D / 16, kAnchor = 3;
    pdl_wait();  // see quantize_kernel
    pdl_launch_dependents();
    __shared__ __align__(16) float paley[D == 96 ? 4 * kPaleyWarpFloats : 4];  // head_dim 96: the rotation's 12-point stage
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* scratch = paley + (D == 96 ? warp * kPaleyWarpFloats : 0);
    const int j = lane & 7, record = lane >> 3;
    const int token = blockIdx.x * 4 + warp;
    const int head = blockIdx.y, plane = p.plane_first + blockIdx.z;
    if (token >= p.num_tokens) return;
    const int64_t slot = p.slots[token];
    if (slot < 0) return;  // padding (the whole warp)
    const bool owner = j < kSlices;

    const __nv_bfloat16* const* sources = plane == 0 ? p.key : p.value;
    const int64_t* strides = plane == 0 ? p.key_stride : p.value_stride;
    const bool rotated = p.rotation[plane] == RQ_ROTATION_SIGNED_HADAMARD;
    const float rscale = p.rscale[plane];
    uint32_t sign16 = 0;
    if (rotated && owner) sign16 = (p.sign[plane][head * (D / 32) + (j >> 1)] >> (16 * (j & 1))) & 0xffffu;
    const bool centered = plane == 0 && p.mean != nullptr;

    float y[16], mean[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = mean[i] = 0.f;
    if (owner) {
        const uint4* src = reinterpret_cast<const uint4*>(sources[record] + static_cast<int64_t>(token) * strides[record] +
                                                          head * D + 16 * j);
        const uint4 lo = __ldg(src), hi = __ldg(src + 1);
        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t flip = (((sign16 >> (2 * i)) & 1u) << 15) | (((sign16 >> (2 * i + 1)) & 1u) << 31);
            const uint32_t word = w[i] ^ flip;  // sign diagonal on the raw bf16 pair
            y[2 * i] = __uint_as_float(word << 16);
            y[2 * i + 1] = __uint_as_float(word & 0xffff0000u);
        }
        if (centered) {
            const float4* m4 = reinterpret_cast<const float4*>(p.mean + (static_cast<int64_t>(record) * p.heads + head) * D + 16 * j);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = __ldg(m4 + i);
                mean[4 * i] = v.x; mean[4 * i + 1] = v.y; mean[4 * i + 2] = v.z; mean[4 * i + 3] = v.w;
            }
        }
    }
    if (rotated) rotate_row<D, false>(y, j, sign16, rscale, scratch);
    const int P = p.page_tokens;
    const int tok = static_cast<int>(slot % P);
    uint8_t* page = p.cache + plane * p.plane_stride + (slot / P * p.heads + head) * static_cast<int64_t>(P) * p.page_width;
    uint8_t* out = page + static_cast<int64_t>(P) * p.record_offset[record];
    auto store_parameters = [&](int code_bytes, int group, const GroupCode& q, uint16_t alpha_bits) {
        const int groups = D / group;
        uint8_t* scales = out + P * code_bytes;
        uint8_t* offsets = scales + P * groups;
        if (group == 16) {
            scales[tok * groups + j] = q.scale8;
            offsets[tok * groups + j] = q.offset8;
        } else if ((j & 1) == 0) {
            scales[tok * groups + (j >> 1)] = q.scale8;
            offsets[tok * groups + (j >> 1)] = q.offset8;
        }
        if (j == 0) *reinterpret_cast<uint16_t*>(out + P * (code_bytes + 2 * groups) + tok * 2) = alpha_bits;
    };

    // ---- the anchor (every group runs the arithmetic on its own row, only the anchor's group keeps the result) ----
    float ref[16];
    {
        float z[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) z[i] = centered ? __fsub_rn(y[i], mean[i]) : y[i];
        const GroupCode q = group_quantize<4>(z, 32);
        if (record == kAnchor && owner) {
            *reinterpret_cast<uint2*>(out + tok * (D / 2) + 8 * j) =
                make_uint2(pack_codes<4, 8>(q.magic), pack_codes<4, 8>(q.magic + 8));
            store_parameters(D / 2, 32, q, 0x3F80u);
        }
        const float scale = fp8_decode(q.scale8), offset = fp8_decode(q.offset8);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float restored = restore_bf16(q.magic[i], scale, offset);
            if (centered) restored = bf16_add(restored, bf16_round(mean[i]));
            ref[i] = __shfl_sync(kFullMask, restored, 8 * kAnchor + j);  // the anchor group's value for this slice
        }
    }
    // ---- the three residual records, side by side ----
    const float den = row_dot(ref, ref);
    const __nv_bfloat16 stored = __float2bfloat16_rn(__fdiv_rn(row_dot(y, ref), fmaxf(den, 1e-12f)));
    const float alpha = __bfloat162float(stored);
    const float2 minus_alpha = make_float2(-alpha, -alpha);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float2 v = fma2(RQ_PAIR(ref, i), minus_alpha, RQ_PAIR(y, i));
        if (centered) v = sub2(v, RQ_PAIR(mean, i));
        RQ_UNPAIR(y, i, v);
    }
    const GroupCode q = group_quantize<2>(y, RESIDUAL_GROUP);
    if (record != kAnchor && owner) {
        *reinterpret_cast<uint32_t*>(out + tok * (D / 4) + 4 * j) = pack_codes<2, 16>(q.magic);
        store_parameters(D / 4, RESIDUAL_GROUP, q, __bfloat16_as_ushort(stored));
    }
}

template <class Kernel>
cudaError_t launch_with_order(Kernel kernel, dim3 grid, size_t shared_bytes, const QuantizeParams& p, cudaStream_t stream) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(128);
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = p.programmatic_launch ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, p);
}

// The dense kernel needs more than the default 48 KB of dynamic shared memory: raised once per device and instantiation.
template <class Kernel>
cudaError_t allow_shared_bytes(Kernel kernel, size_t bytes, std::atomic<unsigned long long>& configured) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    const unsigned long long bit = 1ull << (device & 63);
    if (configured.load(std::memory_order_acquire) & bit) return cudaSuccess;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (err == cudaSuccess) configured.fetch_or(bit, std::memory_order_release);
    return err;
}

template <int D, class S>
cudaError_t launch_dense(const QuantizeParams& p, cudaStream_t stream) {
    static std::atomic<unsigned long long> configured{0ull};
    const size_t bytes = dense_shared_bytes<D>(RQ_MAX_RECORDS);  // the attribute covers every group size
    cudaError_t err = allow_shared_bytes(quantize_dense_kernel<D, S>, bytes, configured);
    if (err != cudaSuccess) return err;
    const dim3 grid((p.num_tokens + 16 * p.dense_tiles - 1) / (16 * p.dense_tiles), p.heads, p.dense_planes);
    return launch_with_order(quantize_dense_kernel<D, S>, grid, dense_shared_bytes<D>(p.num_records), p, stream);
}

// One launch for the planes `first` .. `first + count - 1`, none of which has a dense rotation.
cudaError_t launch_plain(QuantizeParams p, int head_dim, bool headline, int first, int count, cudaStream_t stream) {
    p.plane_first = first;
    const dim3 grid((p.num_tokens + 15) / 16, p.heads, count);
    // decode-sized writes of aligned bf16 rows: one warp per token with the records side by side
    if (headline && p.num_tokens <= 256 && p.vector_loads) {
        const dim3 token_grid((p.num_tokens + 3) / 4, p.heads, count);
        if (head_dim == 128 && p.group[0] == 32) return launch_with_order(quantize_token_kernel<128, 32>, token_grid, 0, p, stream);
        if (head_dim == 128) return launch_with_order(quantize_token_kernel<128, 16>, token_grid, 0, p, stream);
        if (p.group[0] == 32) return launch_with_order(quantize_token_kernel<96, 32>, token_grid, 0, p, stream);
        return launch_with_order(quantize_token_kernel<96, 16>, token_grid, 0, p, stream);
    }
    if (headline && p.group[0] == 32) {
        if (head_dim == 128) return launch_with_order(quantize_kernel<128, Anchor2224<32>>, grid, 0, p, stream);
        return launch_with_order(quantize_kernel<96, Anchor2224<32>>, grid, 0, p, stream);
    }
    if (headline && p.group[0] == 16) {
        if (head_dim == 128) return launch_with_order(quantize_kernel<128, Anchor2224<16>>, grid, 0, p, stream);
        return launch_with_order(quantize_kernel<96, Anchor2224<16>>, grid, 0, p, stream);
    }
    if (head_dim == 128) return launch_with_order(quantize_kernel<128, AnySchedule>, grid, 0, p, stream);
    return launch_with_order(quantize_kernel<96, AnySchedule>, grid, 0, p, stream);
}

cudaError_t launch_dense_planes(QuantizeParams p, int head_dim, bool headline, int first, int count, cudaStream_t stream) {
    p.plane_first = first;
    p.dense_planes = count;
    // short (decode-sized) writes: one tile per CTA, so that the few tokens spread over as many SMs as possible
    // long writes: the matrix is staged once per CTA, so more tiles per CTA as long as the grid keeps several waves
    p.dense_tiles = p.num_tokens <= 1024 ? 1 : p.num_tokens <= 4096 ? kDenseTiles : 2 * kDenseTiles;
    if (headline && p.group[0] == 32)
        return head_dim == 128 ? launch_dense<128, Anchor2224<32>>(p, stream) : launch_dense<96, Anchor2224<32>>(p, stream);
    if (headline && p.group[0] == 16)
        return head_dim == 128 ? launch_dense<128, Anchor2224<16>>(p, stream) : launch_dense<96, Anchor2224<16>>(p, stream);
    return head_dim == 128 ? launch_dense<128, AnySchedule>(p, stream) : launch_dense<96, AnySchedule>(p, stream);
}

}  // namespace

// Neither plane dense: one launch.  A dense plane: short (decode-sized) writes still take one launch -- the fused
// kernel covers both planes and a plane without a dense rotation takes the plain path inside it, because there the
// launch is what costs; long writes take one launch per plane, so that the plain plane runs at the plain kernel's
// higher occupancy.  No scratch buffer and no separate rotation launch either way.
cudaError_t launch_quantize(const QuantizeParams& p, int head_dim, cudaStream_t stream) {
    const bool headline = p.num_records == 4 && p.anchor == 3 && p.mode == RQ_REFERENCE_ANCHOR &&
                          p.coefficient == RQ_COEFF_LS && p.chain == RQ_CHAIN_KERNEL && p.bits[3] == 4 && p.group[3] == 32 &&
                          p.bits[0] == 2 && p.bits[1] == 2 && p.bits[2] == 2 && p.group[0] == p.group[1] &&
                          p.group[1] == p.group[2];
    const bool dense[2] = {p.dense_matrix[0] != nullptr, p.dense_matrix[1] != nullptr};
    if (!dense[0] && !dense[1]) return launch_plain(p, head_dim, headline, 0, 2, stream);
    if (p.num_tokens <= 1024 || (dense[0] && dense[1])) return launch_dense_planes(p, head_dim, headline, 0, 2, stream);
    for (int plane = 0; plane < 2; ++plane) {
        const cudaError_t err = dense[plane] ? launch_dense_planes(p, head_dim, headline, plane, 1, stream)
                                             : launch_plain(p, head_dim, headline, plane, 1, stream);
        if (err != cudaSuccess) return err;
    }
    return cudaSuccess;
}

}  // namespace rq
