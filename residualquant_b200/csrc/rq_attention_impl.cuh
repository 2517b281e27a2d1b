// Packed paged decode attention (anchor and adjacent reference modes), one launch per call.
//
// Replaces the reference's three kernels -- attention_prepare_kernel, attention_kernel, attention_merge_kernel
// (plugins/residual_quantization/csrc/attention/prepare.cuh:391-430, compute.cuh:226-727, merge.cuh:9-84) --
// and its page staging (attention/async_copy.cuh:109-168).
//
// Shape of the computation
//   CTA  = one (work item, head); a work item is one KV partition of one query row.  grid = items * heads, heads
//          fastest so that CTAs that run together read neighbouring pages of the same block.  How many partitions a
//          row gets is decided on the device from the sequence lengths (find_work): proportional to the row's pages,
//          inside a capacity the host fixed, so the grid stays CUDA-graph static.
//   warp = an independent consumer of every 4th page of the partition with its OWN ring of shared-memory
//          stages.  Default staging: every lane issues 16-byte cp.async.cg copies, one commit group per page, STAGES
//          pages ahead (build flag RQ_ATTENTION_BULK_COPY=1: lane 0 issues cp.async.bulk copies that complete on an
//          mbarrier instead).  There is no CTA-wide barrier inside the page loop.
//   lane = (token slot, 32-channel slice): 4 lanes per token, 8 tokens per warp step.  A slice is exactly one
//          INT4 g32 anchor group, so scale/offset handling is per lane, not per channel.
//   maths: no code is ever converted to a floating-point number one at a time.
//          K: integer dot products (dp2a) of the masked code bytes against the rotated query quantized once per CTA
//             to 11 bits (INT4 records) or 13 bits (INT2 records), factored per slice as scale * sum(q*code) + offset * sum(q);
//          softmax: one online-softmax stream per 4-lane token slot (fp32 reference exponent that moves only when a
//             score exceeds it by more than a slack, denominator and offsets in fp32, base-2 exponent);
//          V: `word & mask` read as a half2 IS a pair of codes times 2^-24 (subnormal halves are linear in their bit
//             pattern), so one half2 FMA per channel pair with probability * alpha * scale * 2^11 as the weight;
//             half2 sums are flushed to fp32 every 8 tokens; the offset part is accumulated once per group.
//   merge: each warp folds its 8 streams, the CTA folds its 4 warps, and -- when the row has several
//          partitions -- the LAST CTA to arrive (one atomic ticket per (row, head)) folds the partitions, adds the
//          live token, undoes an explicit value rotation and stores bf16.  No second launch, no spin wait.
//   launch: as a programmatic dependent of the previous kernel of the stream.  Every CTA waits for the PREVIOUS kernel
//          to complete (griddepcontrol.wait) before it reads anything, then lets the NEXT kernel be scheduled
//          (griddepcontrol.launch_dependents) -- so launch latency and CTA scheduling overlap the previous kernel.
//          When the caller promises that this call's metadata and cache pages were not written by that previous kernel
//          (early_start), the work lookup, the page-table fetch and the first page copies run BEFORE the wait as well
//          (through L2 only: ld.global.cg / cp.async.cg), and only the q/k/v rows are read after it.
//   gather: with KV heads sharded over GPUs the finished rows also go into every GPU's gathered buffer (peer stores); the
//          CTA that finishes the call's last row can publish completion and wait for the peers (bounded).
//
// The query rotation is fused into the prologue of every CTA: a signed Walsh-Hadamard transform (128 values, one warp),
// or, for a dense learned matrix, a row-times-matrix product shared by the four warps.
//
// In the bulk-copy build every wait on an mbarrier is bounded; on expiry the kernel raises the workspace status word,
// drains what it can and returns.  The default build has no wait that can fail.
#include <atomic>
#include <type_traits>

#include "rq_common.cuh"
#include "rq_kernels.h"

namespace rq {
namespace {

#ifndef RQ_ATTENTION_BULK_COPY
#define RQ_ATTENTION_BULK_COPY 0
#endif
// Page staging engine: 1 = one elected lane issues cp.async.bulk copies that complete on an mbarrier,
// 0 = every lane issues 16-byte cp.async copies tracked by commit groups (fewer instructions per page).
constexpr bool kBulkCopy = RQ_ATTENTION_BULK_COPY != 0;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNever = -1e30f;  // exponent of a stream that has seen no token: exp2(kNever - anything real) == 0

// P[i][j] == -1  <=>  bit j of kPaleyRow[i]  <=>  bit i of kPaleyCol[j]
__constant__ uint32_t kPaleyRowA[16] = {0x0, 0x476, 0x8ec, 0x1da, 0x3b4, 0x768, 0xed0, 0xda2,
                                        0xb46, 0x68e, 0xd1c, 0xa3a, 0, 0, 0, 0};
__constant__ uint32_t kPaleyColA[16] = {0x0, 0xb8a, 0x716, 0xe2c, 0xc5a, 0x8b6, 0x16e, 0x2dc,
                                        0x5b8, 0xb70, 0x6e2, 0xdc4, 0, 0, 0, 0};

template <int D_, int AB_, int AG_, int RB_, int RG_, int P_, bool MEAN_, bool ADJ_ = false>
struct Config {
    static constexpr int D = D_, AB = AB_, AG = AG_, RB = RB_, RG = RG_, P = P_;
    static constexpr bool kMean = MEAN_, kResidual = RB_ != 0;
    // Adjacent mode stages the whole prefix of records 0..loop (run-time size, at most four INT4 g32 records).
    static constexpr bool kAdjacent = ADJ_;
    static constexpr int kMaxPrefixBytes = P * 4 * (D / 2 + 2 * (D / 32) + 2);
    static_assert(AB == 2 || AB == 4, "anchor record must be INT2 or INT4");
    static_assert(RB == 0 || RB == 2 || RB == 4, "residual record must be absent, INT2 or INT4");
    static_assert(D == 128 || D == 96, "head_dim 128 or 96");
    static constexpr int kAnchorCode = D * AB / 8, kAnchorGroups = D / AG;
    static constexpr int kAnchorBytes = P * (kAnchorCode + 2 * kAnchorGroups);  // staged without its alpha column
    static constexpr int kResidualCode = kResidual ? D * RB / 8 : 0;
    static constexpr int kResidualGroups = kResidual ? D / RG : 0;
    static constexpr int kResidualBytes = kResidual ? P * (kResidualCode + 2 * kResidualGroups + 2) : 0;
    static constexpr int kPlaneBytes = kAnchorBytes + kResidualBytes;
    static constexpr int kStageBytes = kAdjacent ? 2 * kMaxPrefixBytes : 2 * kPlaneBytes;
    // pages in flight per warp; sized so that four CTAs (16 warps) fit in one SM's shared memory at block size 16
    static constexpr int kMinBlocks = 4;  // CTAs per SM the register allocation aims for (5 for the anchor loop measured no faster)
    static constexpr int kBaseStages = kAdjacent ? 2 : (P == 16 ? (kResidual ? 3 : 4) : 2);
    static constexpr int kScratchStages = (32 * 33 * 4 + kStageBytes - 1) / kStageBytes;  // the ring doubles as merge scratch
    static constexpr int kStages = kBaseStages > kScratchStages ? kBaseStages : kScratchStages;
    static constexpr int kRingBytes = kStages * kStageBytes;
    static_assert(kAnchorBytes % 16 == 0 && kResidualBytes % 16 == 0, "bulk copies need 16-byte multiples");
    static_assert(kRingBytes >= 32 * 33 * 4, "the ring doubles as the warp's merge scratch");
    // shared memory map (bytes)
    static constexpr int kOffRing = 0;
    static constexpr int kOffQuery = kOffRing + kWarps * kRingBytes;       // float[D]
    static constexpr int kOffWarpAcc = kOffQuery + D * 4;                  // float[kWarps][D]
    static constexpr int kOffWarpStat = kOffWarpAcc + kWarps * D * 4;      // float[kWarps][2] + float misc[8]
    static constexpr int kOffBarriers = kOffWarpStat + 64;                 // uint64[kWarps][kStages]
    static constexpr int kOffWork = kOffBarriers + kWarps * kStages * 8;   // the CTA's WorkItem (6 ints)
    static constexpr int kSmemBytes = kOffWork + 32;
};

// ---- PTX wrappers --------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// 16-byte asynchronous copy global -> shared (L1 bypass), one per lane.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// Copy `BYTES` (a multiple of 16) with the whole warp: lane l moves chunks l, l+32, ...  `dst` and `src` already
// point at the lane's first chunk, so every copy differs from them by a compile-time constant only.
template <int BYTES>
__device__ __forceinline__ void warp_copy(uint32_t dst, const uint8_t* src, int lane) {
    constexpr int kChunks = BYTES / 16;
#pragma unroll
    for (int i = 0; i < (kChunks + 31) / 32; ++i) {
        if (32 * (i + 1) <= kChunks || lane + 32 * i < kChunks) cp_async16(dst + 512 * i, src + 512 * i);
    }
}
// Same with a run-time size.
__device__ __forceinline__ void warp_copy_bytes(uint32_t dst, const uint8_t* src, int bytes, int lane) {
    for (int at = 16 * lane; at < bytes; at += 512) cp_async16(dst + at, src + at);
}
// Bounded wait.  false = gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
    return d;
}
__device__ __forceinline__ __half2 as_half2(uint32_t bits) { return *reinterpret_cast<const __half2*>(&bits); }

// Shared-memory loads by 32-bit shared address (no generic-pointer arithmetic in the hot loop).
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
// d = c + a.s16[0] * b.u8[0|2] + a.s16[1] * b.u8[1|3]
__device__ __forceinline__ int dp2a_lo(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Two FP8-e4m3 bytes (first in bits 0-7, second in bits 8-15) -> two floats, one hardware conversion.
__device__ __forceinline__ float2 fp8x2_to_float2(uint32_t pair) {
    uint32_t h2;
    asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(h2) : "r"(pair));
    return __half22float2(as_half2(h2));
}
__device__ __forceinline__ uint32_t pack_s16(int lo, int hi) {
    return (static_cast<uint32_t>(lo) & 0xffffu) | (static_cast<uint32_t>(hi) << 16);
}

// half2 arithmetic on raw 32-bit registers.
__device__ __forceinline__ uint32_t hfma2_raw(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_raw(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// lo += low half of `pair`, hi += high half: mixed-precision adds (fp32 accumulator, fp16 addend), one instruction each.
__device__ __forceinline__ void add_half2_to_floats(uint32_t pair, float& lo, float& hi) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tadd.rn.f32.f16 %0, l, %0;\n\tadd.rn.f32.f16 %1, h, %1;\n\t}"
        : "+f"(lo), "+f"(hi)
        : "r"(pair));
}
__device__ __forceinline__ uint32_t half2_from(float v) {  // (v, v), saturating to the largest finite half
    uint32_t d;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %1;" : "=r"(d) : "f"(v));
    return d;
}
// V codes are never converted: a half whose raw bits are an integer N < 2048 is the number N * 2^-24 (subnormals and
// the first normal binade are linear in the bit pattern), so `word & mask` IS a pair of scaled codes and the scale
// goes into the weight.  weight * 2^11 stays a finite half for |weight| < 32 (it saturates beyond: a V group would
// need a range above ~240 for that); the half2 sums then carry a factor 2^-13: 11-bit relative precision for sums
// above 0.5, 2^-11 absolute below.
// The factor 2^11 rides on the probabilities themselves (the softmax exponent is biased by kWeightBits), so the
// denominator and the offset sums carry it too and drop it once per warp at the end.
constexpr float kWeightBits = 11.f;
constexpr float kWeightDown = 1.f / 2048.f;
constexpr float kSumDown = 8192.f;

// ---- one packed record (codes + FP8 group parameters) against a 32-channel slice ------------------------------
// Query operands for the integer dot products of one code width, built once per CTA from the rotated query slice.
//   INT4: the word itself carries bytes c_even + 16 c_odd, word & 0xF0F0F0F0 carries 16 c_odd: even channels get
//         16*q, odd ones q - 16*q_even (which takes back what the unmasked byte added); 11-bit query.
//   INT2: word & (0x03030303 << 2k) carries 4^k c: positions 0,1 get 4q, q and feed one sum, positions 2,3 get 4q, q
//         and feed a second sum that carries an extra factor 16 (shifted out exactly); 13-bit query.
template <int BITS>
struct QueryOperands {
    uint32_t op[16];
    float sum0, sum1;  // sum of the quantized query over channels 0..15 / 16..31 of the slice (real units)
    float dot_unit;    // real value of one unit of the integer dot product
};

template <int BITS>
__device__ __forceinline__ void build_operands(const float* qslice, bool slice_ok, float qmax, QueryOperands<BITS>& out) {
    constexpr float kLevels = BITS == 4 ? 1900.f : 8191.f;
    const float to_int = (slice_ok && qmax > 0.f) ? kLevels / qmax : 0.f, unit = qmax / kLevels;
    // Round to the nearest integer by adding 1.5 * 2^23: the integer sits in the low significand bits (round half to even,
    // like a float-to-int conversion), and neither the rounding nor the sums below touch the conversion unit, which the
    // four warps of a CTA would otherwise queue on right after the query arrives.
    constexpr float kMagic = 12582912.f;
    constexpr int kMagicBits = 0x4B400000;
    int iq[32];
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
        iq[c] = __float_as_int(__fmaf_rn(qslice[c], to_int, kMagic)) - kMagicBits;
        if (c < 16) s0 += iq[c]; else s1 += iq[c];
    }
    out.sum0 = static_cast<float>(s0) * unit;
    out.sum1 = static_cast<float>(s1) * unit;
    if (BITS == 4) {
        out.dot_unit = unit * 0.0625f;  // the integer dot product carries a factor 16
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            out.op[4 * w + 0] = pack_s16(16 * iq[8 * w + 0], 16 * iq[8 * w + 2]);
            out.op[4 * w + 1] = pack_s16(16 * iq[8 * w + 4], 16 * iq[8 * w + 6]);
            out.op[4 * w + 2] = pack_s16(iq[8 * w + 1] - 16 * iq[8 * w + 0], iq[8 * w + 3] - 16 * iq[8 * w + 2]);
            out.op[4 * w + 3] = pack_s16(iq[8 * w + 5] - 16 * iq[8 * w + 4], iq[8 * w + 7] - 16 * iq[8 * w + 6]);
        }
    } else {
        out.dot_unit = unit * 0.25f;  // ... a factor 4
#pragma unroll
        for (int v = 0; v < 2; ++v) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int shift = (k & 1) ? 1 : 4;
                out.op[8 * v + 2 * k] = pack_s16(shift * iq[16 * v + k], shift * iq[16 * v + 4 + k]);
                out.op[8 * v + 2 * k + 1] = pack_s16(shift * iq[16 * v + 8 + k], shift * iq[16 * v + 12 + k]);
            }
        }
    }
}

// Geometry of a record staged in shared memory: codes [P][kCode], scales [P][kGroups], offsets [P][kGroups], alpha [P].
template <int BITS, int GROUP, int P, int D>
struct StagedRecord {
    static_assert((BITS == 2 || BITS == 4) && (GROUP == 16 || GROUP == 32), "INT2/INT4 codes, groups of 16 or 32");
    static constexpr int kCode = D * BITS / 8, kGroups = D / GROUP;
    static constexpr int kLaneBytes = 4 * BITS;  // bytes of codes per 32-channel slice
    static constexpr int kAlphaAt = P * (kCode + 2 * kGroups);
    static constexpr int kBytes = kAlphaAt;      // without the alpha column
};

// (scale, offset) of the slice's group(s) of token t: one pair for 32-channel groups, two for 16-channel groups.
template <int BITS, int GROUP, int P, int D>
__device__ __forceinline__ void load_parameters(uint32_t base, int t, int js, float2& scales, float2& offsets) {
    using R = StagedRecord<BITS, GROUP, P, D>;
    const uint32_t meta = base + P * R::kCode + t * R::kGroups;
    if (GROUP == 32) {
        const float2 so = fp8x2_to_float2(prmt(lds8(meta + js), lds8(meta + P * R::kGroups + js), 0x0040u));
        scales = make_float2(so.x, so.x);
        offsets = make_float2(so.y, so.y);
    } else {
        scales = fp8x2_to_float2(lds16(meta + 2 * js));
        offsets = fp8x2_to_float2(lds16(meta + P * R::kGroups + 2 * js));
    }
}

// sum over the slice of q[c] * (code[c] * scale + offset) for token t of one record.
template <int BITS, int GROUP, int P, int D>
__device__ __forceinline__ float score_record(uint32_t base, int t, int js, const QueryOperands<BITS>& q) {
    using R = StagedRecord<BITS, GROUP, P, D>;
    int d0 = 0, d1 = 0;  // integer dot products over channels 0..15 / 16..31 of the slice
    if (BITS == 4) {
        const uint4 codes = lds128(base + t * R::kCode + 16 * js);
        const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t odd = words[w] & 0xF0F0F0F0u;
            int& d = w < 2 ? d0 : d1;
            d = dp2a_lo(q.op[4 * w + 0], words[w], d);
            d = dp2a_hi(q.op[4 * w + 1], words[w], d);
            d = dp2a_lo(q.op[4 * w + 2], odd, d);
            d = dp2a_hi(q.op[4 * w + 3], odd, d);
        }
    } else {
        const uint2 codes = lds64(base + t * R::kCode + 8 * js);
        int h0 = 0, h1 = 0;  // sums of code positions 2 and 3: they carry an extra factor 16
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t m0 = codes.x & (0x03030303u << (2 * k)), m1 = codes.y & (0x03030303u << (2 * k));
            int& s0 = k < 2 ? d0 : h0;
            int& s1 = k < 2 ? d1 : h1;
            s0 = dp2a_lo(q.op[2 * k], m0, s0);
            s0 = dp2a_hi(q.op[2 * k + 1], m0, s0);
            s1 = dp2a_lo(q.op[8 + 2 * k], m1, s1);
            s1 = dp2a_hi(q.op[8 + 2 * k + 1], m1, s1);
        }
        if (GROUP == 32) {
            d0 += (h0 + h1) >> 4;  // exact: a multiple of 16
        } else {
            d0 += h0 >> 4;
            d1 += h1 >> 4;
        }
    }
    float2 scales, offsets;
    load_parameters<BITS, GROUP, P, D>(base, t, js, scales, offsets);
    if (GROUP == 32)
        return scales.x * (static_cast<float>(d0 + d1) * q.dot_unit) + offsets.x * (q.sum0 + q.sum1);
    return scales.x * (static_cast<float>(d0) * q.dot_unit) + offsets.x * q.sum0 +
           scales.y * (static_cast<float>(d1) * q.dot_unit) + offsets.y * q.sum1;
}

// acc += weight * (code * scale + offset) over the slice for token t of one record: the code part goes into the half2
// sums (pair 4b+i = channels 8b+i and 8b+i+4 of the slice), the offset part into one fp32 sum per 16 channels.
// GUARDED (the last, partial page of a sequence): a token beyond the history has weight zero, but its bytes were never
// written and may decode to NaN or infinity, so its parameters are replaced by zeros instead of being multiplied by zero.
template <int BITS, int GROUP, int P, int D, bool TWO_OFFSETS, bool GUARDED = false>
__device__ __forceinline__ void accumulate_record(uint32_t base, int t, int js, float weight, uint32_t (&acc_b)[16],
                                                  float& acc_off0, float& acc_off1, bool live = true) {
    using R = StagedRecord<BITS, GROUP, P, D>;
    float2 scales, offsets;
    load_parameters<BITS, GROUP, P, D>(base, t, js, scales, offsets);
    if (GUARDED && !live) {
        scales = make_float2(0.f, 0.f);
        offsets = make_float2(0.f, 0.f);
        weight = 0.f;
    }
    acc_off0 += weight * offsets.x;
    if (TWO_OFFSETS) acc_off1 += weight * offsets.y;
    if (BITS == 4) {
        const uint4 codes = lds128(base + t * R::kCode + 16 * js);
        const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
        uint32_t w_low = 0, w_high = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            if (w == 0 || (w == 2 && GROUP == 16)) {
                w_low = half2_from(weight * (w == 0 ? scales.x : scales.y));
                w_high = hmul2_raw(w_low, 0x2C002C00u);  // w/16, exact
            }
            const uint32_t upper = words[w] >> 8;
            acc_b[4 * w + 0] = hfma2_raw(words[w] & 0x000F000Fu, w_low, acc_b[4 * w + 0]);
            acc_b[4 * w + 1] = hfma2_raw(words[w] & 0x00F000F0u, w_high, acc_b[4 * w + 1]);
            acc_b[4 * w + 2] = hfma2_raw(upper & 0x000F000Fu, w_low, acc_b[4 * w + 2]);
            acc_b[4 * w + 3] = hfma2_raw(upper & 0x00F000F0u, w_high, acc_b[4 * w + 3]);
        }
    } else {
        const uint2 codes = lds64(base + t * R::kCode + 8 * js);
        const uint32_t quarter = 0x34003400u, sixteenth = 0x2C002C00u, sixtyfourth = 0x24002400u;  // half2
        const uint32_t words[2] = {codes.x, codes.y};
        uint32_t wk[4];  // weights for code positions 0..3 of a byte: w, w/4, w/16, w/64
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            if (v == 0 || GROUP == 16) {
                wk[0] = half2_from(weight * (v == 0 ? scales.x : scales.y));
                wk[1] = hmul2_raw(wk[0], quarter);  // exact: powers of two
                wk[2] = hmul2_raw(wk[0], sixteenth);
                wk[3] = hmul2_raw(wk[0], sixtyfourth);
            }
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const uint32_t tb = prmt(words[v], 0u, b == 0 ? 0x4140u : 0x4342u);  // bytes [2b, 0, 2b+1, 0]
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    acc_b[8 * v + 4 * b + k] = hfma2_raw(tb & (0x00030003u << (2 * k)), wk[k], acc_b[8 * v + 4 * b + k]);
            }
        }
    }
}

// Dense learned key rotation: this warp's share of q @ R[head] for the CTA's query row -- k in [warp D/4, (warp + 1) D/4),
// lane L owning output channels 4L .. 4L+3 -- into parts[warp][D].  bf16 query entries times fp16 matrix entries are
// exact in binary32 and the sums are binary32, like the reference's TF32 product with fp32 accumulation
// (plugins/residual_quantization/csrc/attention/prepare.cuh:61-145); only the order of the sum differs.  A row of R[head]
// is D contiguous halves, so each of the D/4 loads of a warp is one coalesced 2D-byte line from L2 (every CTA of the
// head reads the same matrix); no separate rotation launch, no scratch.
template <int D>
__device__ __forceinline__ void rotate_query_dense(const AttentionParams& p, int row, int head, float* parts) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kShare = D / kWarps;   // 32 or 24 values of k per warp
    const __nv_bfloat16* q = p.query + static_cast<int64_t>(row) * p.query_stride + head * D + warp * kShare;
    const float mine = lane < kShare ? __bfloat162float(q[lane]) : 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool owner = 4 * lane < D;
    const __half* r = p.query_matrix + (static_cast<int64_t>(head) * D + warp * kShare) * D + (owner ? 4 * lane : 0);
#pragma unroll 8
    for (int k = 0; k < kShare; ++k) {
        const float qk = __shfl_sync(kFullMask, mine, k);   // every lane takes part in the shuffle
        if (owner) {
            const uint2 packed = __ldg(reinterpret_cast<const uint2*>(r + k * D));
            const float2 lo = __half22float2(as_half2(packed.x)), hi = __half22float2(as_half2(packed.y));
            acc[0] += qk * lo.x; acc[1] += qk * lo.y; acc[2] += qk * hi.x; acc[3] += qk * hi.y;
        }
    }
    if (owner) *reinterpret_cast<float4*>(parts + warp * D + 4 * lane) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

// Rotated, pre-scaled query of this (row, head) into shared memory: qs[c] = (q @ R)[c] * D^-1/2 * log2(e).
// Executed by warp 0; lane L owns channels 4L .. 4L+3.
// Also computes the score of the live token (its K row is the raw bf16 input, original coordinates):
// live = q.k * D^-1/2 * log2(e) - sum_c qs[c] * mean[loop][c]; the history scores leave out the same q.mean[loop]
// constant (reference: prepare.cuh:229).
// `dense_parts`: with a dense key rotation, the four warps' partial sums of q @ R (float [kWarps][D], see
// rotate_query_dense) that this warp adds up.
template <int D, bool MEAN>
__device__ __forceinline__ void prepare_query(const AttentionParams& p, int row, int head, float* qs, float* qmax_out,
                                              float* live_out, const float* dense_parts) {
    const int lane = threadIdx.x & 31;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    float live_dot = 0.f;
    const bool owner = 4 * lane < D;
    if (owner) {
        const __nv_bfloat16* q = p.query + static_cast<int64_t>(row) * p.query_stride + head * D + 4 * lane;
        const __nv_bfloat16* k = p.key + static_cast<int64_t>(row) * p.key_stride + head * D + 4 * lane;
        const uint2 raw = *reinterpret_cast<const uint2*>(q);
        const uint2 live = *reinterpret_cast<const uint2*>(k);
        x[0] = bf16_bits_to_float(raw.x & 0xffffu);
        x[1] = bf16_bits_to_float(raw.x >> 16);
        x[2] = bf16_bits_to_float(raw.y & 0xffffu);
        x[3] = bf16_bits_to_float(raw.y >> 16);
        live_dot = x[0] * bf16_bits_to_float(live.x & 0xffffu) + x[1] * bf16_bits_to_float(live.x >> 16) +
                   x[2] * bf16_bits_to_float(live.y & 0xffffu) + x[3] * bf16_bits_to_float(live.y >> 16);
    }
    float scale = rsqrtf(static_cast<float>(D)) * kLog2e;
    if (p.query_matrix != nullptr) {
        // dense learned rotation: the CTA's warps each summed a quarter of the k range
        if (owner) {
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float4 v = *reinterpret_cast<const float4*>(dense_parts + w * D + 4 * lane);
                x[0] += v.x; x[1] += v.y; x[2] += v.z; x[3] += v.w;
            }
        }
    } else if (p.key_sign != nullptr) {
        if (owner) {
            const uint32_t sign = p.key_sign[head * (D / 32) + (lane >> 3)] >> (4 * (lane & 7));
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if ((sign >> i) & 1u) x[i] = -x[i];
        }
        butterflies_in_lane<4>(x);
        butterfly_across_lanes<4>(x, 1, (lane & 1) != 0);
        if (D == 128) {
            butterfly_across_lanes<4>(x, 2, (lane & 2) != 0);
            butterfly_across_lanes<4>(x, 4, (lane & 4) != 0);
            butterfly_across_lanes<4>(x, 8, (lane & 8) != 0);
            butterfly_across_lanes<4>(x, 16, (lane & 16) != 0);
        } else {
            const uint32_t mask = kPaleyColA[(lane >> 1) & 15];
            float out[4];
#pragma unroll
            for (int a = 0; a < 12; ++a) {
                const bool negative = (mask >> a) & 1u;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float v = __shfl_sync(kFullMask, x[i], 2 * a + (lane & 1));
                    const float t = negative ? -v : v;
                    out[i] = a == 0 ? t : out[i] + t;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] = out[i];
        }
        scale *= p.key_rscale;
    }
    float biggest = 0.f, shift = 0.f;
    if (owner) {
        float mean[4] = {0.f, 0.f, 0.f, 0.f};
        if (MEAN) {
            const float4 v = *reinterpret_cast<const float4*>(
                p.mean + (static_cast<int64_t>(p.loop_index) * p.heads + head) * D + 4 * lane);
            mean[0] = v.x; mean[1] = v.y; mean[2] = v.z; mean[3] = v.w;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float v = x[i] * scale;
            qs[4 * lane + i] = v;
            biggest = fmaxf(biggest, fabsf(v));
            shift += v * mean[i];
        }
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        biggest = fmaxf(biggest, __shfl_xor_sync(kFullMask, biggest, d));
        live_dot += __shfl_xor_sync(kFullMask, live_dot, d);
        if (MEAN) shift += __shfl_xor_sync(kFullMask, shift, d);
    }
    if (lane == 0) {
        *qmax_out = biggest;
        *live_out = live_dot * rsqrtf(static_cast<float>(D)) * kLog2e - shift;
    }
}

// Undo an explicit value rotation on the history sum: h <- ((h H^T) * rscale) * sign.  Warp 0, in place in smem.
template <int D>
__device__ __forceinline__ void unrotate_history(const AttentionParams& p, int head, float* hist) {
    const int lane = threadIdx.x & 31;
    const bool owner = 4 * lane < D;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (owner) {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = hist[4 * lane + i];
    }
    butterflies_in_lane<4>(x);
    butterfly_across_lanes<4>(x, 1, (lane & 1) != 0);
    if (D == 128) {
        butterfly_across_lanes<4>(x, 2, (lane & 2) != 0);
        butterfly_across_lanes<4>(x, 4, (lane & 4) != 0);
        butterfly_across_lanes<4>(x, 8, (lane & 8) != 0);
        butterfly_across_lanes<4>(x, 16, (lane & 16) != 0);
    } else {
        const uint32_t mask = kPaleyRowA[(lane >> 1) & 15];
        float out[4];
#pragma unroll
        for (int a = 0; a < 12; ++a) {
            const bool negative = (mask >> a) & 1u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float v = __shfl_sync(kFullMask, x[i], 2 * a + (lane & 1));
                const float t = negative ? -v : v;
                out[i] = a == 0 ? t : out[i] + t;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = out[i];
    }
    if (owner) {
        const uint32_t sign = p.value_sign[head * (D / 32) + (lane >> 3)] >> (4 * (lane & 7));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float v = x[i] * p.value_rscale;
            hist[4 * lane + i] = ((sign >> i) & 1u) ? -v : v;
        }
    }
}

// ---- phase timestamps (build flag RQ_ATTENTION_TIMELINE=1; compiled out otherwise) ---------------------------
// Where a small call's time goes cannot be read off a profiler's per-kernel counters: it is a chain of latencies inside
// each CTA.  In a timeline build thread 0 of every CTA records clock64() at the phase boundaries below (and the global
// timer at entry and exit) into a device array that rq_timeline_d128 / rq_timeline_d96 copy out; launches alternate
// between two halves of the array by loop_index & 1, so that two consecutive launches can be laid side by side.
// `python -m residualquant_b200.timeline` drives it.  The regular build has no trace of it.
#ifndef RQ_ATTENTION_TIMELINE
#define RQ_ATTENTION_TIMELINE 0
#endif
enum TimelineSlot {
    kAtEntryGlobalNs = 0, kAtEntry, kAfterLookup, kAfterStaging, kAfterWait, kAfterQuery, kAfterPages, kAfterWarpFold,
    kAfterTicket, kAfterPartitions, kAtExit, kAtExitGlobalNs, kLookupLoadsIssued, kLookupLoadsArrived, kLookupChosen,
    kQueryRotated, kQueryShared, kSmId, kTimelineSlots
};
constexpr int kTimelineCtas = 4096;
#if RQ_ATTENTION_TIMELINE
__device__ unsigned long long g_timeline[2][kTimelineCtas][kTimelineSlots];
#define RQ_STAMP(slot)                                                                               \
    do {                                                                                             \
        if (threadIdx.x == 0 && blockIdx.x < kTimelineCtas) g_timeline[p.loop_index & 1][blockIdx.x][slot] = clock64(); \
    } while (0)
#define RQ_STAMP_GLOBAL(slot)                                                                        \
    do {                                                                                             \
        if (threadIdx.x == 0 && blockIdx.x < kTimelineCtas) {                                        \
            unsigned long long now_ns;                                                               \
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now_ns));                                \
            g_timeline[p.loop_index & 1][blockIdx.x][slot] = now_ns;                                 \
        }                                                                                            \
    } while (0)
#else
#define RQ_STAMP(slot) do {} while (0)
#define RQ_STAMP_GLOBAL(slot) do {} while (0)
#endif

// ---- work decomposition ------------------------------------------------------------------------------------
// A work item is one KV partition of one query row (all heads of it: the CTA index is item * heads + head).
struct WorkItem {
    int row, request, seq_len;
    int part, parts;  // this CTA's partition of the row and how many the row has
    int first;        // index of the row's first work item: partial results of the row sit at items first .. first+parts-1
};

// Cost of running `items` equally sized CTAs per head, in units of (pages one CTA consumes while four share an SM):
// full waves of `slots` CTAs plus a tail wave in which an SM holding 1/2/3/4 CTAs delivers 0.45/0.85/0.92/1 of its
// throughput (fitted to measurements on B200: the kernel is bound by instruction issue).
// (a + b - 1) / b for 0 <= a < 2^21, 0 < b: the quotient of the approximate division is within 2 ulp, far inside the
// half-unit margin that a + 0.5 leaves on either side of an integer.  An integer division costs a few hundred cycles of
// dependent instructions, and the work lookup sits in front of everything a CTA does.
__device__ __forceinline__ int ceil_div_small(int a, int b) {
    return static_cast<int>(__fdividef(static_cast<float>(a + b - 1) + 0.5f, static_cast<float>(b)));
}

__device__ __forceinline__ float wave_count(float ctas, float slots, float sms) {
    const float full = floorf(__fdividef(ctas + 0.5f, slots));   // ctas and slots are integers
    const float rest = ctas - full * slots;
    const int per_sm = static_cast<int>(ceilf(__fdividef(rest - 0.5f, sms)));
    const float tail = per_sm <= 0 ? 0.f : per_sm == 1 ? 1.f / 0.45f : per_sm == 2 ? 2.f / 0.85f : per_sm == 3 ? 3.f / 0.92f : 4.f;
    return full + 0.25f * tail;
}

// Maps a work-item index to (row, partition).  Replaces the reference's prepare_partition_schedule
// (plugins/residual_quantization/csrc/attention/prepare.cuh:237-386), which a single CTA of a separate kernel runs
// and parks in a work list; here every CTA derives the same answer from the sequence lengths in a few warp-wide
// steps, so there is no extra launch and no list to read back.
//   * p.splits > 0 (forced): every row has exactly p.splits partitions.
//   * p.splits < 0: as below with the chunk size fixed by the caller to -p.splits pages (a tuning knob).
//   * p.splits == 0: one chunk size c (pages) is chosen for the whole call from the TOTAL number of pages of the batch,
//     row r gets max(1, ceil(pages_r / c)) partitions -- proportional to its length -- and the items are laid out
//     request by request.  c is the candidate (4, 8, ..., 1024 pages, or "never split"; for a batch of equal lengths:
//     the row cut into 1..32 equal partitions) with the lowest modelled time among those whose item count fits
//     p.capacity, which fixed the grid on the host.
// Every lane of the warp calls this with the same arguments and gets the same result.  Metadata is read through L2
// (ld.global.cg): with early_start this runs while the previous kernel of the stream may still be executing, and an L1
// line left over from an earlier launch must not be trusted.
template <int P>
__device__ __forceinline__ bool find_work(const AttentionParams& p, int item, int lane, WorkItem& out) {
    const int num_requests = p.num_requests;
    const int total_rows = min(__ldcg(p.query_start_loc + num_requests), p.num_rows);
    if (p.splits > 0) {
        const int row = item / p.splits;
        if (row >= total_rows) return false;
        // Decode batches have one row per request, so request == row is the guess; it is re-read only if wrong.
        int request = min(row, num_requests - 1);
        const int guess_begin = __ldcg(p.query_start_loc + request), guess_end = __ldcg(p.query_start_loc + request + 1);
        int seq_len = __ldcg(p.seq_lens + request);
        if (!(guess_begin <= row && row < guess_end)) {
            int lo = 0, hi = num_requests - 1;  // largest r with query_start_loc[r] <= row
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (__ldcg(p.query_start_loc + mid) <= row) lo = mid; else hi = mid - 1;
            }
            request = lo;
            seq_len = __ldcg(p.seq_lens + request);
        }
        out.row = row;
        out.request = request;
        out.seq_len = seq_len;
        out.parts = p.splits;
        out.part = item - row * p.splits;
        out.first = row * p.splits;
        return true;
    }
    if (item >= p.capacity) return false;

    constexpr int kCandidates = 9;          // chunk sizes 4 << k pages, k = 0..8; candidate 9 = one partition per row
    constexpr float kOverhead = 256.f / P;  // fixed cost of a CTA (prologue, first fetch, fold), in pages
    // A sweep covers 64 requests: lane L holds request base + L and request base + 32 + L.  All six loads of a sweep
    // are independent, so a batch of up to 64 requests costs one round trip to L2, and its values stay in registers
    // for the second pass.
    struct Request { int begin, rows, pages, len; };
    auto load_sweep = [&](int base, Request (&q)[2]) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int r = base + 32 * u + lane;
            q[u].begin = q[u].rows = q[u].pages = q[u].len = 0;
            if (r < num_requests) {
                q[u].len = __ldcg(p.seq_lens + r);
                q[u].begin = __ldcg(p.query_start_loc + r);
                q[u].rows = max(0, min(__ldcg(p.query_start_loc + r + 1), total_rows) - q[u].begin);
                q[u].pages = q[u].rows > 0 ? (max(q[u].len - 1, 0) + P - 1) / P : 0;
            }
        }
    };
    // pass 1: pages of the whole batch, and how many items each candidate chunk size would make
    Request first[2];
    load_sweep(0, first);
    int total_pages = 0, longest = 0, shortest = 0x7fffffff;
    int counts[kCandidates];
#pragma unroll
    for (int k = 0; k < kCandidates; ++k) counts[k] = 0;
    auto tally = [&](const Request (&q)[2]) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            total_pages += q[u].rows * q[u].pages;
            longest = max(longest, q[u].pages);
            if (q[u].rows > 0) shortest = min(shortest, q[u].pages);
#pragma unroll
            for (int k = 0; k < kCandidates; ++k) counts[k] += q[u].rows * max(1, (q[u].pages + (4 << k) - 1) >> (k + 2));
        }
    };
    RQ_STAMP(kLookupLoadsIssued);
#if RQ_ATTENTION_TIMELINE
    if (first[0].len + first[1].len + total_rows == -12345) return false;   // a use of the loaded values: they have arrived
#endif
    RQ_STAMP(kLookupLoadsArrived);
    tally(first);
    for (int base = 64; base < num_requests; base += 64) {
        Request more[2];
        load_sweep(base, more);
        tally(more);
    }
    total_pages = __reduce_add_sync(kFullMask, total_pages);
    // No chunk is smaller than four pages, so the call never has more than rows + pages / 4 items: the spare CTAs
    // beyond that leave here, before the partition choice.
    if (item >= total_rows + (total_pages >> 2) && p.splits == 0) return false;
    longest = __reduce_max_sync(kFullMask, longest);
    shortest = __reduce_min_sync(kFullMask, shortest);
    const float sms = static_cast<float>(p.sm_count), slots = sms * 4.f;  // four CTAs of this kernel fit on an SM
    // modelled time of `items` items per head whose largest spans `largest` pages
    auto cost_of = [&](int items_in, float largest) {
        const float items = static_cast<float>(max(items_in, 1));
        const float cost = wave_count(items * p.heads, slots, sms) * (__fdividef(static_cast<float>(total_pages), items) + kOverhead);
        return fmaxf(cost, (0.25f / 0.45f) * (largest + kOverhead));  // the largest item alone on an SM is the floor
    };
    int chunk;
    if (shortest == longest) {
        // Every row spans the same number of pages (a decode batch of equal lengths, one request): the item count of a
        // chunk size needs no sum over the requests, so every lane tries its own partition count 1..32.
        const int mine = max(4, ceil_div_small(longest, lane + 1));
        const int parts = max(1, ceil_div_small(longest, mine));
        float cost = cost_of(total_rows * parts, static_cast<float>(min(mine, longest)));
        cost *= 1.f + 0.04f * __log2f(static_cast<float>(parts));  // near ties go to fewer partitions (measured: they win them)
        uint32_t key = (__float_as_uint(cost) & ~31u) | static_cast<uint32_t>(lane);
        if (total_rows * parts > p.capacity && lane > 0) key = 0xffffffffu;  // does not fit the grid (one partition always does)
        const int chosen = static_cast<int>(__reduce_min_sync(kFullMask, key) & 31u);
        chunk = max(4, __shfl_sync(kFullMask, mine, chosen));
    } else {
        int my_items = total_rows;  // lanes >= kCandidates stand for "never split"
#pragma unroll
        for (int k = 0; k < kCandidates; ++k) {
            const int sum = __reduce_add_sync(kFullMask, counts[k]);
            if (lane == k) my_items = sum;
        }
        const int candidate = min(lane, kCandidates);
        const float largest = candidate < kCandidates ? fminf(static_cast<float>(4 << candidate), static_cast<float>(longest))
                                                      : static_cast<float>(longest);
        float cost = cost_of(my_items, largest);
        cost *= 1.f + 0.01f * static_cast<float>(kCandidates - candidate);  // near ties go to fewer partitions
        uint32_t key = (__float_as_uint(cost) & ~15u) | static_cast<uint32_t>(kCandidates - candidate);
        if (my_items > p.capacity) key = 0xffffffffu;  // does not fit the grid ("never split" always does)
        const int chosen = kCandidates - static_cast<int>(__reduce_min_sync(kFullMask, key) & 15u);
        chunk = chosen < kCandidates ? 4 << chosen : 0x40000000;  // pages; "never split" = larger than any row
    }
    if (p.splits < 0) {
        // the caller fixed the chunk size (pages); it still has to fit the capacity: sum ceil(pages / c) <= T / c + rows
        const int spare = max(1, p.capacity - total_rows);
        chunk = max(-p.splits, (total_pages + spare - 1) / spare);
    }
#if RQ_ATTENTION_TIMELINE
    if (chunk == -777) return false;   // a use of the choice
#endif
    RQ_STAMP(kLookupChosen);
    auto parts_of = [&](int pages) { return max(1, (pages + chunk - 1) / chunk); };

    // pass 2: which request owns this item.  Requests are numbered sweep by sweep, first half (lanes 0..31) then second.
    int before = 0;
    for (int base = 0; base < num_requests; base += 64) {
        Request q[2];
        if (base == 0) { q[0] = first[0]; q[1] = first[1]; } else load_sweep(base, q);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int parts = parts_of(q[u].pages);
            const int mine = q[u].rows * parts;
            int upto = mine;  // inclusive prefix sum over the lanes
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int v = __shfl_up_sync(kFullMask, upto, d);
                if (lane >= d) upto += v;
            }
            const uint32_t owners = __ballot_sync(kFullMask, item < before + upto);
            if (owners != 0u) {
                const int src = __ffs(owners) - 1;
                const int local = item - before - (__shfl_sync(kFullMask, upto, src) - __shfl_sync(kFullMask, mine, src));
                const int owner_parts = __shfl_sync(kFullMask, parts, src);
                const int row_in_request = owner_parts == 1 ? local : local / owner_parts;
                out.request = base + 32 * u + src;
                out.seq_len = __shfl_sync(kFullMask, q[u].len, src);
                out.row = __shfl_sync(kFullMask, q[u].begin, src) + row_in_request;
                out.parts = owner_parts;
                out.part = local - row_in_request * owner_parts;
                out.first = item - out.part;
                return true;
            }
            before += __shfl_sync(kFullMask, upto, 31);
        }
    }
    return false;
}

// Wait until peer `peer` has published epoch `target` (one epoch per completed call).  Bounded by the GPU's global timer
// and a poll count; on expiry the status word of the state block is raised and the call goes on.
__device__ __forceinline__ void wait_for_peers(const AttentionParams& p, int peer, uint32_t target) {
    const uint32_t* arrival = p.gather_flags[p.gather_rank] + peer;
    unsigned long long start = 0;
    for (uint32_t polls = 0;; ++polls) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(arrival) : "memory");
        if (static_cast<int32_t>(seen - target) >= 0) return;  // a fast peer may already be a call ahead
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (polls == 0) start = now;
        if (polls > 64) __nanosleep(100);
        if (polls > (1u << 26) || now - start > p.gather_timeout_ns) {
            atomicExch(p.gather_state + 1, static_cast<uint32_t>(RQ_ERR_DEVICE_TIMEOUT));
            return;
        }
    }
}

template <class C>
__global__ void __launch_bounds__(kThreads, C::kMinBlocks) attention_kernel(const __grid_constant__ AttentionParams p) {
    constexpr int D = C::D, P = C::P;
    constexpr int kFlushPages = 64 / P;   // a lane adds 8 tokens between flushes
    constexpr float kSlack = 1.f;         // probabilities stay below 2
    extern __shared__ __align__(128) uint8_t smem[];
    float* qs = reinterpret_cast<float*>(smem + C::kOffQuery);
    float* warp_acc = reinterpret_cast<float*>(smem + C::kOffWarpAcc);
    float* warp_stat = reinterpret_cast<float*>(smem + C::kOffWarpStat);  // [w][2] then misc at [8..15]
    uint64_t* barriers = reinterpret_cast<uint64_t*>(smem + C::kOffBarriers);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int heads = p.heads;
    const int head = blockIdx.x % heads;

    // Nothing is read before the previous kernel of the stream has completed -- unless the caller vouched for the
    // metadata and the cache pages (early_start): then only the q/k/v rows wait, further down.  Once the wait is over
    // the NEXT kernel of the stream may be scheduled (it waits for this grid's completion in the same way); not
    // earlier, so that at most two kernels of a stream are ever in flight together.
    const bool early_start = p.early_start != 0;
#if RQ_ATTENTION_TIMELINE
    if (threadIdx.x == 0 && blockIdx.x < kTimelineCtas)
        for (int i = 0; i < kTimelineSlots; ++i) g_timeline[p.loop_index & 1][blockIdx.x][i] = 0ull;
#endif
    RQ_STAMP_GLOBAL(kAtEntryGlobalNs);
#if RQ_ATTENTION_TIMELINE
    if (threadIdx.x == 0 && blockIdx.x < kTimelineCtas) {
        uint32_t sm;
        asm volatile("mov.u32 %0, %smid;" : "=r"(sm));
        g_timeline[p.loop_index & 1][blockIdx.x][kSmId] = sm + 1u;   // which SM the CTA ran on (+1: 0 means not launched)
    }
#endif
    if (!early_start) {
        pdl_wait();
        pdl_launch_dependents();
    }
    RQ_STAMP(kAtEntry);   // without the early start: after the wait, so that the phases below are the kernel's own time

    // ---- which work item: (row, partition) and the row's request ---------------------------------------
    // Warp 0 looks it up (the lookup is warp-wide work that every warp would repeat) and shares the answer.
    WorkItem* shared_work = reinterpret_cast<WorkItem*>(smem + C::kOffWork);
    if (warp == 0) {
        WorkItem mine;
        if (!find_work<P>(p, blockIdx.x / heads, lane, mine)) mine.row = -1;  // graph padding or spare capacity
        if (lane == 0) *shared_work = mine;
    }
    __syncthreads();
    const WorkItem work = *shared_work;
    RQ_STAMP(kAfterLookup);
    if (work.row < 0) return;  // nothing to do
    const int row = work.row, request = work.request, split = work.part, splits = work.parts;
    const int history = max(0, work.seq_len - 1);
    const int pages = (history + P - 1) / P;
    const int chunk = (pages + splits - 1) / splits;
    const int page_begin = min(pages, split * chunk), page_end = min(pages, page_begin + chunk);
    // pages of this warp: page_begin + warp, + kWarps, ...
    const int warp_pages = page_begin + warp < page_end ? (page_end - page_begin - warp + kWarps - 1) / kWarps : 0;
    const int32_t* table = p.block_table + static_cast<int64_t>(request) * p.block_table_stride;

    // ---- per-warp ring: init barriers, start the first copies ----------------------------------------
    uint8_t* ring = smem + C::kOffRing + warp * C::kRingBytes;
    const uint32_t ring_addr = smem_addr(ring);
    const uint32_t bar_addr = smem_addr(barriers + warp * C::kStages);
    if (kBulkCopy) {
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < C::kStages; ++s) mbar_init(bar_addr + 8 * s, 1);
            fence_proxy_async();
        }
        __syncwarp();
    }

    const int64_t page_bytes = static_cast<int64_t>(P) * p.page_width;
    const uint8_t* head_base = p.cache + head * page_bytes;
    const int64_t block_bytes = heads * page_bytes;
    const int anchor_at = P * p.anchor_offset, residual_at = P * p.residual_offset;
    const uint32_t lane_anchor_at = anchor_at + 16 * lane, lane_residual_at = residual_at + 16 * lane;
    const uint32_t lane_ring = ring_addr + 16 * lane;
    auto issue = [&](int block, int stage) {
        const uint8_t* k_page = head_base + block * block_bytes;
        const uint8_t* v_page = k_page + p.plane_stride;
        const uint32_t dst = ring_addr + stage * C::kStageBytes;
        if (C::kAdjacent) {
            const int prefix = P * p.chain_offset[p.chain_count];
            warp_copy_bytes(dst, k_page, prefix, lane);
            warp_copy_bytes(dst + C::kMaxPrefixBytes, v_page, prefix, lane);
        } else if (kBulkCopy) {
            if (lane == 0) {
                const uint32_t bar = bar_addr + 8 * stage;
                fence_proxy_async();
                mbar_expect_tx(bar, C::kStageBytes);
                bulk_load(dst, k_page + anchor_at, C::kAnchorBytes, bar);
                if (C::kResidual) bulk_load(dst + C::kAnchorBytes, k_page + residual_at, C::kResidualBytes, bar);
                bulk_load(dst + C::kPlaneBytes, v_page + anchor_at, C::kAnchorBytes, bar);
                if (C::kResidual)
                    bulk_load(dst + C::kPlaneBytes + C::kAnchorBytes, v_page + residual_at, C::kResidualBytes, bar);
            }
        } else {
            // two source pointers per plane (the lane's first chunk of each region), everything else is an immediate
            const uint32_t to = lane_ring + stage * C::kStageBytes;
            const uint8_t* k_from = k_page + lane_anchor_at;
            warp_copy<C::kAnchorBytes>(to, k_from, lane);
            warp_copy<C::kAnchorBytes>(to + C::kPlaneBytes, k_from + p.plane_stride, lane);
            if (C::kResidual) {
                const uint8_t* r_from = k_page + lane_residual_at;
                warp_copy<C::kResidualBytes>(to + C::kAnchorBytes, r_from, lane);
                warp_copy<C::kResidualBytes>(to + C::kPlaneBytes + C::kAnchorBytes, r_from + p.plane_stride, lane);
            }
        }
    };
    // block ids of this warp's next 32 pages, one per lane
    int batch_base = 0;
    int my_block = 0;
    auto load_batch = [&](int base) {
        batch_base = base;
        my_block = base + lane < warp_pages ? __ldcg(table + page_begin + warp + kWarps * (base + lane)) : 0;
    };
    load_batch(0);
    int issued = 0;
    {
        // commit-group bookkeeping wants exactly kStages groups here and one more per loop iteration
#pragma unroll
        for (int s = 0; s < C::kStages; ++s) {
            if (s < warp_pages) {
                const int block = __shfl_sync(kFullMask, my_block, s);
                issue(block, s);
                ++issued;
            }
            if (!kBulkCopy) cp_async_commit();
        }
    }

    RQ_STAMP(kAfterStaging);
    if (early_start) {
        pdl_wait();  // the q/k/v rows usually ARE the previous kernel's output
        pdl_launch_dependents();
    }
    RQ_STAMP(kAfterWait);
    // Head-sharded serving: q depends, through the output projection, on the gathered rows of the previous call, so this
    // is where the call waits for every peer's stores of that call (bounded; ordered before the barrier below).
    if (p.gather_wait && warp == 1 && lane < p.num_peers) wait_for_peers(p, lane, __ldcg(p.gather_state));

    // ---- query: rotate + scale (warp 0), then every lane takes its 32-channel slice -------------------
    float* misc = warp_stat + 8;         // [0] last-arrival flag, [1] live score, [2] max |q|
    if (p.query_matrix != nullptr) {
        rotate_query_dense<D>(p, row, head, warp_acc);   // all four warps; warp_acc is free until the warp fold
        __syncthreads();
    }
    if (warp == 0) prepare_query<D, C::kMean>(p, row, head, qs, misc + 2, misc + 1, warp_acc);
    RQ_STAMP(kQueryRotated);
    if (warp == 1 && lane < D / 64) {
        // the live token's V row is read at the very end of the CTA: have it in L2 by then
        const __nv_bfloat16* v_row = p.value + static_cast<int64_t>(row) * p.value_stride + head * D + 64 * lane;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(v_row));
    }
    __syncthreads();

    // The K side runs on integer dot products (dp2a: two s16 x u8 products per instruction) against a query slice
    // quantized once per CTA; see QueryOperands.
    // 4 lanes per token, 8 tokens per warp step.  At head_dim 96 the fourth lane of a token has no slice: it runs along
    // with zero operands.  (A 3-lanes-per-token variant that streams 10 tokens per step across page boundaries was
    // measured at the same speed: what it saves in idle lanes it spends on per-step address arithmetic that the
    // fixed token positions of this layout fold into immediate offsets.)
    RQ_STAMP(kQueryShared);
    const int j = lane & 3;              // slice: channels 32j .. 32j+31
    const bool slice_ok = 32 * j < D;
    const int js = slice_ok ? j : 0;     // lanes without a slice read slice 0 and contribute zero
    const float qmax = misc[2];
    constexpr bool kUse4 = C::kAdjacent || C::AB == 4 || C::RB == 4, kUse2 = C::kAdjacent || C::AB == 2 || C::RB == 2;
    QueryOperands<4> q4;
    QueryOperands<2> q2;
    if (kUse4) build_operands<4>(qs + 32 * js, slice_ok, qmax, q4);
    if (kUse2) build_operands<2>(qs + 32 * js, slice_ok, qmax, q2);
    auto operands = [&](auto bits_tag) -> const auto& {
        if constexpr (decltype(bits_tag)::value == 4) return q4; else return q2;
    };
    float chain_qmean[4] = {0.f, 0.f, 0.f, 0.f};  // adjacent mode: sum_c q[c] * mean[r][c] for the records before the loop's own
    if (C::kAdjacent && C::kMean && slice_ok) {
        const float* qslice = qs + 32 * js;
        for (int r = 0; r + 1 < p.chain_count; ++r) {
            const float* mean = p.mean + (static_cast<int64_t>(r) * heads + head) * D + 32 * js;
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 32; ++c) sum += qslice[c] * mean[c];
            chain_qmean[r] = sum;
        }
    }
    float qmean = 0.f;                   // sum_c q[c] * mean[anchor][c] over the slice (residual loops with a mean)
    if (!C::kAdjacent && C::kMean && C::kResidual && slice_ok) {
        const float* qslice = qs + 32 * js;
        const float* mean = p.mean + (static_cast<int64_t>(p.anchor_index) * heads + head) * D + 32 * js;
#pragma unroll
        for (int c = 0; c < 32; ++c) qmean += qslice[c] * mean[c];
    }

    RQ_STAMP(kAfterQuery);
    // ---- page loop -----------------------------------------------------------------------------------
    float m_biased = kNever, l = 0.f;  // online-softmax state of this lane's token slot (base-2 logits), see below
    uint32_t acc_b[16];                  // half2 partial sums of V, pair 4b+i = (channel 8b+i, channel 8b+i+4)
    float acc[32];
    constexpr bool kTwoOffsets = C::kAdjacent || C::AG == 16 || (C::kResidual && C::RG == 16);  // a record with two groups per slice
    float acc_off0 = 0.f, acc_off1 = 0.f;  // offset part of V for channels 0..15 / 16..31 of the slice (one sum if equal)
#pragma unroll
    for (int i = 0; i < 16; ++i) acc_b[i] = 0u;
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    bool failed = false;
    const int slot = lane >> 2;          // token slot 0..7 inside a warp step
    float carry = 1.f;                   // factor the fp32 sums still have to be multiplied by (deferred rescale)

    int pages_to_flush = kFlushPages;  // counts down; a token with more than half of its stream's mass so far zeroes it
    // half2 partial sums -> fp32 sums, every 8 tokens of a lane
    auto flush = [&]() {
        if (__any_sync(kFullMask, carry != 1.f)) {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] *= carry;
            carry = 1.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            add_half2_to_floats(acc_b[i], acc[2 * i], acc[2 * i + 1]);
            acc_b[i] = 0u;
        }
    };

    // One token of the lane's slot: score against the query slice, online softmax, value accumulation.
    // `k_anchor` = shared address of the staged page (stage) the token lives in, `t` = its index inside the page.
    [[maybe_unused]] constexpr int kResidualAlphaAt = P * (C::kResidualCode + 2 * C::kResidualGroups);
    // The scores of a page's token steps do not depend on the softmax state, so they are all computed first: the
    // integer dot products of the next step overlap the dependent softmax/value chain of the previous one.
    auto score_token = [&](uint32_t k_anchor, int t, bool live_token) -> float {
        [[maybe_unused]] const uint32_t k_residual = k_anchor + C::kAnchorBytes;
        {
            // ---------------- K: score of token t against the query slice (integer dot products) ----------------
            float part = 0.f;
            if constexpr (C::kAdjacent) {
                // K_hat[loop] = alpha_loop * K_hat[loop-1] + R_loop (+ means of the earlier loops): Horner over the records
                for (int r = 0; r < p.chain_count; ++r) {
                    const uint32_t base = k_anchor + P * p.chain_offset[r];
                    const int bits = p.chain_bits[r], group = p.chain_group[r];
                    float one;
                    if (bits == 4) one = score_record<4, 32, P, D>(base, t, js, q4);
                    else if (group == 32) one = score_record<2, 32, P, D>(base, t, js, q2);
                    else one = score_record<2, 16, P, D>(base, t, js, q2);
                    if (r > 0) {
                        const int alpha_at = P * (D * bits / 8 + 2 * (D / group));
                        part *= bf16_bits_to_float(lds16(base + alpha_at + 2 * t));
                    }
                    part += one + chain_qmean[r];
                }
            } else {
            part = score_record<C::AB, C::AG, P, D>(k_anchor, t, js, operands(std::integral_constant<int, C::AB>{}));
            }
            if constexpr (C::kResidual && !C::kAdjacent) {
                const float alpha = bf16_bits_to_float(lds16(k_residual + kResidualAlphaAt + 2 * t));
                if (C::kMean) part += qmean;
                part = part * alpha +
                       score_record<C::RB, C::RG, P, D>(k_residual, t, js, operands(std::integral_constant<int, C::RB>{}));
            }
            part += __shfl_xor_sync(kFullMask, part, 1);
            part += __shfl_xor_sync(kFullMask, part, 2);
            return live_token ? part : kNever;
        }
    };
    auto absorb_token = [&](auto partial_tag, uint32_t k_anchor, int t, bool live_token, float score) {
        constexpr bool kPartial = decltype(partial_tag)::value;
        const uint32_t v_anchor = k_anchor + (C::kAdjacent ? C::kMaxPrefixBytes : C::kPlaneBytes);
        [[maybe_unused]] const uint32_t v_residual = v_anchor + C::kAnchorBytes;
        {
            // ---------------- online softmax of the token slot ----------------
            // `m` is the stream's reference exponent, not its exact maximum: it only moves when a score exceeds it
            // by more than kSlack, so probabilities stay below 2^kSlack and rescaling is rare.
            // Inside the loop the exponent is kept as m - kWeightBits, so that exp2(score - m_biased) is the probability
            // already multiplied by 2^kWeightBits, the form the value weights need.
            // The rare rescale is taken by the whole warp (lanes that need none multiply by one): no divergence.
            const bool raise = score > m_biased + (kSlack + kWeightBits);
            if (__any_sync(kFullMask, raise)) {
                const float f = raise ? fast_exp2(m_biased + kWeightBits - score) : 1.f;  // a stream without tokens gives 0
                l *= f;
                acc_off0 *= f;
                if (kTwoOffsets) acc_off1 *= f;
                carry *= f;
                const uint32_t f2 = half2_from(f);
#pragma unroll
                for (int i = 0; i < 16; ++i) acc_b[i] = hmul2_raw(acc_b[i], f2);
                if (raise) m_biased = score - kWeightBits;
            }
            const float prob = live_token ? fast_exp2(score - m_biased) : 0.f;
            const float l_before = l;
            l += prob;

            // ---------------- V: accumulate prob * V_hat[t] over the slice ----------------
            if constexpr (C::kAdjacent) {
                // record r enters with weight prob * alpha_{r+1} * ... * alpha_loop (the V plane's own coefficients)
                float weight = prob;
                for (int r = p.chain_count - 1; r >= 0; --r) {
                    const uint32_t base = v_anchor + P * p.chain_offset[r];
                    const int bits = p.chain_bits[r], group = p.chain_group[r];
                    if (bits == 4)
                        accumulate_record<4, 32, P, D, true, kPartial>(base, t, js, weight, acc_b, acc_off0, acc_off1, live_token);
                    else if (group == 32)
                        accumulate_record<2, 32, P, D, true, kPartial>(base, t, js, weight, acc_b, acc_off0, acc_off1, live_token);
                    else
                        accumulate_record<2, 16, P, D, true, kPartial>(base, t, js, weight, acc_b, acc_off0, acc_off1, live_token);
                    if (r > 0) {
                        const int alpha_at = P * (D * bits / 8 + 2 * (D / group));
                        weight *= bf16_bits_to_float(lds16(base + alpha_at + 2 * t));
                    }
                }
            } else {
            float pa = prob;  // the V plane stores its own coefficient
            if constexpr (C::kResidual) pa *= bf16_bits_to_float(lds16(v_residual + kResidualAlphaAt + 2 * t));
            accumulate_record<C::AB, C::AG, P, D, kTwoOffsets, kPartial>(v_anchor, t, js, pa, acc_b, acc_off0, acc_off1, live_token);
            if constexpr (C::kResidual)
                accumulate_record<C::RB, C::RG, P, D, kTwoOffsets, kPartial>(v_residual, t, js, prob, acc_b, acc_off0, acc_off1,
                                                                             live_token);
            }
            // A token that holds a large share of its stream's softmax mass leaves half-precision sums of the size of
            // its own value row behind; every later add would be rounded at THAT magnitude (an 11-bit significand: a
            // value of 30 costs 0.007 per add).  Such tokens are rare; the page loop moves the sums to fp32 right after
            // the page of one.
            if (prob > l_before) pages_to_flush = 0;   // more than half of the stream's mass so far
        }
    };

    int stage = 0;
    uint32_t parity = 0;
    int it_done = 0;  // pages fully consumed
    for (int it = 0; it < warp_pages; ++it) {
        if (kBulkCopy) {
            if (!mbar_wait(bar_addr + 8 * stage, parity)) { failed = true; break; }
        } else {
            cp_async_wait<C::kStages - 1>();
            __syncwarp();  // the other lanes' chunks of this page have landed too
        }
        const uint32_t k_anchor = ring_addr + stage * C::kStageBytes;
        const int first_token = (page_begin + warp + kWarps * it) * P;
        const int valid = history - first_token;  // >= P for every page but the last one of the history

        // Full pages run without any per-token predicate; only the last page of a sequence can be partial.
        float scores[P / 8];
        if (valid >= P) {
#pragma unroll
            for (int sub = 0; sub < P / 8; ++sub) scores[sub] = score_token(k_anchor, sub * 8 + slot, true);
#pragma unroll
            for (int sub = 0; sub < P / 8; ++sub) absorb_token(std::false_type{}, k_anchor, sub * 8 + slot, true, scores[sub]);
        } else {
#pragma unroll
            for (int sub = 0; sub < P / 8; ++sub) scores[sub] = score_token(k_anchor, sub * 8 + slot, sub * 8 + slot < valid);
#pragma unroll
            for (int sub = 0; sub < P / 8; ++sub)
                absorb_token(std::true_type{}, k_anchor, sub * 8 + slot, sub * 8 + slot < valid, scores[sub]);
        }

        if (__any_sync(kFullMask, --pages_to_flush <= 0)) {
            flush();
            pages_to_flush = kFlushPages;
        }
        __syncwarp();  // every lane has finished reading this stage
        if (issued < warp_pages) {
            if (issued - batch_base == 32) load_batch(issued);
            const int block = __shfl_sync(kFullMask, my_block, issued - batch_base);
            issue(block, stage);
            ++issued;
        }
        if (!kBulkCopy) cp_async_commit();
        if (++stage == C::kStages) { stage = 0; parity ^= 1u; }
        it_done = it + 1;
    }
    __syncwarp();
    failed = __any_sync(kFullMask, failed);
    if (failed) {
        if (lane == 0) atomicExch(p.status, 1);
        // Copies already issued still target this CTA's shared memory: give each one more bounded wait.
        int s2 = stage;
        uint32_t par2 = parity;
        for (int k = it_done; k < issued; ++k) {
            mbar_wait(bar_addr + 8 * s2, par2);
            if (++s2 == C::kStages) { s2 = 0; par2 ^= 1u; }
        }
    }
    if (!kBulkCopy) cp_async_wait<0>();
    flush();

    RQ_STAMP(kAfterPages);
    // ---- fold the 8 token slots of the warp ------------------------------------------------------------
    const float m = m_biased + kWeightBits;  // kNever stays kNever
    float m_warp = m;
    m_warp = fmaxf(m_warp, __shfl_xor_sync(kFullMask, m_warp, 4));
    m_warp = fmaxf(m_warp, __shfl_xor_sync(kFullMask, m_warp, 8));
    m_warp = fmaxf(m_warp, __shfl_xor_sync(kFullMask, m_warp, 16));
    const float f_slot = fast_exp2(m - m_warp);  // untouched streams carry zero sums, so their factor is irrelevant
    float l_warp = l * kWeightDown * f_slot;
    l_warp += __shfl_xor_sync(kFullMask, l_warp, 4);
    l_warp += __shfl_xor_sync(kFullMask, l_warp, 8);
    l_warp += __shfl_xor_sync(kFullMask, l_warp, 16);
    __syncwarp();
    {
        float* scratch = reinterpret_cast<float*>(ring) + lane * 33;  // [32 lanes][33]: conflict-free both ways
#pragma unroll
        for (int e = 0; e < 32; ++e) {
            const int pair = e >> 1, b = pair >> 2, i = pair & 3;
            const int local = 8 * b + i + 4 * (e & 1);  // channel inside the slice
            const float off = (kTwoOffsets && local >= 16) ? acc_off1 : acc_off0;
            scratch[local] = (acc[e] * kSumDown + off * kWeightDown) * f_slot;
        }
    }
    __syncwarp();
    if (4 * lane < D) {
        const float* scratch = reinterpret_cast<const float*>(ring);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = 4 * lane + i, slice = c >> 5, local = c & 31;
            float sum = 0.f;
#pragma unroll
            for (int g = 0; g < 8; ++g) sum += scratch[(4 * g + slice) * 33 + local];
            warp_acc[warp * D + c] = sum;
        }
    }
    if (lane == 0) {
        warp_stat[2 * warp] = m_warp;
        warp_stat[2 * warp + 1] = l_warp;
    }
    __syncthreads();

    RQ_STAMP(kAfterWarpFold);
    // ---- fold the warps of the CTA: thread c owns channel c ---------------------------------------------
    float part_m = kNever;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) part_m = fmaxf(part_m, warp_stat[2 * w]);
    float part_l = 0.f, value = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const float mw = warp_stat[2 * w];
        const float f = fast_exp2(mw - part_m);
        part_l += warp_stat[2 * w + 1] * f;
        if (tid < D) value += warp_acc[w * D + tid] * f;
    }

    // ---- several partitions: park the partial, the last CTA to arrive folds them -----------------------
    if (splits > 1) {
        // partial results are stored item-major: the row's partitions are `heads` records apart
        const int64_t item_stride = static_cast<int64_t>(heads) * (D + 2);
        float* mine = p.partials + (static_cast<int64_t>(work.first + split) * heads + head) * (D + 2);
        if (tid == 0) { mine[0] = part_m; mine[1] = part_l; }
        if (tid < D) mine[2 + tid] = value;
        // Release: the barrier orders every thread's stores before thread 0's fence, which is cumulative; the ticket follows
        // it.  Acquire: the thread that drew the last ticket fences again before the barrier that lets the others read
        // (through L2: ld.global.cg).  One thread fences instead of all of them.
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const int ticket = atomicAdd(p.counters + row * heads + head, 1);
            const bool last = ticket == splits - 1;
            if (last) {
                p.counters[row * heads + head] = 0;  // ready for the next call
                __threadfence();
            }
            misc[0] = last ? 1.f : 0.f;
        }
        __syncthreads();
        RQ_STAMP(kAfterTicket);
        if (misc[0] == 0.f) return;
        const float* all = p.partials + (static_cast<int64_t>(work.first) * heads + head) * (D + 2);
        // One pass, eight partitions' (max, denominator, value) loads in flight at a time; the partitions are merged like
        // the tokens of the page loop, by rescaling the running sums when the reference exponent moves.
        part_m = kNever;
        part_l = 0.f;
        value = 0.f;
        for (int base = 0; base < splits; base += 8) {
            float ms[8], ls[8], vs[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float* one = all + min(base + u, splits - 1) * item_stride;   // clamped: a repeated load, not a branch
                ms[u] = __ldcg(one);
                ls[u] = __ldcg(one + 1);
                vs[u] = tid < D ? __ldcg(one + 2 + tid) : 0.f;
            }
            float batch_m = part_m;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (base + u < splits) batch_m = fmaxf(batch_m, ms[u]);
            const float keep = fast_exp2(part_m - batch_m);   // kNever - kNever = 0 the first time: the sums are zero anyway
            part_l *= keep;
            value *= keep;
            part_m = batch_m;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (base + u < splits) {
                    const float f = fast_exp2(ms[u] - part_m);
                    part_l += ls[u] * f;
                    value += vs[u] * f;
                }
            }
        }
    }

    RQ_STAMP(kAfterPartitions);
    // ---- live token (its score was computed in the prologue), normalisation, optional inverse value rotation, store ---
    const float live = misc[1];
    const float total_m = fmaxf(part_m, live);
    const float f_hist = part_l > 0.f ? fast_exp2(part_m - total_m) : 0.f;
    const float f_live = fast_exp2(live - total_m);
    const float denom = part_l * f_hist + f_live;
    float hist = tid < D ? value * f_hist / denom : 0.f;
    if (p.value_matrix != nullptr) {
        // dense explicit value rotation: history <- history @ R^T, one output channel per thread
        float* buffer = warp_acc;  // free again
        __syncthreads();
        if (tid < D) buffer[tid] = hist;
        __syncthreads();
        if (tid < D) {
            const uint4* matrix_row = reinterpret_cast<const uint4*>(p.value_matrix + (static_cast<int64_t>(head) * D + tid) * D);
            float sum = 0.f;
#pragma unroll 4
            for (int k8 = 0; k8 < D / 8; ++k8) {
                const uint4 packed = __ldg(matrix_row + k8);
                const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 pair = __half22float2(as_half2(words[i]));
                    sum += buffer[8 * k8 + 2 * i] * pair.x + buffer[8 * k8 + 2 * i + 1] * pair.y;
                }
            }
            hist = sum;
        }
    } else if (p.value_sign != nullptr) {
        float* buffer = warp_acc;  // free again
        __syncthreads();
        if (tid < D) buffer[tid] = hist;
        __syncthreads();
        if (warp == 0) unrotate_history<D>(p, head, buffer);
        __syncthreads();
        if (tid < D) hist = buffer[tid];
    }
    if (tid < D) {
        const float v_live = __bfloat162float(p.value[static_cast<int64_t>(row) * p.value_stride + head * D + tid]);
        const __nv_bfloat16 result = __float2bfloat16_rn(hist + v_live * (f_live / denom));
        p.output[static_cast<int64_t>(row) * p.output_stride + head * D + tid] = result;
        // head-sharded serving: the same row goes straight into every GPU's gathered buffer (plain stores, own
        // memory or a peer's over NVLink); a warp writes 64 contiguous bytes per peer
        const int64_t gathered = static_cast<int64_t>(row) * p.gather_stride + (p.gather_head_offset + head) * D + tid;
        for (int peer = 0; peer < p.num_peers; ++peer) p.peer_output[peer][gathered] = result;
    }
    RQ_STAMP(kAtExit);
    RQ_STAMP_GLOBAL(kAtExitGlobalNs);
    if (p.gather_publish) {
        // The CTA that finishes the call's last (row, head) tells every GPU that this rank's rows are in place.
        // Every CTA: barrier (orders all of its threads' peer stores before thread 0's fence), a device-scope fence, a
        // ticket.  The CTA that draws the last ticket has thereby observed every other CTA's fence; its own system-scope
        // fence followed by the release stores of the flag extends that order to the peers (causality order composes
        // across scopes), so a peer that has acquired the flag sees every row of the call.
        uint32_t* published = reinterpret_cast<uint32_t*>(misc);  // [0]: the epoch this CTA published, [3]: whether it did
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const uint32_t ticket = atomicAdd(p.gather_state + 2, 1u);
            const uint32_t total_rows = static_cast<uint32_t>(min(__ldcg(p.query_start_loc + p.num_requests), p.num_rows));
            uint32_t epoch = 0u;
            const bool last = ticket + 1u == total_rows * static_cast<uint32_t>(heads);
            if (last) {
                p.gather_state[2] = 0u;  // ready for the next call
                __threadfence_system();
                epoch = *reinterpret_cast<volatile uint32_t*>(p.gather_state) + 1u;
                *reinterpret_cast<volatile uint32_t*>(p.gather_state) = epoch;
                for (int peer = 0; peer < p.num_peers; ++peer)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.gather_flags[peer] + p.gather_rank), "r"(epoch) : "memory");
            }
            published[0] = epoch;
            published[3] = last ? 1u : 0u;
        }
        if (p.gather_complete) {
            // ... and stays until every peer's signal of the same call is here: the launch then ends only when this GPU's
            // gathered buffer is complete.  The peers' kernels run on their own GPUs whatever this one does, so the wait
            // cannot block them; it is bounded all the same.
            __syncthreads();
            if (published[3] != 0u && warp == 0 && lane < p.num_peers) wait_for_peers(p, lane, published[0]);
        }
    }
}

template <class C>
cudaError_t launch_one(const AttentionParams& p, cudaStream_t stream) {
    // Raise the dynamic shared memory limit once per device (bit d of the mask = device d is configured).
    static std::atomic<unsigned long long> configured{0ull};
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    const unsigned long long bit = 1ull << (device & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        err = cudaFuncSetAttribute(attention_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (err != cudaSuccess) return err;
        configured.fetch_or(bit, std::memory_order_release);
    }
    const int64_t items = p.splits > 0 ? static_cast<int64_t>(p.num_rows) * p.splits : p.capacity;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(items * p.heads));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = C::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = p.programmatic_launch ? 1 : 0;
    return cudaLaunchKernelEx(&config, attention_kernel<C>, p);
}

template <int D, int AB, int AG, int RB, int RG, int P>
cudaError_t launch_mean(bool has_mean, const AttentionParams& p, cudaStream_t stream) {
    if (has_mean) return launch_one<Config<D, AB, AG, RB, RG, P, true>>(p, stream);
    return launch_one<Config<D, AB, AG, RB, RG, P, false>>(p, stream);
}

// The (anchor record, loop record) pairs of the reference's schedule lists
// (plugins/residual_quantization/csrc/dispatch/decode_*_anchor_*.cu): 2224 / 4222 / 4444 / 2222 and single-record groups.
template <int D, int P>
cudaError_t launch_records(const AttentionVariant& v, const AttentionParams& p, cudaStream_t stream) {
    if (v.adjacent) {
        if (v.has_mean) return launch_one<Config<D, 4, 32, 0, 32, P, true, true>>(p, stream);
        return launch_one<Config<D, 4, 32, 0, 32, P, false, true>>(p, stream);
    }
    const int ab = v.anchor_bits, ag = v.anchor_group, rb = v.residual_bits, rg = v.residual_group;
    if (ab == 4 && ag == 32) {
        if (rb == 0) return launch_mean<D, 4, 32, 0, 32, P>(v.has_mean, p, stream);
        if (rb == 2 && rg == 32) return launch_mean<D, 4, 32, 2, 32, P>(v.has_mean, p, stream);
        if (rb == 2 && rg == 16) return launch_mean<D, 4, 32, 2, 16, P>(v.has_mean, p, stream);
        if (rb == 4 && rg == 32) return launch_mean<D, 4, 32, 4, 32, P>(v.has_mean, p, stream);
    } else if (ab == 2 && ag == 32) {
        if (rb == 0) return launch_mean<D, 2, 32, 0, 32, P>(v.has_mean, p, stream);
        if (rb == 2 && rg == 32) return launch_mean<D, 2, 32, 2, 32, P>(v.has_mean, p, stream);
        if (rb == 4 && rg == 32) return launch_mean<D, 2, 32, 4, 32, P>(v.has_mean, p, stream);  // "4222"/"2224", INT2 anchor
    } else if (ab == 2 && ag == 16) {
        if (rb == 0) return launch_mean<D, 2, 16, 0, 32, P>(v.has_mean, p, stream);
        if (rb == 2 && rg == 16) return launch_mean<D, 2, 16, 2, 16, P>(v.has_mean, p, stream);
        if (rb == 4 && rg == 32) return launch_mean<D, 2, 16, 4, 32, P>(v.has_mean, p, stream);
    }
    return cudaErrorInvalidDeviceFunction;
}

}  // namespace

// One translation unit per head dimension (they compile in parallel).
#if RQ_ATTENTION_TIMELINE
// Copies the timeline array (uint64 [2][kTimelineCtas][kTimelineSlots]) of this head dimension's kernels to the host.
#if RQ_ATTENTION_HEAD_DIM == 128
extern "C" int rq_timeline_d128(void* host, size_t bytes) {
#else
extern "C" int rq_timeline_d96(void* host, size_t bytes) {
#endif
    if (bytes != sizeof(g_timeline)) return -1;
    return static_cast<int>(cudaMemcpyFromSymbol(host, g_timeline, sizeof(g_timeline)));
}
#endif

#if RQ_ATTENTION_HEAD_DIM == 128
cudaError_t launch_attention_d128(const AttentionVariant& v, const AttentionParams& p, cudaStream_t stream) {
    return v.page_tokens == 16 ? launch_records<128, 16>(v, p, stream) : launch_records<128, 32>(v, p, stream);
}
#else
cudaError_t launch_attention_d96(const AttentionVariant& v, const AttentionParams& p, cudaStream_t stream) {
    return v.page_tokens == 16 ? launch_records<96, 16>(v, p, stream) : launch_records<96, 32>(v, p, stream);
}
#endif

}  // namespace rq
