// Dense rotation of bf16 rows by a learned fp16 matrix: y[t][h][:] = x[t][h][:] @ R[h]   (fp32 out).  Used for the
// query rows of an attention call (one row per request); the quantizer rotates inside its own kernel (rq_quantize.cu).
//
// The reference runs this product inside its query preparation with TF32 m16n8k8 MMAs
// (plugins/residual_quantization/csrc/attention/prepare.cuh:61-145).
// Here R[h] is staged once per CTA in shared memory and reused for 64 rows.  bf16 inputs and fp16 matrix entries
// are both exactly representable in TF32, so every product is exact and the accumulation is fp32, as in the
// reference; only the summation order differs.
//
// CTA = 64 rows (tokens) x 1 head x 1 source tensor, 4 warps; warp = 16 rows x all D columns.
#include <atomic>

#include "rq_common.cuh"
#include "rq_kernels.h"

namespace rq {
namespace {

constexpr int kRotateRows = 64;

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int D>
__global__ void __launch_bounds__(128) rotate_rows_kernel(const __grid_constant__ RotateParams p) {
    constexpr int kPad = D + 4;  // row stride in floats: conflict-free fragment loads
    extern __shared__ __align__(16) float shared[];
    float* matrix = shared;                 // [D][kPad]   R[h][k][n] as fp32 (TF32-exact)
    float* rows = shared + D * kPad;        // [64][kPad]  the input rows as fp32
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.y, source = blockIdx.z;
    const int first = blockIdx.x * kRotateRows;

    const __half* r = p.matrix + static_cast<int64_t>(head) * D * D;
    for (int i = tid; i < D * D / 2; i += 128) {
        const __half2 pair = reinterpret_cast<const __half2*>(r)[i];
        const int k = (2 * i) / D, n = (2 * i) % D;
        matrix[k * kPad + n] = __low2float(pair);
        matrix[k * kPad + n + 1] = __high2float(pair);
    }
    const __nv_bfloat16* src = p.source[source];
    const int64_t stride = p.source_stride[source];
    for (int i = tid; i < kRotateRows * D / 2; i += 128) {
        const int row = (2 * i) / D, c = (2 * i) % D;
        const int token = first + row;
        float lo = 0.f, hi = 0.f;
        if (token < p.num_rows && (p.slots == nullptr || p.slots[token] >= 0)) {
            const __nv_bfloat16* x = src + token * stride + head * D + c;
            lo = __bfloat162float(x[0]);
            hi = __bfloat162float(x[1]);
        }
        rows[row * kPad + c] = lo;
        rows[row * kPad + c + 1] = hi;
    }
    __syncthreads();

    const int g = lane >> 2, t = lane & 3;
    const float* a_rows = rows + (warp * 16) * kPad;
    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
#pragma unroll 4
    for (int k = 0; k < D; k += 8) {
        uint32_t a[4];
        a[0] = __float_as_uint(a_rows[g * kPad + k + t]);
        a[1] = __float_as_uint(a_rows[(g + 8) * kPad + k + t]);
        a[2] = __float_as_uint(a_rows[g * kPad + k + t + 4]);
        a[3] = __float_as_uint(a_rows[(g + 8) * kPad + k + t + 4]);
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            uint32_t b[2];
            b[0] = __float_as_uint(matrix[(k + t) * kPad + 8 * n + g]);
            b[1] = __float_as_uint(matrix[(k + t + 4) * kPad + 8 * n + g]);
            mma_tf32(acc[n], a, b);
        }
    }
    float* out = p.output + (static_cast<int64_t>(source) * p.num_rows) * p.heads * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int token = first + warp * 16 + g + 8 * half;
            if (token < p.num_rows) {
                float2 v = make_float2(acc[n][2 * half] * p.scale, acc[n][2 * half + 1] * p.scale);
                *reinterpret_cast<float2*>(out + (static_cast<int64_t>(token) * p.heads + head) * D + 8 * n + 2 * t) = v;
            }
        }
    }
}

}  // namespace

size_t rotate_shared_bytes(int head_dim) { return static_cast<size_t>(head_dim + kRotateRows) * (head_dim + 4) * sizeof(float); }

cudaError_t launch_rotate(const RotateParams& p, int head_dim, cudaStream_t stream) {
    if (p.num_rows <= 0 || p.num_sources <= 0) return cudaSuccess;
    const dim3 grid((p.num_rows + kRotateRows - 1) / kRotateRows, p.heads, p.num_sources);
    const size_t smem = rotate_shared_bytes(head_dim);
    // the shared-memory limit is raised once per device (bit d of the mask = device d is configured), not per launch
    static std::atomic<unsigned long long> configured[2];
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    const unsigned long long bit = 1ull << (device & 63);
    std::atomic<unsigned long long>& done = configured[head_dim == 128 ? 0 : 1];
    if (!(done.load(std::memory_order_acquire) & bit)) {
        err = head_dim == 128
                  ? cudaFuncSetAttribute(rotate_rows_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))
                  : cudaFuncSetAttribute(rotate_rows_kernel<96>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess) return err;
        done.fetch_or(bit, std::memory_order_release);
    }
    if (head_dim == 128) rotate_rows_kernel<128><<<grid, 128, smem, stream>>>(p);
    else rotate_rows_kernel<96><<<grid, 128, smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace rq
