// Internal launch interface between the C ABI (rq_capi.cu) and the kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/rq_b200.h"

namespace rq {

struct QuantizeParams {
    const __nv_bfloat16* key[RQ_MAX_RECORDS];
    const __nv_bfloat16* value[RQ_MAX_RECORDS];
    int64_t key_stride[RQ_MAX_RECORDS];
    int64_t value_stride[RQ_MAX_RECORDS];
    uint8_t* cache;
    int64_t plane_stride;
    const int64_t* slots;
    const uint32_t* sign[2];  // per plane: [heads][head_dim/32] sign bit masks (signed-Hadamard rotation)
    float rscale[2];
    int rotation[2];          // RqRotationKind per plane
    const float* mean;        // [records][heads][head_dim] or nullptr
    int num_tokens, heads, page_tokens, page_width;
    int num_records, anchor, mode, coefficient, chain;
    int bits[RQ_MAX_RECORDS], group[RQ_MAX_RECORDS], record_offset[RQ_MAX_RECORDS];
    int vector_loads;         // rows are 16-byte aligned
    // Dense learned rotation per plane: fp16 [heads][head_dim][head_dim], y = x @ R, applied inside the quantizer CTA
    // (nullptr = rotate with the fused Walsh-Hadamard transform, or not at all).
    const __half* dense_matrix[2];
    int plane_first;          // a launch covers planes plane_first .. plane_first + gridDim.z - 1
    int dense_tiles;          // tiles of 16 tokens a CTA of the fused dense kernel walks over
    int dense_planes;         // planes its launch covers (gridDim.z)
    int programmatic_launch;  // launch with the programmatic-stream-serialization attribute
};

cudaError_t launch_quantize(const QuantizeParams& p, int head_dim, cudaStream_t stream);

// Layout of the attention workspace (all offsets multiples of 256 bytes):
//   [0, 256)                         status word (int32) + padding
//   [256, 256 + C)                   arrival counters, one int32 per (row, head); C = 64 KiB, or the next power of two
//                                    that holds them: the same for every shape of up to 16384 (row, head) pairs
//   [256 + C, ...)           float [work items][heads][head_dim + 2]  (max, denominator, value sums);
//                                    work items = rows * splits, or the capacity when the device picks the partitions
struct AttentionParams {
    const __nv_bfloat16* query;
    const __nv_bfloat16* key;
    const __nv_bfloat16* value;
    __nv_bfloat16* output;
    int64_t query_stride, key_stride, value_stride, output_stride;
    const uint8_t* cache;
    int64_t plane_stride;
    const int32_t* query_start_loc;
    const int32_t* seq_lens;
    const int32_t* block_table;
    int num_rows, num_requests, block_table_stride, max_blocks;
    const uint32_t* key_sign;    // signed-Hadamard key rotation or nullptr
    const uint32_t* value_sign;  // explicit value rotation (undone on the history sum) or nullptr
    float key_rscale, value_rscale;
    const __half* query_matrix;  // dense key rotation: fp16 [heads][head_dim][head_dim], q @ R is formed in the prologue; else nullptr
    const __half* value_matrix;  // dense explicit value rotation [heads][head_dim][head_dim]; else nullptr
    const float* mean;           // [records][heads][head_dim] or nullptr
    int heads, page_width;
    int anchor_offset;           // bytes per token before the anchor record
    int residual_offset;         // bytes per token before the current loop's record (unused on the anchor loop)
    int anchor_index, loop_index;
    // Adjacent reference mode: the loop's value is a chain over records 0..loop_index, all of which are read.
    int chain_count;             // loop_index + 1 (0 in anchor mode)
    int chain_bits[4], chain_group[4];
    int chain_offset[5];         // bytes per token before record r; [chain_count] = bytes of the staged prefix
    // Work decomposition (splits < 0: as splits == 0 with the chunk size fixed to -splits pages).  splits > 0: every row is cut into exactly `splits` partitions (grid = rows * splits * heads).
    // splits == 0: the grid is capacity * heads and every CTA derives the (row, partition) of its work item from the
    // sequence lengths on the device: partitions per row proportional to the row's pages (see find_work).
    int splits;
    int capacity;                // work items per head the grid and the partial-result buffer provide (splits == 0)
    int sm_count;                // multiprocessors of the device (input of the on-device partition choice)
    int programmatic_launch;     // launch with the programmatic-stream-serialization attribute
    int early_start;             // metadata and cache pages may be read before the previous kernel of the stream completed
    int32_t* status;
    int32_t* counters;
    float* partials;
    // Fused head gather: finished rows also go to [rows][gather_stride] buffers of num_peers GPUs at gather_head_offset.
    int num_peers, gather_head_offset;
    int64_t gather_stride;
    __nv_bfloat16* peer_output[RQ_MAX_PEERS];
    // Completion signal of the fused gather: flag arrays of every GPU, this rank's state block ([0] epoch, [1] status,
    // [2] arrival counter), what this call does with them.
    uint32_t* gather_flags[RQ_MAX_PEERS];
    uint32_t* gather_state;
    int gather_rank, gather_publish, gather_wait, gather_complete;
    unsigned long long gather_timeout_ns;
};

// Node-level barrier kernel behind rq_peer_barrier.
struct PeerBarrierParams {
    uint32_t* flags[RQ_MAX_PEERS];
    uint32_t* state;  // [0] epoch, [1] status
    int world, rank;
    unsigned long long timeout_ns;
    int wait_only;
    int programmatic_launch;
};
cudaError_t launch_peer_barrier(const PeerBarrierParams& p, cudaStream_t stream);

// Kernel variant selector: which residual record (if any) is read next to the INT4/INT2 anchor.
struct AttentionVariant {
    int head_dim;       // 128 | 96
    int anchor_bits;    // 2 | 4
    int anchor_group;   // 16 | 32
    int residual_bits;  // 0 (anchor loop) | 2 | 4
    int residual_group; // 16 | 32 (ignored on the anchor loop)
    int page_tokens;    // 16 | 32
    bool has_mean;
    bool adjacent;      // adjacent reference mode: record types are run-time data (AttentionParams::chain_*)
};

// Returns cudaErrorInvalidDeviceFunction when the variant is not compiled in.
cudaError_t launch_attention(const AttentionVariant& v, const AttentionParams& p, cudaStream_t stream);
bool attention_variant_available(const AttentionVariant& v);

}  // namespace rq
