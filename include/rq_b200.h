/*
 * rq_b200.h -- C ABI of the B200 (sm_100a) packed-KV kernels.
 *
 * Two operators, the same two the reference's extension module `residual_quantization._cuda`
 * exports (plugins/residual_quantization/csrc/dispatch/binding.cpp:19-37):
 *
 *   rq_quantize   replaces  quantize()   plugins/residual_quantization/csrc/common/api.h:22-31
 *                                        (quantize/api.cpp:8-95, quantize/launch.cuh:45-86)
 *   rq_attention  replaces  attention()  plugins/residual_quantization/csrc/common/api.h:11-20
 *                                        (attention/api.cpp:8-115, attention/launch.cuh:34-132)
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless stated otherwise, `stream` is a
 * cudaStream_t passed as void*.  Nothing here allocates, synchronizes or reads device memory on the host,
 * so both calls can be captured in a CUDA graph and replayed with changing slot mappings, sequence lengths
 * and block tables.  All functions return RQ_OK (0) or a negative RqStatus; they never throw and never abort.
 * rq_last_error() gives a human-readable message for the calling thread's most recent failure.
 *
 * Page layout (identical to the reference, plugins/residual_quantization/csrc/common/cache.cuh:10-106):
 * the cache is uint8 [2][num_blocks][heads][page_tokens][page_width], plane 0 = K, plane 1 = V.  One
 * (plane, block, head) page is page_tokens*page_width bytes, record-major: record r (loop order) occupies
 * bytes [P*off_r, P*off_{r+1}); inside a record: codes [P][D*bits/8], FP8-e4m3 scales [P][D/group], FP8-e4m3
 * offsets [P][D/group], bf16 alpha [P].  Four consecutive channels share a storage word (uint8 for INT2,
 * little-endian uint16 for INT4), channel c at bit (c%4)*bits.
 */
#ifndef RQ_B200_H_
#define RQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RQ_MAX_RECORDS 8
#define RQ_MAX_PEERS 8 /* GPUs of one node that a head-sharded output can be stored to */

/* RqQuantizeArgs.flags / RqAttentionArgs.flags.
 *
 * By default both kernels are launched as PROGRAMMATIC DEPENDENTS of the previous kernel of the stream
 * (cudaLaunchAttributeProgrammaticStreamSerialization): the launch and the scheduling of the CTAs overlap that kernel,
 * and every CTA then waits (griddepcontrol.wait) for that kernel to complete before it reads or writes anything.  That
 * is indistinguishable from plain stream order for the caller, only faster.  Each kernel lets its own successor be
 * scheduled once that wait is over, so at most two kernels of a stream overlap.
 *
 * RQ_FLAG_SERIAL_LAUNCH        launch this call with plain stream order instead (rq_set_programmatic_launch(0) or
 *                              RQ_PROGRAMMATIC_LAUNCH=0 in the environment does so for every call).
 * RQ_FLAG_STABLE_METADATA      rq_attention only; a promise by the caller: the kernel launched immediately before this
 *                              call on the same stream did not write query_start_loc, seq_lens, block_table or the
 *                              cached tokens this call reads.  The work lookup, the page-table fetch and the first page
 *                              copies then run BEFORE the wait, i.e. in the shadow of the previous kernel; q, k, v are
 *                              still read after it.  True under a serving engine, which writes the metadata once per
 *                              step and whose previous kernel is the projection that produces q/k/v.  The library
 *                              withdraws the early start by itself when the last rq_quantize on the stream wrote the
 *                              same cache.
 * RQ_FLAG_GATHER_PUBLISH       rq_attention with num_peers > 0: the CTA that finishes the call's last output row advances
 *                              this rank's epoch (gather_state[0]) and publishes it in slot gather_rank of every
 *                              peer's flag array, after all of the call's peer stores (system-scope release).
 * RQ_FLAG_GATHER_WAIT          rq_attention with num_peers > 0: before a CTA reads q/k/v it waits (bounded by
 *                              gather_timeout_ns) until every peer has published the epoch this rank has reached, i.e.
 *                              until the PREVIOUS call's gathered rows are complete on this GPU -- the point where a
 *                              model's next attention call depends on them through the output projection.
 * RQ_FLAG_GATHER_COMPLETE      rq_attention with num_peers > 0 (implies RQ_FLAG_GATHER_PUBLISH): the CTA that published
 *                              then waits (bounded by gather_timeout_ns) until every peer's signal of the SAME call has
 *                              arrived, so the launch does not end before this GPU's gathered buffer holds every
 *                              rank's rows: whatever follows on the stream -- a library GEMM included -- may read them,
 *                              and no barrier kernel is needed.  Every rank must issue the same sequence of calls. */
#define RQ_FLAG_SERIAL_LAUNCH 1
#define RQ_FLAG_STABLE_METADATA 2
#define RQ_FLAG_GATHER_PUBLISH 4
#define RQ_FLAG_GATHER_WAIT 8
#define RQ_FLAG_GATHER_COMPLETE 16

typedef enum RqStatus {
    RQ_OK = 0,
    RQ_ERR_INVALID_ARGUMENT = -1, /* a shape, pointer, alignment or enum is wrong (the TORCH_CHECKs of api.cpp) */
    RQ_ERR_UNSUPPORTED = -2,      /* no kernel is compiled for this (head_dim, records, mode, ...) combination
                                     (kernel_registry.h:66-72 raises the same way) */
    RQ_ERR_WORKSPACE = -3,        /* workspace missing, misaligned or too small */
    RQ_ERR_CUDA = -4,             /* a CUDA runtime call failed; rq_last_error() holds its message */
    RQ_ERR_DEVICE_TIMEOUT = -5    /* reported by rq_attention_status(): a bounded on-chip wait gave up */
} RqStatus;

typedef enum RqReferenceMode { RQ_REFERENCE_ANCHOR = 0, RQ_REFERENCE_ADJACENT = 1 } RqReferenceMode; /* common/types.h:3 */
typedef enum RqCoefficient { RQ_COEFF_UNIT = 0, RQ_COEFF_NORM = 1, RQ_COEFF_LS = 2 } RqCoefficient;  /* quantize/types.h:4 */

/* Where the least-squares coefficient and the residual are formed.
 * KERNEL:      in rotated coordinates against the bf16 reconstruction of the anchor, as the reference's CUDA
 *              quantizer does (quantize/kernel.cuh:76-120).
 * CALIBRATION: in original coordinates with bf16 prediction and bf16 residual target, as the reference's
 *              PyTorch statement does (scripts/calibration/quantization.py:16-71).
 * Both store the same fields in the same layout. */
typedef enum RqChain { RQ_CHAIN_KERNEL = 0, RQ_CHAIN_CALIBRATION = 1 } RqChain;

typedef enum RqRotationKind {
    RQ_ROTATION_NONE = 0,
    /* R[h] = diag(sign[h]) * H_D * scale, y = x @ R.  `data` = uint32 [heads][head_dim/32], bit c%32 of word c/32
     * set when sign[h][c] is -1.  H_128 is the Sylvester matrix, H_96 = Paley-12 (x) Sylvester-8
     * (scripts/calibration/rotation_math.py:6-32). */
    RQ_ROTATION_SIGNED_HADAMARD = 1,
    /* dense fp16 [heads][head_dim][head_dim], y = x @ R (common/api.h:42-55): any learned rotation.  The quantizer
     * rotates inside its own CTAs (TF32 tensor-core products, fp32 accumulation, rows staged in shared memory); the
     * attention call rotates the query rows with one small launch in front of its kernel. */
    RQ_ROTATION_DENSE_FP16 = 2
} RqRotationKind;

typedef struct RqRotation {
    int32_t kind;     /* RqRotationKind */
    float scale;      /* SIGNED_HADAMARD: magnitude of the matrix entries, e.g. (float)fp16(1/sqrt(D)) */
    const void* data; /* see RqRotationKind */
} RqRotation;

/* One KV group: its records in loop order and how residuals refer to the anchor
 * (common/cache.cuh:10-67, the registry key of dispatch/kernel_registry.h:16-18). */
typedef struct RqGroupSpec {
    int32_t num_records;
    int32_t bits[RQ_MAX_RECORDS];       /* 2 or 4 */
    int32_t group_size[RQ_MAX_RECORDS]; /* 16 or 32 */
    int32_t anchor_index;
    int32_t reference_mode; /* RqReferenceMode */
    int32_t heads;
    int32_t head_dim;    /* 128 or 96 */
    int32_t page_tokens; /* 16 or 32 */
} RqGroupSpec;

/* Bytes per token of one (head, plane): sum over records of D*bits/8 + 2*D/group + 2
 * (cache.cuh:14-17; install_model.py:34-38 computes the same).  Negative RqStatus on a bad spec. */
int32_t rq_page_width(const RqGroupSpec* spec);
/* Byte offset (per token) of record `index` inside a page row; index == num_records gives the page width. */
int32_t rq_record_offset(const RqGroupSpec* spec, int32_t index);

typedef struct RqQuantizeArgs {
    RqGroupSpec spec;
    /* One K and one V tensor per record, bf16 [>= num_tokens][heads][head_dim], last two dims packed,
     * row stride in ELEMENTS (common/api.h:33-40). */
    const void* key[RQ_MAX_RECORDS];
    const void* value[RQ_MAX_RECORDS];
    int64_t key_stride[RQ_MAX_RECORDS];
    int64_t value_stride[RQ_MAX_RECORDS];
    void* kv_cache;          /* uint8 [2][num_blocks][heads][page_tokens][page_width], contiguous */
    int64_t num_blocks;
    int64_t plane_stride;    /* bytes between plane 0 and plane 1 (kv_cache.stride(0)) */
    const int64_t* slot_mapping; /* [num_tokens]; slot = block*page_tokens + offset; negative = skip */
    int64_t num_tokens;
    RqRotation key_rotation;
    RqRotation value_rotation;
    const float* key_mean;   /* fp32 [num_records][heads][head_dim] in rotated coordinates, or NULL */
    int32_t coefficient;     /* RqCoefficient */
    int32_t chain;           /* RqChain */
    void* stream;
    void* workspace;         /* unused: no rotation kind needs scratch (rq_quantize_workspace_bytes() is 0) */
    size_t workspace_bytes;
    int32_t flags;           /* RQ_FLAG_* */
} RqQuantizeArgs;

/* Scratch a quantize call needs: always 0 (dense rotations are applied inside the quantizer's CTAs). */
size_t rq_quantize_workspace_bytes(const RqGroupSpec* spec, int64_t num_tokens, int32_t key_rotation_kind,
                                   int32_t value_rotation_kind);
/* Rotate, quantize and bit-pack the K/V rows of every record of a group into their pages.  One launch (two for
 * a long write in which exactly one plane has a dense rotation). */
int32_t rq_quantize(const RqQuantizeArgs* args);

typedef struct RqAttentionArgs {
    RqGroupSpec spec;
    /* bf16 [num_query_rows][heads][head_dim], last two dims packed, row strides in ELEMENTS.
     * key/value hold the live (current) token of every query row (attention/types.h:31-40). */
    const void* query;
    const void* key;
    const void* value;
    void* output;
    int64_t query_stride, key_stride, value_stride, output_stride;
    int32_t num_query_rows; /* rows of the tensors (graph capture size); rows >= query_start_loc[num_requests]
                               are padding and are left untouched (prepare.cuh:405-406, merge.cuh:16) */
    const void* kv_cache;
    int64_t num_blocks;
    int64_t plane_stride;
    const int32_t* query_start_loc; /* [num_requests + 1] */
    const int32_t* seq_lens;        /* [num_requests]; a row attends to seq_len-1 cached tokens + the live one */
    const int32_t* block_table;     /* [>= num_requests][block_table_stride] */
    int32_t num_requests;
    int32_t block_table_stride;
    int32_t max_blocks_per_request; /* block_table.size(1) */
    RqRotation key_rotation;
    RqRotation value_rotation;      /* kind NONE when the model's weights absorbed it (weights.py:9-37) */
    const float* key_mean;          /* fp32 [num_records][heads][head_dim], rotated coordinates, or NULL */
    int32_t loop_index;             /* which record of the group this layer slot reads, 0 <= loop < num_records */
    int32_t num_splits;             /* 0 = the kernel cuts every row into KV partitions in proportion to its OWN length, read
                                       on the device (the reference's per-call schedule, attention/prepare.cuh:237-386);
                                       n > 0 = exactly n partitions for every row;
                                       n < 0 = partitions of -n pages each (length-proportional, chunk size forced) */
    void* workspace;                /* rq_attention_workspace_bytes() bytes, 256-byte aligned, zeroed once with
                                       rq_attention_workspace_init() before its first use */
    size_t workspace_bytes;
    void* stream;
    /* Head-sharded serving (each GPU holds a slice of the KV heads, the output projection needs all of them): when
     * num_peers > 0 the kernel's epilogue ALSO stores every finished output row into the gathered buffer
     * bf16 [rows][gather_stride] of each of the num_peers GPUs (its own included), at head gather_head_offset, with plain
     * stores over NVLink -- the all-gather that would follow the kernel is fused into its epilogue (the reference is single-GPU).
     * peer_output[i] is GPU i's buffer as mapped into THIS process (cudaIpcOpenMemHandle or equivalent).  The stores
     * are complete on the peers after rq_peer_barrier.  Zero-initialised fields (num_peers = 0) switch this off. */
    int32_t num_peers;
    int32_t gather_head_offset;      /* first head of this rank inside a gathered row */
    int64_t gather_stride;           /* ELEMENTS between rows of the gathered buffers (>= total heads * head_dim) */
    void* peer_output[RQ_MAX_PEERS];
    int32_t flags;                   /* RQ_FLAG_* */
    /* Completion signal of the fused gather (RQ_FLAG_GATHER_PUBLISH / _WAIT / _COMPLETE): the same flag arrays and
     * state block rq_peer_barrier uses, so that no barrier kernel is needed between calls.  peer_flags[i] is GPU i's
     * flag array uint32 [RQ_MAX_PEERS] as mapped into this process; gather_state is this rank's own 256 bytes
     * ([0] epoch, [1] status, [2] arrival counter), zeroed once. */
    void* peer_flags[RQ_MAX_PEERS];
    void* gather_state;
    int32_t gather_rank;
    uint64_t gather_timeout_ns;      /* 0 = 2 s */
} RqAttentionArgs;

/* A uniform partition count for callers that want to force one (num_splits > 0): what a host-side cost model picks
 * for a batch whose rows all span max_blocks_per_request pages.  rq_attention does not use it when num_splits == 0. */
int32_t rq_attention_default_splits(int32_t num_query_rows, int32_t heads, int32_t max_blocks_per_request,
                                    int32_t page_tokens);
/* Work items (row partitions) per head that a num_splits == 0 call provides for: the rows plus spare items that long
 * rows are cut into (one wave of resident CTAs; room for two partitions per row where the unsplit rows would leave
 * a second wave nearly empty).  A pure host function of its arguments and the SM count -- never of sequence lengths or of the
 * page-table width -- so the grid is stable across CUDA-graph replays (attention/launch.cuh:53-80 of the reference
 * sizes its work list the same way). */
int32_t rq_attention_work_capacity(int32_t num_query_rows, int32_t heads);
/* Bytes of scratch one rq_attention call needs: per-work-item (max, denominator, value sums), one arrival
 * counter per (row, head) and a status word.  num_splits as in
 * RqAttentionArgs (0 = sized for rq_attention_work_capacity()).  The reference allocates the equivalent per call
 * (attention/launch.cuh:85-98). */
size_t rq_attention_workspace_bytes(int32_t num_query_rows, int32_t heads, int32_t head_dim, int32_t num_splits);
/* Zero the counters and the status word (asynchronous, on `stream`).  Needed once per workspace; every call
 * leaves the counters zero again, and the counters occupy the same 64 KiB of the workspace whatever the shape, so one
 * workspace (sized for the largest call) can serve calls of different shapes one after the other.  Only calls with more
 * than 16384 (row, head) pairs use a larger counter region: give those a workspace of their own, or initialise again
 * when switching. */
int32_t rq_attention_workspace_init(void* workspace, size_t workspace_bytes, void* stream);
/* Split-KV online-softmax decode attention over the packed pages.  One launch. */
int32_t rq_attention(const RqAttentionArgs* args);
/* Synchronizes `stream` and reads the workspace status word: RQ_OK, or RQ_ERR_DEVICE_TIMEOUT if a bounded
 * wait inside the kernel ever gave up since the last init (outputs of that call are then undefined).  Only the
 * bulk-copy build of the kernel (RQ_ATTENTION_BULK_COPY=1) contains such a wait; the default build stages pages with
 * cp.async commit groups, which cannot time out, and never raises the word. */
int32_t rq_attention_status(const void* workspace, void* stream);
/* Process-wide switch for the programmatic dependent launch described at RQ_FLAG_SERIAL_LAUNCH (default on). */
void rq_set_programmatic_launch(int32_t enabled);

/* Maximum scratch rq_attention_noalloc can serve: the size of the library's built-in device buffer. */
#define RQ_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
/* Same operator as rq_attention for callers that are not allowed to allocate device memory -- a serving loop
 * that runs after the framework froze its memory pool, a plugin that is only handed tensors, code running where a
 * cudaMalloc would synchronize the device.  (No counterpart in the reference, which allocates five temporaries per
 * call.)  `workspace` and `workspace_bytes` of the arguments are ignored: the partition results and arrival
 * counters live in a buffer of RQ_STATIC_SCRATCH_BYTES that is compiled into the library as device memory, so every
 * GPU that loads the library holds those 8 MiB until the process exits.  A shape whose
 * rq_attention_workspace_bytes() exceeds that size is rejected with RQ_ERR_WORKSPACE.  The call makes no
 * cudaMalloc/cudaFree and uses no allocating library.  The first call on each device (whichever thread makes it)
 * looks up the buffer's device address, with that device current, and should therefore be made before any stream
 * capture begins.  Every call clears the status word and the counters it is about to use, on `stream`, before the
 * kernel, and launches the kernel in plain stream order (RQ_FLAG_SERIAL_LAUNCH).  All
 * calls on a device share the one buffer: two calls whose kernels overlap on the GPU (different streams) race;
 * keep them on one stream or order them with events. */
int32_t rq_attention_noalloc(const RqAttentionArgs* args);
/* rq_attention_status() for the built-in buffer of the current device (callers of rq_attention_noalloc never see
 * its address). */
int32_t rq_attention_noalloc_status(void* stream);

/* Barrier between the GPUs of one node, for the fused output gather above: a one-CTA kernel on `stream` that publishes
 * this rank's arrival in every peer's flag array (system-scope release store over NVLink) and then waits until every
 * peer has published the same epoch in this rank's own array.  When it completes, all peer stores issued by earlier
 * work of every rank's stream are visible here.  CUDA-graph capturable: the epoch lives in device memory and advances
 * by one per launch.  The wait is bounded (timeout_ns of the GPU's global timer, 0 = 2 s): on expiry the kernel records
 * RQ_ERR_DEVICE_TIMEOUT in `state` and returns, it never spins forever.
 *   flags[i]  rank i's flag array, uint32 [RQ_MAX_PEERS], as mapped into this process; zeroed once before first use
 *   state     this rank's own 256 bytes of device memory (epoch counter, status), zeroed once before first use */
typedef struct RqPeerBarrierArgs {
    int32_t world, rank;
    void* flags[RQ_MAX_PEERS];
    void* state;
    uint64_t timeout_ns;
    void* stream;
    int32_t wait_only; /* 1: do not publish; wait until every peer has published the epoch that this rank's attention
                          calls have reached (RQ_FLAG_GATHER_PUBLISH) -- what a consumer of the gathered rows runs */
} RqPeerBarrierArgs;
int32_t rq_peer_barrier(const RqPeerBarrierArgs* args);
/* Device memory that other processes of the node can map: a plain cudaMalloc (zero-filled), exported and opened
 * with CUDA IPC handles of RQ_PEER_HANDLE_BYTES bytes that the host side exchanges however it likes
 * (torch.distributed in this repository).  rq_peer_open maps a peer's allocation into the calling process with
 * peer access from the current device; the pointer is what RqAttentionArgs.peer_output and
 * RqPeerBarrierArgs.flags take.  Setup-time calls: they allocate and synchronize. */
#define RQ_PEER_HANDLE_BYTES 64
int32_t rq_peer_alloc(size_t bytes, void** pointer);
int32_t rq_peer_free(void* pointer);
int32_t rq_peer_export(const void* pointer, unsigned char* handle /* [RQ_PEER_HANDLE_BYTES] */);
int32_t rq_peer_open(const unsigned char* handle, void** mapped);
int32_t rq_peer_close(void* mapped);
/* Synchronizes `stream` and returns the status recorded in `state`: RQ_OK or RQ_ERR_DEVICE_TIMEOUT. */
int32_t rq_peer_barrier_status(const void* state, void* stream);

const char* rq_last_error(void);
const char* rq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RQ_B200_H_ */
