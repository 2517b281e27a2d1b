// C ABI: argument validation (the checks of the reference's quantize/api.cpp:8-95 and attention/api.cpp:8-115
// restated on plain pointers), kernel selection (dispatch/kernel_registry.h:48-75) and launches.
// No allocation, no synchronization, no host read of device memory on the launch path.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "rq_kernels.h"

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_error, sizeof(g_error), format, args);
    va_end(args);
    return code;
}

int fail_cuda(cudaError_t err, const char* what) {
    return fail(RQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int check_spec(const RqGroupSpec* s) {
    if (s == nullptr) return fail(RQ_ERR_INVALID_ARGUMENT, "null group spec");
    if (s->num_records < 1 || s->num_records > RQ_MAX_RECORDS)
        return fail(RQ_ERR_INVALID_ARGUMENT, "a group needs 1..%d records, got %d", RQ_MAX_RECORDS, s->num_records);
    if (s->head_dim != 128 && s->head_dim != 96)
        return fail(RQ_ERR_UNSUPPORTED, "no kernel for head_dim=%d (128 or 96)", s->head_dim);
    if (s->page_tokens != 16 && s->page_tokens != 32)
        return fail(RQ_ERR_UNSUPPORTED, "no kernel for page_tokens=%d (16 or 32)", s->page_tokens);
    if (s->heads < 1) return fail(RQ_ERR_INVALID_ARGUMENT, "heads must be positive");
    for (int r = 0; r < s->num_records; ++r) {
        if (s->bits[r] != 2 && s->bits[r] != 4)
            return fail(RQ_ERR_UNSUPPORTED, "record %d: bits=%d (2 or 4)", r, s->bits[r]);
        if (s->group_size[r] != 16 && s->group_size[r] != 32)
            return fail(RQ_ERR_UNSUPPORTED, "record %d: group size %d (16 or 32)", r, s->group_size[r]);
    }
    if (s->anchor_index < 0 || s->anchor_index >= s->num_records)
        return fail(RQ_ERR_INVALID_ARGUMENT, "anchor_index %d outside the %d records", s->anchor_index, s->num_records);
    if (s->reference_mode != RQ_REFERENCE_ANCHOR && s->reference_mode != RQ_REFERENCE_ADJACENT)
        return fail(RQ_ERR_INVALID_ARGUMENT, "unknown packed reference mode %d", s->reference_mode);
    if (s->reference_mode == RQ_REFERENCE_ADJACENT && s->anchor_index != 0)
        return fail(RQ_ERR_INVALID_ARGUMENT, "adjacent reference requires anchor_index 0");
    return RQ_OK;
}

int record_bytes(const RqGroupSpec* s, int r) {
    return s->head_dim * s->bits[r] / 8 + 2 * s->head_dim / s->group_size[r] + 2;
}

int check_rotation(const RqRotation& r, const char* name) {
    if (r.kind == RQ_ROTATION_NONE) return RQ_OK;
    if (r.kind == RQ_ROTATION_SIGNED_HADAMARD) {
        if (r.data == nullptr || !aligned(r.data, 4))
            return fail(RQ_ERR_INVALID_ARGUMENT, "%s: sign masks must be a 4-byte aligned device pointer", name);
        if (!(r.scale > 0.f)) return fail(RQ_ERR_INVALID_ARGUMENT, "%s: scale must be positive", name);
        return RQ_OK;
    }
    if (r.kind == RQ_ROTATION_DENSE_FP16) {
        if (r.data == nullptr || !aligned(r.data, 16))
            return fail(RQ_ERR_INVALID_ARGUMENT, "%s: contiguous 16-byte aligned FP16 [heads, channels, channels] rotation required", name);
        return RQ_OK;
    }
    return fail(RQ_ERR_INVALID_ARGUMENT, "%s: unknown rotation kind %d", name, r.kind);
}

constexpr size_t kStatusBytes = 256;
size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Bytes reserved for the arrival counters.  The region has the SAME size for every call of up to 16384 (row, head)
// pairs, so that one workspace can serve calls of different shapes: a counter slot of one call is never a
// partial-result slot of another (partial results are left behind by every call, counters must read zero on entry).
size_t counter_bytes(int64_t rows, int64_t heads) {
    size_t bytes = 64 * 1024;
    while (bytes < static_cast<size_t>(rows) * heads * sizeof(int32_t)) bytes *= 2;
    return bytes;
}

// Multiprocessors of the current device, looked up once per device and process.
int current_sm_count() {
    static std::atomic<int> cache[64];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    int sms = cache[device].load(std::memory_order_relaxed);
    if (sms == 0) {
        int value = 0;
        if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && value > 0) sms = value;
        else sms = 148;
        cache[device].store(sms, std::memory_order_relaxed);
    }
    return sms;
}

// Programmatic dependent launch of the attention and quantize kernels: on unless RQ_PROGRAMMATIC_LAUNCH=0 is in the
// environment or rq_set_programmatic_launch(0) was called.
std::atomic<int> g_programmatic{-1};
bool programmatic_launch_enabled() {
    int state = g_programmatic.load(std::memory_order_relaxed);
    if (state < 0) {
        const char* text = getenv("RQ_PROGRAMMATIC_LAUNCH");
        state = (text != nullptr && text[0] == '0') ? 0 : 1;
        g_programmatic.store(state, std::memory_order_relaxed);
    }
    return state != 0;
}

// Which cache the most recent rq_quantize on a stream wrote.  An attention call that reads the same cache next must not
// start its page copies early (RQ_FLAG_STABLE_METADATA): the pages may still be in flight.  Any attention call clears the
// stream's entry, since it then is the stream's most recent kernel of this library.
struct RecentWrite { void* stream; const void* cache; bool used; };
std::mutex g_recent_mutex;
RecentWrite g_recent[32];
void note_quantize(void* stream, const void* cache) {
    std::lock_guard<std::mutex> lock(g_recent_mutex);
    int slot = -1;
    for (int i = 0; i < 32; ++i) {
        if (g_recent[i].used && g_recent[i].stream == stream) { slot = i; break; }
        if (!g_recent[i].used && slot < 0) slot = i;
    }
    if (slot < 0) slot = static_cast<int>((reinterpret_cast<uintptr_t>(stream) >> 4) % 32);  // table full: evict
    g_recent[slot] = {stream, cache, true};
}
// true when the stream's most recent library kernel was a quantize that wrote `cache`; forgets the entry either way
bool take_recent_write(void* stream, const void* cache) {
    std::lock_guard<std::mutex> lock(g_recent_mutex);
    bool all_used = true, hit = false, known = false;
    for (int i = 0; i < 32; ++i) {
        all_used = all_used && g_recent[i].used;
        if (g_recent[i].used && g_recent[i].stream == stream) {
            known = true;
            hit = g_recent[i].cache == cache;
            g_recent[i].used = false;
        }
    }
    // a full table may have evicted this stream's entry: be cautious then
    return hit || (!known && all_used);
}

size_t work_items(int32_t rows, int32_t heads, int32_t num_splits) {
    return num_splits > 0 ? static_cast<size_t>(rows) * num_splits : static_cast<size_t>(rq_attention_work_capacity(rows, heads));
}

}  // namespace

extern "C" {

const char* rq_last_error(void) { return g_error; }
const char* rq_version(void) { return "residualquant_b200 0.1 (sm_100a)"; }

int32_t rq_page_width(const RqGroupSpec* spec) { return rq_record_offset(spec, spec ? spec->num_records : 0); }

int32_t rq_record_offset(const RqGroupSpec* spec, int32_t index) {
    const int status = check_spec(spec);
    if (status != RQ_OK) return status;
    if (index < 0 || index > spec->num_records) return fail(RQ_ERR_INVALID_ARGUMENT, "record index %d out of range", index);
    int offset = 0;
    for (int r = 0; r < index; ++r) offset += record_bytes(spec, r);
    return offset;
}

size_t rq_quantize_workspace_bytes(const RqGroupSpec* spec, int64_t num_tokens, int32_t key_kind, int32_t value_kind) {
    // Kept for callers written against the first version of this interface: no rotation kind needs scratch any more.
    (void)spec; (void)num_tokens; (void)key_kind; (void)value_kind;
    return 0;
}

int32_t rq_quantize(const RqQuantizeArgs* a) {
    if (a == nullptr) return fail(RQ_ERR_INVALID_ARGUMENT, "null arguments");
    int status = check_spec(&a->spec);
    if (status != RQ_OK) return status;
    const RqGroupSpec& s = a->spec;
    if (a->num_tokens < 0) return fail(RQ_ERR_INVALID_ARGUMENT, "negative token count");
    if (a->num_tokens == 0) return RQ_OK;  // quantize/launch.cuh:59
    if (a->num_tokens > 0x7fffffff / 16) return fail(RQ_ERR_INVALID_ARGUMENT, "too many tokens in one call");
    const int width = rq_page_width(&s);
    if (a->kv_cache == nullptr || !aligned(a->kv_cache, 16))
        return fail(RQ_ERR_INVALID_ARGUMENT, "16-byte aligned uint8 [2, blocks, heads, page tokens, page width] cache required");
    if (a->num_blocks < 1 || a->plane_stride < a->num_blocks * s.heads * static_cast<int64_t>(s.page_tokens) * width)
        return fail(RQ_ERR_INVALID_ARGUMENT, "plane stride %lld is smaller than one plane of %lld blocks (page width %d)",
                    static_cast<long long>(a->plane_stride), static_cast<long long>(a->num_blocks), width);
    if (a->slot_mapping == nullptr || !aligned(a->slot_mapping, 8))
        return fail(RQ_ERR_INVALID_ARGUMENT, "contiguous int64 slot mapping required");
    if (a->coefficient != RQ_COEFF_UNIT && a->coefficient != RQ_COEFF_NORM && a->coefficient != RQ_COEFF_LS)
        return fail(RQ_ERR_INVALID_ARGUMENT, "unsupported coefficient %d", a->coefficient);
    if (a->chain != RQ_CHAIN_KERNEL && a->chain != RQ_CHAIN_CALIBRATION)
        return fail(RQ_ERR_INVALID_ARGUMENT, "unknown chain %d", a->chain);
    if (a->chain == RQ_CHAIN_CALIBRATION && s.reference_mode != RQ_REFERENCE_ANCHOR)
        return fail(RQ_ERR_UNSUPPORTED, "the calibration chain is defined for the anchor reference mode");
    if ((status = check_rotation(a->key_rotation, "key_rotation")) != RQ_OK) return status;
    if ((status = check_rotation(a->value_rotation, "value_rotation")) != RQ_OK) return status;
    if (a->key_mean != nullptr && !aligned(a->key_mean, 4))
        return fail(RQ_ERR_INVALID_ARGUMENT, "fp32 [records, heads, channels] key mean required");

    rq::QuantizeParams p;
    memset(&p, 0, sizeof(p));
    bool vector_loads = true;
    for (int r = 0; r < s.num_records; ++r) {
        if (a->key[r] == nullptr || a->value[r] == nullptr)
            return fail(RQ_ERR_INVALID_ARGUMENT, "one K/V input per record required (record %d is null)", r);
        if (!aligned(a->key[r], 2) || !aligned(a->value[r], 2) || a->key_stride[r] < s.heads * s.head_dim ||
            a->value_stride[r] < s.heads * s.head_dim)
            return fail(RQ_ERR_INVALID_ARGUMENT, "bf16 [tokens, heads, channels] with packed trailing strides required");
        p.key[r] = static_cast<const __nv_bfloat16*>(a->key[r]);
        p.value[r] = static_cast<const __nv_bfloat16*>(a->value[r]);
        p.key_stride[r] = a->key_stride[r];
        p.value_stride[r] = a->value_stride[r];
        vector_loads = vector_loads && aligned(a->key[r], 16) && aligned(a->value[r], 16) &&
                       a->key_stride[r] % 8 == 0 && a->value_stride[r] % 8 == 0;
        p.bits[r] = s.bits[r];
        p.group[r] = s.group_size[r];
        p.record_offset[r] = rq_record_offset(&s, r);
    }
    p.cache = static_cast<uint8_t*>(a->kv_cache);
    p.plane_stride = a->plane_stride;
    p.slots = a->slot_mapping;
    p.sign[0] = static_cast<const uint32_t*>(a->key_rotation.data);
    p.sign[1] = static_cast<const uint32_t*>(a->value_rotation.data);
    p.rscale[0] = a->key_rotation.scale;
    p.rscale[1] = a->value_rotation.scale;
    p.rotation[0] = a->key_rotation.kind;
    p.rotation[1] = a->value_rotation.kind;
    p.mean = a->key_mean;
    p.num_tokens = static_cast<int>(a->num_tokens);
    p.heads = s.heads;
    p.page_tokens = s.page_tokens;
    p.page_width = width;
    p.num_records = s.num_records;
    p.anchor = s.anchor_index;
    // A single-record group has only its base record, whatever the reference mode (dispatch/schedules.cuh:24-37).
    p.mode = s.num_records == 1 ? RQ_REFERENCE_ANCHOR : s.reference_mode;
    p.coefficient = a->coefficient;
    p.chain = a->chain;
    p.vector_loads = vector_loads ? 1 : 0;
    p.programmatic_launch = programmatic_launch_enabled() && !(a->flags & RQ_FLAG_SERIAL_LAUNCH) ? 1 : 0;
    // Dense learned rotations are applied inside the quantizer CTA (tensor-core product in shared memory).
    for (int plane = 0; plane < 2; ++plane) {
        const RqRotation& rot = plane == 0 ? a->key_rotation : a->value_rotation;
        if (rot.kind != RQ_ROTATION_DENSE_FP16) continue;
        if (a->chain == RQ_CHAIN_CALIBRATION)
            return fail(RQ_ERR_UNSUPPORTED, "the calibration chain needs an invertible structured rotation");
        p.dense_matrix[plane] = static_cast<const __half*>(rot.data);
    }
    const cudaError_t err = rq::launch_quantize(p, s.head_dim, static_cast<cudaStream_t>(a->stream));
    if (err != cudaSuccess) return fail_cuda(err, "quantize launch");
    note_quantize(a->stream, a->kv_cache);
    return RQ_OK;
}

int32_t rq_attention_default_splits(int32_t num_query_rows, int32_t heads, int32_t max_blocks_per_request,
                                    int32_t page_tokens) {
    if (num_query_rows < 1 || heads < 1) return 1;
    const int sms = current_sm_count();
    // Cost model fitted to measurements on B200 (batch 1..64 x 16 heads and 16 x 55 heads, contexts 2k..8k).  A CTA
    // costs its pages plus a fixed overhead worth about 16 pages (prologue, first fetch, merge).  Four CTAs fit on an
    // SM; the grid runs as full waves of 4 per SM plus a tail wave of c = ceil(rest / SMs) per SM, and an SM holding c
    // CTAs delivers 0.45 / 0.85 / 0.92 / 1 of its throughput for c = 1..4 (the kernel is bound by instruction issue, so
    // a tail wave that leaves SMs half empty is what hurts).  Partition counts are powers of two with at least four
    // pages (one per warp) each; ties go to fewer partitions.
    const int64_t base = static_cast<int64_t>(num_query_rows) * heads;
    const int64_t pages = max_blocks_per_request > 0 ? max_blocks_per_request : 1;
    const double tail_cost[5] = {0.0, 1.0 / 0.45, 2.0 / 0.85, 3.0 / 0.92, 4.0};
    int32_t best = 1;
    double best_cost = 0.0;
    for (int32_t candidate = 1; candidate <= 64 && (candidate == 1 || candidate * 4 <= pages); candidate *= 2) {
        const int64_t ctas = base * candidate;
        const int64_t full_waves = ctas / (4LL * sms);
        const int64_t rest = ctas - full_waves * 4LL * sms;
        const int64_t per_sm = (rest + sms - 1) / sms;
        const double waves = 4.0 * static_cast<double>(full_waves) + tail_cost[per_sm];
        const double cost = waves * (static_cast<double>(pages) / candidate + 16.0);
        if (candidate == 1 || cost < best_cost * 0.99) {
            best = candidate;
            best_cost = cost;
        }
    }
    (void)page_tokens;
    return best;
}

int32_t rq_attention_work_capacity(int32_t num_query_rows, int32_t heads) {
    if (num_query_rows < 1 || heads < 1) return 0;
    // Every row is one work item; the spare items are what long rows can be cut into.  One wave of resident CTAs
    // (four per multiprocessor) on top of the rows is as many as the partition choice on the device asks for (CTAs
    // without work still cost a launch slot and a schedule lookup each), fifteen spare items per row is the
    // reference's ceiling (attention/launch.cuh:70-80: sixteen partitions per request), and a single long row among
    // short ones can always have its sixteen.
    const int64_t slots = 4LL * current_sm_count();
    int64_t spare = (slots + heads - 1) / heads;
    if (spare > 15LL * num_query_rows) spare = 15LL * num_query_rows;
    if (spare < 15) spare = 15;
    // A batch whose unsplit rows make between one and about one and a half waves runs a nearly empty second wave; two
    // partitions per row (three waves of half-size CTAs) are measurably faster there (40 rows x 16 heads x 8192 tokens:
    // 236 against 280 us), so such a batch gets room for them.
    const int64_t unsplit = static_cast<int64_t>(num_query_rows) * heads;
    if (unsplit > slots && 5 * unsplit < 8 * slots && spare < num_query_rows) spare = num_query_rows;
    // Beyond that the rows alone fill the GPU for several waves and only an outlier row is ever cut: half a wave of spare
    // items is plenty for it, and every spare CTA that finds no work still costs a slot for a microsecond or two.
    if (5 * unsplit >= 8 * slots) spare = (spare + 1) / 2 < 15 ? 15 : (spare + 1) / 2;
    const int64_t capacity = num_query_rows + spare;
    return capacity > 0x7fffffff / 64 ? 0 : static_cast<int32_t>(capacity);
}

size_t rq_attention_workspace_bytes(int32_t num_query_rows, int32_t heads, int32_t head_dim, int32_t num_splits) {
    if (num_query_rows < 0 || heads < 1 || head_dim < 1 || num_splits < -65536) return 0;
    const size_t counters = counter_bytes(num_query_rows, heads);
    const size_t partials =
        num_splits != 1 ? work_items(num_query_rows, heads, num_splits) * heads * (head_dim + 2) * sizeof(float) : 0;
    return kStatusBytes + counters + round_up(partials, 256);
}

int32_t rq_attention_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
    if (workspace == nullptr || !aligned(workspace, 256) || workspace_bytes < kStatusBytes)
        return fail(RQ_ERR_WORKSPACE, "workspace must be a 256-byte aligned device buffer");
    const cudaError_t err = cudaMemsetAsync(workspace, 0, workspace_bytes, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "workspace init");
    return RQ_OK;
}

int32_t rq_attention_status(const void* workspace, void* stream) {
    if (workspace == nullptr) return fail(RQ_ERR_WORKSPACE, "null workspace");
    int32_t word = 0;
    cudaError_t err = cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost,
                                      static_cast<cudaStream_t>(stream));
    if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "status read");
    if (word != 0) return fail(RQ_ERR_DEVICE_TIMEOUT, "a bounded wait inside the attention kernel gave up");
    return RQ_OK;
}

int32_t rq_attention(const RqAttentionArgs* a) {
    if (a == nullptr) return fail(RQ_ERR_INVALID_ARGUMENT, "null arguments");
    int status = check_spec(&a->spec);
    if (status != RQ_OK) return status;
    const RqGroupSpec& s = a->spec;
    if (a->num_query_rows < 0) return fail(RQ_ERR_INVALID_ARGUMENT, "negative query row count");
    if (a->num_query_rows == 0) return RQ_OK;  // attention/launch.cuh:46
    if (a->loop_index < 0 || a->loop_index >= s.num_records) return fail(RQ_ERR_INVALID_ARGUMENT, "invalid loop index");
    const int64_t row_elems = static_cast<int64_t>(s.heads) * s.head_dim;
    if (a->query == nullptr || a->key == nullptr || a->value == nullptr || a->output == nullptr)
        return fail(RQ_ERR_INVALID_ARGUMENT, "Q/K/V/output must be device pointers");
    if (a->query_stride < row_elems || a->key_stride < row_elems || a->value_stride < row_elems ||
        a->output_stride < row_elems)
        return fail(RQ_ERR_INVALID_ARGUMENT, "bf16 [tokens, heads, channels] with packed trailing strides required");
    if (!aligned(a->query, 8) || !aligned(a->key, 8) || a->query_stride % 4 != 0 || a->key_stride % 4 != 0)
        return fail(RQ_ERR_INVALID_ARGUMENT, "Q/K addresses and token strides must be 8-byte aligned");
    if (!aligned(a->value, 2) || !aligned(a->output, 2))
        return fail(RQ_ERR_INVALID_ARGUMENT, "V/output must be bf16 pointers");
    const int width = rq_page_width(&s);
    if (a->kv_cache == nullptr || !aligned(a->kv_cache, 16) || a->plane_stride % 16 != 0)
        return fail(RQ_ERR_INVALID_ARGUMENT, "16-byte aligned contiguous uint8 KV cache required");
    if (a->num_blocks < 1 || a->plane_stride < a->num_blocks * s.heads * static_cast<int64_t>(s.page_tokens) * width)
        return fail(RQ_ERR_INVALID_ARGUMENT, "plane stride %lld is smaller than one plane of %lld blocks (page width %d)",
                    static_cast<long long>(a->plane_stride), static_cast<long long>(a->num_blocks), width);
    if (a->query_start_loc == nullptr || a->seq_lens == nullptr || a->block_table == nullptr || a->num_requests < 1)
        return fail(RQ_ERR_INVALID_ARGUMENT, "int32 query starts [requests+1], sequence lengths [requests] and page table required");
    if (a->block_table_stride < a->max_blocks_per_request || a->max_blocks_per_request < 0)
        return fail(RQ_ERR_INVALID_ARGUMENT, "int32 page table with packed rows required");
    if (a->key_mean != nullptr && !aligned(a->key_mean, 16))
        return fail(RQ_ERR_INVALID_ARGUMENT, "16-byte aligned contiguous fp32 key mean required");
    if ((status = check_rotation(a->key_rotation, "key_rotation")) != RQ_OK) return status;
    if ((status = check_rotation(a->value_rotation, "value_rotation")) != RQ_OK) return status;
    const bool adjacent = s.reference_mode == RQ_REFERENCE_ADJACENT && s.num_records > 1;
    if (adjacent) {
        if (s.num_records > 4)
            return fail(RQ_ERR_UNSUPPORTED, "No compiled packed CUDA kernel for adjacent groups of more than 4 records");
        for (int r = 0; r <= a->loop_index; ++r)
            if (s.bits[r] == 4 && s.group_size[r] != 32)
                return fail(RQ_ERR_UNSUPPORTED, "No compiled packed CUDA kernel for an INT4 record with groups of %d",
                            s.group_size[r]);
    }

    rq::AttentionVariant v;
    v.head_dim = s.head_dim;
    v.anchor_bits = s.bits[s.anchor_index];
    v.anchor_group = s.group_size[s.anchor_index];
    const bool anchor_loop = a->loop_index == s.anchor_index;
    v.residual_bits = anchor_loop ? 0 : s.bits[a->loop_index];
    v.residual_group = anchor_loop ? 32 : s.group_size[a->loop_index];
    v.page_tokens = s.page_tokens;
    v.has_mean = a->key_mean != nullptr;
    v.adjacent = adjacent;
    if (!rq::attention_variant_available(v))
        return fail(RQ_ERR_UNSUPPORTED,
                    "No compiled packed CUDA kernel for heads=%d, head_dim=%d, anchor=(%d,%d), loop record=(%d,%d), "
                    "has_mean=%d, page_tokens=%d",
                    s.heads, s.head_dim, v.anchor_bits, v.anchor_group, v.residual_bits, v.residual_group,
                    int(v.has_mean), s.page_tokens);

    // 0 = the kernel cuts every row into partitions proportional to its length; n > 0 = exactly n per row
    const int splits = a->num_splits;
    if (splits < -65536 || splits > 1024) return fail(RQ_ERR_INVALID_ARGUMENT, "num_splits %d outside -65536..1024", splits);
    const int capacity = splits <= 0 ? rq_attention_work_capacity(a->num_query_rows, s.heads) : 0;
    if (splits <= 0 && capacity < a->num_query_rows) return fail(RQ_ERR_INVALID_ARGUMENT, "too many query rows in one call");
    if (static_cast<int64_t>(work_items(a->num_query_rows, s.heads, splits)) * s.heads > 0x7fffffffLL)
        return fail(RQ_ERR_INVALID_ARGUMENT, "grid too large");
    const size_t need = rq_attention_workspace_bytes(a->num_query_rows, s.heads, s.head_dim, splits);
    if (a->workspace == nullptr || !aligned(a->workspace, 256) || a->workspace_bytes < need)
        return fail(RQ_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) required, got %zu", need, a->workspace_bytes);

    rq::AttentionParams p;
    memset(&p, 0, sizeof(p));
    p.query = static_cast<const __nv_bfloat16*>(a->query);
    p.key = static_cast<const __nv_bfloat16*>(a->key);
    p.value = static_cast<const __nv_bfloat16*>(a->value);
    p.output = static_cast<__nv_bfloat16*>(a->output);
    p.query_stride = a->query_stride;
    p.key_stride = a->key_stride;
    p.value_stride = a->value_stride;
    p.output_stride = a->output_stride;
    p.cache = static_cast<const uint8_t*>(a->kv_cache);
    p.plane_stride = a->plane_stride;
    p.query_start_loc = a->query_start_loc;
    p.seq_lens = a->seq_lens;
    p.block_table = a->block_table;
    p.num_rows = a->num_query_rows;
    p.num_requests = a->num_requests;
    p.block_table_stride = a->block_table_stride;
    p.max_blocks = a->max_blocks_per_request;
    p.key_sign = a->key_rotation.kind == RQ_ROTATION_SIGNED_HADAMARD ? static_cast<const uint32_t*>(a->key_rotation.data) : nullptr;
    p.value_sign = a->value_rotation.kind == RQ_ROTATION_SIGNED_HADAMARD ? static_cast<const uint32_t*>(a->value_rotation.data) : nullptr;
    p.key_rscale = a->key_rotation.scale;
    p.value_rscale = a->value_rotation.scale;
    p.mean = a->key_mean;
    p.heads = s.heads;
    p.page_width = width;
    p.anchor_offset = rq_record_offset(&s, s.anchor_index);
    p.residual_offset = rq_record_offset(&s, a->loop_index);
    p.anchor_index = s.anchor_index;
    p.loop_index = a->loop_index;
    if (adjacent) {
        p.chain_count = a->loop_index + 1;
        for (int r = 0; r < p.chain_count; ++r) {
            p.chain_bits[r] = s.bits[r];
            p.chain_group[r] = s.group_size[r];
        }
        for (int r = 0; r <= p.chain_count; ++r) p.chain_offset[r] = rq_record_offset(&s, r);
    }
    p.splits = splits;
    p.capacity = capacity;
    p.sm_count = current_sm_count();
    p.programmatic_launch = programmatic_launch_enabled() && !(a->flags & RQ_FLAG_SERIAL_LAUNCH) ? 1 : 0;
    const bool just_written = take_recent_write(a->stream, a->kv_cache);
    p.early_start = p.programmatic_launch && (a->flags & RQ_FLAG_STABLE_METADATA) && !just_written ? 1 : 0;
    uint8_t* base = static_cast<uint8_t*>(a->workspace);
    p.status = reinterpret_cast<int32_t*>(base);
    p.counters = reinterpret_cast<int32_t*>(base + kStatusBytes);
    p.partials = reinterpret_cast<float*>(base + kStatusBytes + counter_bytes(a->num_query_rows, s.heads));
    // a dense key rotation is applied to the query row inside the attention kernel's prologue
    if (a->key_rotation.kind == RQ_ROTATION_DENSE_FP16) p.query_matrix = static_cast<const __half*>(a->key_rotation.data);
    if (a->value_rotation.kind == RQ_ROTATION_DENSE_FP16) p.value_matrix = static_cast<const __half*>(a->value_rotation.data);
    if (a->num_peers != 0) {
        if (a->num_peers < 0 || a->num_peers > RQ_MAX_PEERS)
            return fail(RQ_ERR_INVALID_ARGUMENT, "num_peers %d outside 0..%d", a->num_peers, RQ_MAX_PEERS);
        if (a->gather_head_offset < 0 || a->gather_stride < (static_cast<int64_t>(a->gather_head_offset) + s.heads) * s.head_dim)
            return fail(RQ_ERR_INVALID_ARGUMENT, "gathered rows of %lld elements cannot hold heads %d..%d",
                        static_cast<long long>(a->gather_stride), a->gather_head_offset, a->gather_head_offset + s.heads);
        for (int i = 0; i < a->num_peers; ++i) {
            if (a->peer_output[i] == nullptr || !aligned(a->peer_output[i], 2))
                return fail(RQ_ERR_INVALID_ARGUMENT, "peer_output[%d] must be a mapped bf16 buffer", i);
            p.peer_output[i] = static_cast<__nv_bfloat16*>(a->peer_output[i]);
        }
        p.num_peers = a->num_peers;
        p.gather_head_offset = a->gather_head_offset;
        p.gather_stride = a->gather_stride;
        if (a->flags & (RQ_FLAG_GATHER_PUBLISH | RQ_FLAG_GATHER_WAIT | RQ_FLAG_GATHER_COMPLETE)) {
            if (a->gather_state == nullptr || !aligned(a->gather_state, 8) || a->gather_rank < 0 || a->gather_rank >= a->num_peers)
                return fail(RQ_ERR_INVALID_ARGUMENT, "the gather signal needs this rank's state block and a rank below num_peers");
            for (int i = 0; i < a->num_peers; ++i) {
                if (a->peer_flags[i] == nullptr || !aligned(a->peer_flags[i], 4))
                    return fail(RQ_ERR_INVALID_ARGUMENT, "peer_flags[%d] must be a mapped uint32 array", i);
                p.gather_flags[i] = static_cast<uint32_t*>(a->peer_flags[i]);
            }
            p.gather_state = static_cast<uint32_t*>(a->gather_state);
            p.gather_rank = a->gather_rank;
            p.gather_complete = (a->flags & RQ_FLAG_GATHER_COMPLETE) ? 1 : 0;
            p.gather_publish = (a->flags & (RQ_FLAG_GATHER_PUBLISH | RQ_FLAG_GATHER_COMPLETE)) ? 1 : 0;
            p.gather_wait = (a->flags & RQ_FLAG_GATHER_WAIT) ? 1 : 0;
            p.gather_timeout_ns = a->gather_timeout_ns ? a->gather_timeout_ns : 2000000000ull;
        }
    }
    const cudaError_t err = rq::launch_attention(v, p, static_cast<cudaStream_t>(a->stream));
    if (err != cudaSuccess) return fail_cuda(err, "attention launch");
    return RQ_OK;
}

// ---- attention without any allocation: scratch compiled into the library -------------------------------
// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address the kernel
// needs comes from cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[RQ_STATIC_SCRATCH_BYTES];

// Device address of the built-in buffer on the current device.  The cache is process-wide (one slot per device), so
// the lookup runs once per device whichever thread gets there first.
static int static_scratch_address(void** address) {
    static std::atomic<void*> addresses[64];
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return fail_cuda(err, "cudaGetDevice");
    if (device < 0 || device >= 64) return fail(RQ_ERR_INVALID_ARGUMENT, "device index %d not supported", device);
    void* known = addresses[device].load(std::memory_order_acquire);
    if (known == nullptr) {
        err = cudaGetSymbolAddress(&known, g_static_scratch);
        if (err != cudaSuccess) return fail_cuda(err, "cudaGetSymbolAddress(static scratch)");
        addresses[device].store(known, std::memory_order_release);
    }
    *address = known;
    return RQ_OK;
}

int32_t rq_attention_noalloc(const RqAttentionArgs* a) {
    if (a == nullptr) return fail(RQ_ERR_INVALID_ARGUMENT, "null arguments");
    void* scratch = nullptr;
    int status = static_scratch_address(&scratch);
    if (status != RQ_OK) return status;
    if ((status = check_spec(&a->spec)) != RQ_OK) return status;  // a bad spec is reported as such, not as a size problem
    if (a->num_query_rows <= 0) return rq_attention(a);            // nothing to launch; reuse the argument checks
    if (a->num_splits < -65536 || a->num_splits > 1024)
        return fail(RQ_ERR_INVALID_ARGUMENT, "num_splits %d outside -65536..1024", a->num_splits);
    const size_t need = rq_attention_workspace_bytes(a->num_query_rows, a->spec.heads, a->spec.head_dim, a->num_splits);
    if (need == 0 || need > RQ_STATIC_SCRATCH_BYTES)
        return fail(RQ_ERR_WORKSPACE,
                    "this shape needs %zu bytes of scratch; the built-in buffer holds %u (use rq_attention with a "
                    "caller-provided workspace, or fewer rows per call)", need, RQ_STATIC_SCRATCH_BYTES);
    // The buffer keeps whatever the previous call left: the status word and the arrival counters must start at zero.
    const size_t clear = kStatusBytes + round_up(static_cast<size_t>(a->num_query_rows) * a->spec.heads * sizeof(int32_t), 256);
    const cudaError_t err = cudaMemsetAsync(scratch, 0, clear, static_cast<cudaStream_t>(a->stream));
    if (err != cudaSuccess) return fail_cuda(err, "clearing the static scratch");
    RqAttentionArgs copy = *a;
    copy.workspace = scratch;
    copy.workspace_bytes = RQ_STATIC_SCRATCH_BYTES;
    copy.flags |= RQ_FLAG_SERIAL_LAUNCH;  // the kernel follows a memset of its own counters: plain stream order
    return rq_attention(&copy);
}

int32_t rq_attention_noalloc_status(void* stream) {
    void* scratch = nullptr;
    const int status = static_scratch_address(&scratch);
    if (status != RQ_OK) return status;
    return rq_attention_status(scratch, stream);
}

void rq_set_programmatic_launch(int32_t enabled) { g_programmatic.store(enabled ? 1 : 0, std::memory_order_relaxed); }

// ---- node-level barrier for the fused head gather ------------------------------------------------------------
int32_t rq_peer_barrier(const RqPeerBarrierArgs* a) {
    if (a == nullptr) return fail(RQ_ERR_INVALID_ARGUMENT, "null arguments");
    if (a->world < 1 || a->world > RQ_MAX_PEERS || a->rank < 0 || a->rank >= a->world)
        return fail(RQ_ERR_INVALID_ARGUMENT, "rank %d of %d: at most %d GPUs of one node", a->rank, a->world, RQ_MAX_PEERS);
    if (a->state == nullptr || !aligned(a->state, 8)) return fail(RQ_ERR_INVALID_ARGUMENT, "barrier state must be device memory");
    rq::PeerBarrierParams p;
    memset(&p, 0, sizeof(p));
    for (int i = 0; i < a->world; ++i) {
        if (a->flags[i] == nullptr || !aligned(a->flags[i], 4))
            return fail(RQ_ERR_INVALID_ARGUMENT, "flags[%d] must be a mapped uint32 array", i);
        p.flags[i] = static_cast<uint32_t*>(a->flags[i]);
    }
    p.state = static_cast<uint32_t*>(a->state);
    p.world = a->world;
    p.rank = a->rank;
    p.timeout_ns = a->timeout_ns ? a->timeout_ns : 2000000000ull;
    p.wait_only = a->wait_only ? 1 : 0;
    p.programmatic_launch = programmatic_launch_enabled() ? 1 : 0;
    const cudaError_t err = rq::launch_peer_barrier(p, static_cast<cudaStream_t>(a->stream));
    if (err != cudaSuccess) return fail_cuda(err, "peer barrier launch");
    return RQ_OK;
}

int32_t rq_peer_alloc(size_t bytes, void** pointer) {
    if (pointer == nullptr || bytes == 0) return fail(RQ_ERR_INVALID_ARGUMENT, "a size and a place for the pointer required");
    static_assert(RQ_PEER_HANDLE_BYTES == sizeof(cudaIpcMemHandle_t), "handle size");
    void* p = nullptr;
    cudaError_t err = cudaMalloc(&p, bytes);
    if (err != cudaSuccess) return fail_cuda(err, "cudaMalloc(peer buffer)");
    err = cudaMemset(p, 0, bytes);
    if (err != cudaSuccess) {
        cudaFree(p);
        return fail_cuda(err, "clearing the peer buffer");
    }
    *pointer = p;
    return RQ_OK;
}

int32_t rq_peer_free(void* pointer) {
    const cudaError_t err = cudaFree(pointer);
    return err == cudaSuccess ? RQ_OK : fail_cuda(err, "cudaFree(peer buffer)");
}

int32_t rq_peer_export(const void* pointer, unsigned char* handle) {
    if (pointer == nullptr || handle == nullptr) return fail(RQ_ERR_INVALID_ARGUMENT, "null pointer");
    cudaIpcMemHandle_t h;
    const cudaError_t err = cudaIpcGetMemHandle(&h, const_cast<void*>(pointer));
    if (err != cudaSuccess) return fail_cuda(err, "cudaIpcGetMemHandle");
    memcpy(handle, &h, sizeof(h));
    return RQ_OK;
}

int32_t rq_peer_open(const unsigned char* handle, void** mapped) {
    if (handle == nullptr || mapped == nullptr) return fail(RQ_ERR_INVALID_ARGUMENT, "null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    const cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) return fail_cuda(err, "cudaIpcOpenMemHandle");
    *mapped = p;
    return RQ_OK;
}

int32_t rq_peer_close(void* mapped) {
    const cudaError_t err = cudaIpcCloseMemHandle(mapped);
    return err == cudaSuccess ? RQ_OK : fail_cuda(err, "cudaIpcCloseMemHandle");
}

int32_t rq_peer_barrier_status(const void* state, void* stream) {
    if (state == nullptr) return fail(RQ_ERR_INVALID_ARGUMENT, "null barrier state");
    uint32_t words[2] = {0u, 0u};
    cudaError_t err = cudaMemcpyAsync(words, state, sizeof(words), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
    if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "reading the barrier state");
    if (words[1] != 0u) return fail(static_cast<int32_t>(words[1]), "a peer did not reach barrier %u in time", words[0]);
    return RQ_OK;
}

}  // extern "C"
