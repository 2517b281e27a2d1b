#!/usr/bin/env python
"""Benchmark of the packed-KV hot path: decode tokens/s of an Ouro-1.4B-shaped stack of KV groups.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one decode step of the hot path for the whole stack: for each of `layers` physical layers, the
packed paged decode attention of the 4 loops (4 launches) and the KV-write quantizer of the group (1 launch),
captured once in a CUDA graph and replayed.  Sequence lengths and slot mappings advance on the device inside
the graph, as they do under vLLM's decode capture.  Workload (standalone kernel sweep, no model): 16 heads x 128,
vLLM block size 16, INT4 g32 anchor in the last loop + INT2 g32 residuals, batch 64 at context 8192; seeded
synthetic K/V (N(0,1) x log-normal channel scales, 4 outlier channels x8 per head, earlier loops
0.9*anchor + 0.3*N(0,1)), signed-Hadamard rotation, block tables randomly permuted over the page pool.

Printed JSON line:
  value     tokens/s with every input resident in HBM (CUDA-event time of K graph replays, max over ranks)
  e2e       tokens/s when each step also copies its q/k/v rows from pinned host memory and reads the outputs back
  roofline  the dominant kernel (attention of a residual loop): algorithmic packed-KV bytes per launch / CUDA-event
            time per launch, against the measured HBM copy bandwidth of MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle (a restatement of the reference's algorithm) timed on a bounded sample, scaled
            to the same unit

`--impl reference` times that CPU restatement alone (the reference has no native CPU path and its PyTorch
code cannot travel to the benchmark machine).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"
HEADS, HEAD_DIM, PAGE = 16, 128, 16
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=8)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--batch", type=int, default=64)
    p.add_argument("--context", type=int, default=8192)
    p.add_argument("--group", type=int, default=32, choices=[16, 32])
    p.add_argument("--layers", type=int, default=24)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--head-dim", type=int, default=128, choices=[128, 96])
    p.add_argument("--page", type=int, default=16, choices=[16, 32], help="vLLM block size")
    p.add_argument("--shard", default="sequences", choices=["sequences", "heads"],
                   help="sequences: every rank owns its own batch (weak scaling, no collective); heads: every rank holds "
                        "all sequences but only its KV heads and all-gathers the attention output (strong scaling)")
    p.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                   help="with --shard heads: fused = the attention kernel stores into every GPU's gathered output over "
                        "NVLink and a barrier kernel follows (captured in the graph); nccl = one all-gather per call, eager")
    p.add_argument("--splits", type=int, default=0, help="force the number of KV partitions per row (0 = library default)")
    p.add_argument("--compare-bf16", action="store_true",
                   help="also time a BF16-KV decode attention (torch SDPA, contiguous KV) of one layer's 4 loops")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--sweep", action="store_true", help="also time attention alone over the batch x context grid")
    return p.parse_args()


def record_bytes(bits, group, dim=None):
    dim = HEAD_DIM if dim is None else dim
    return dim * bits // 8 + 2 * dim // group + 2


def attention_bytes(batch, context, group, loop_is_anchor, heads=None, dim=None):
    """Algorithmic bytes of one attention launch: every cached token's anchor record without its alpha column,
    plus the loop's own residual record, for K and V; plus q, live k, live v, out in bf16."""
    heads = HEADS if heads is None else heads
    dim = HEAD_DIM if dim is None else dim
    anchor = record_bytes(4, 32, dim) - 2
    per_token = anchor if loop_is_anchor else anchor + record_bytes(2, group, dim)
    return batch * (context - 1) * heads * 2 * per_token + batch * heads * dim * 8


def quantize_bytes(tokens, group, heads=None, dim=None):
    heads = HEADS if heads is None else heads
    dim = HEAD_DIM if dim is None else dim
    width = 3 * record_bytes(2, group, dim) + record_bytes(4, 32, dim)
    return 2 * 4 * tokens * heads * dim * 2 + 2 * tokens * heads * width


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------------------------------------
# CPU restatement (oracle) timed on a bounded sample
# ----------------------------------------------------------------------------------------------------------


def cpu_sample(context, group, layers, batch, sample_context=2048, seed=0):
    """One sequence, one layer, context `sample_context`: quantize of the whole prompt (K and V, 4 loops) and the
    decode attention of the 4 loops.  Returns (tokens/s scaled to the full workload, description)."""
    from oracle import rq_oracle as O
    from tests import helpers

    case = helpers.make_case(seed, HEAD_DIM, HEADS, [sample_context], group, PAGE)
    t0 = time.perf_counter()
    cache = helpers.oracle_cache(case)
    t1 = time.perf_counter()
    for loop in range(4):
        helpers.oracle_attention(case, cache, loop)
    t2 = time.perf_counter()
    quantize_per_token = (t1 - t0) / max(1, sample_context - 1)
    attention_per_cached_token = (t2 - t1) / max(1, sample_context - 1)
    # one decode step of the full workload for ONE sequence: `layers` x (4 attentions over `context` + 1 write)
    step_seconds = layers * (attention_per_cached_token * (context - 1) + quantize_per_token)
    description = (
        f"numpy oracle, 1 sequence x 1 layer x context {sample_context} (quantize {t1 - t0:.2f}s, "
        f"4 attentions {t2 - t1:.2f}s), scaled linearly to {layers} layers x context {context}"
    )
    return 1.0 / step_seconds, description, (t2 - t0)


def _reference_worker(job):
    context, group, layers, batch, sample_context, seed = job
    import numpy  # noqa: F401  (each worker is a fresh interpreter)
    value, description, seconds = cpu_sample(context, group, layers, batch, sample_context, seed)
    return value, description, seconds


def run_reference(args):
    """The CPU restatement on every host core: one worker process per core, each running the hot path of one
    sequence (quantize of a 512-token prompt for one layer + the 4 decode attentions), scaled to the workload's unit."""
    import concurrent.futures

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = max(1, min(os.cpu_count() or 1, 64))
    values, description = [], ""
    begin = time.perf_counter()
    with concurrent.futures.ProcessPoolExecutor(max_workers=cores) as pool:
        for i in range(args.warmup + args.steps):
            jobs = [(args.context, args.group, args.layers, args.batch, 512, 1000 * i + w) for w in range(cores)]
            t0 = time.perf_counter()
            results = list(pool.map(_reference_worker, jobs))
            wall = time.perf_counter() - t0
            description = results[0][1]
            # `cores` sequences advanced concurrently; each needs sum(seconds)/cores of wall time per sample
            per_sequence = [1.0 / r[0] for r in results]            # scaled step seconds of one sequence
            busy = sum(r[2] for r in results)
            stretch = wall * cores / busy if busy > 0 else 1.0      # oversubscription / turbo effects
            step_seconds = statistics.mean(per_sequence) * stretch
            if i >= args.warmup:
                values.append(cores / step_seconds)
    elapsed = time.perf_counter() - begin
    value = statistics.median(values)
    sample = f"{cores} worker processes x ({description})"
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1000.0 * elapsed / max(1, args.warmup + args.steps),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def workload_config(args):
    return {
        "workload": f"config1 kernel sweep point: batch {args.batch} x context {args.context}, INT2 g{args.group} "
                    f"residuals + INT4 g32 anchor, {args.layers} layers x 4 loops, {args.heads} heads x {args.head_dim}, block {args.page}, "
                    "CUDA-graph decode step (4 attention + 1 quantize launch per layer)"
                    + ("" if args.shard != "heads" else
                       "; KV heads sharded over the ranks, output rows stored into every GPU's gathered buffer by the attention "
                       "kernel + one barrier kernel per call, captured in the graph" if args.gather == "fused" else
                       "; KV heads sharded over the ranks, one NCCL all-gather of the output per attention call, eager step"),
        "batch_per_gpu": args.batch,
        "sharding": args.shard,
        "context": args.context,
        "layers": args.layers,
        "l2": "inputs larger than L2 (each layer's packed cache is read once per step)",
    }


# ----------------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------------


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        clocks, max_clocks, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in out.strip().splitlines():
            cells = [c.strip() for c in row.split(",")]
            if len(cells) < 9:
                continue
            try:
                clocks.append(float(cells[1]))
                max_clocks.append(float(cells[2]))
            except ValueError:
                continue
            for name, cell in zip(names, cells[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(max_clocks), "reasons": sorted(reasons),
                "samples": len(clocks)}


def build_stack(args, device, torch):
    """Packed caches of `layers` layers for `batch` sequences of `context` tokens (+ head room), filled by the
    quantizer kernel from seeded synthetic rows; every layer shares one block table, as under vLLM."""
    from residualquant_b200 import _cuda, rotation, synth

    records = [[2, args.group]] * 3 + [[4, 32]]
    width = 3 * record_bytes(2, args.group) + record_bytes(4, 32)
    head_room = 128
    blocks_per_seq = (args.context + head_room + PAGE - 1) // PAGE
    num_blocks = args.batch * blocks_per_seq + 1
    rng = np.random.default_rng(1234 + int(os.environ.get("RANK", "0")))
    pool = rng.permutation(num_blocks - 1) + 1          # block 0 stays unused, like vLLM's null block
    table_np = pool.reshape(args.batch, blocks_per_seq).astype(np.int32)
    block_table = torch.from_numpy(table_np).to(device)
    key_rot = rotation.signed_hadamard(synth.signs(rng, HEADS, HEAD_DIM), float(synth.fp16_rsqrt(HEAD_DIM)), device)
    value_rot = rotation.signed_hadamard(synth.signs(rng, HEADS, HEAD_DIM), float(synth.fp16_rsqrt(HEAD_DIM)), device)

    gen = torch.Generator(device=device)
    gen.manual_seed(99 + int(os.environ.get("RANK", "0")))
    channel_scale = torch.exp(0.5 * torch.randn(HEADS, HEAD_DIM, device=device, generator=gen))
    outlier = torch.ones(HEADS, HEAD_DIM, device=device)
    for h in range(HEADS):
        outlier[h, torch.randperm(HEAD_DIM, device=device, generator=gen)[:4]] = 8.0
    channel_scale = channel_scale * outlier

    def rows(tokens):
        anchor = torch.randn(tokens, HEADS, HEAD_DIM, device=device, generator=gen) * channel_scale
        loops = [(0.9 * anchor + 0.3 * torch.randn(tokens, HEADS, HEAD_DIM, device=device, generator=gen)).bfloat16()
                 for _ in range(3)]
        return loops + [anchor.bfloat16()]

    caches = [torch.zeros((2, num_blocks, HEADS, PAGE, width), dtype=torch.uint8, device=device)]
    # fill layer 0 sequence by sequence, then clone it into the other layers
    positions = torch.arange(args.context, device=device)
    for b in range(args.batch):
        slots = block_table[b, positions // PAGE].long() * PAGE + positions % PAGE
        k, v = rows(args.context), rows(args.context)
        _cuda.quantize(list(zip(k, v)), caches[0], slots, key_rot, None, None, records, "anchor", 3, "ls")
    torch.cuda.synchronize(device)
    for _ in range(1, args.layers):
        caches.append(caches[0].clone())
    return {
        "records": records, "caches": caches, "block_table": block_table, "key_rot": key_rot, "value_rot": value_rot,
        "rows": rows, "width": width,
    }


def run_gpu(args):
    import torch
    import torch.distributed as dist

    from residualquant_b200 import _cuda, sharding
    from residualquant_b200 import build as kernel_build

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the kernels have no CPU fallback")
    if rank == 0:
        kernel_build.build()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        dist.barrier()
    else:
        kernel_build.build()

    global HEADS
    heads_total = args.heads
    shard_heads = args.shard == "heads"
    if shard_heads:
        HEADS = sharding.shard_counts(heads_total, world)[rank]   # this rank's slice of every cache and of q/k/v
        if HEADS == 0:
            raise RuntimeError("more ranks than KV heads")
    replicas = 1 if shard_heads else world                          # independent copies of the batch in the job
    B, L, layers = args.batch, args.context, args.layers
    _cuda.set_attention_splits(args.splits)
    stack = build_stack(args, device, torch)
    records, caches = stack["records"], stack["caches"]
    # The model's weights absorb the value rotation in the served configuration (weights.py:9-37 of the reference),
    # so the kernels see value_rotation=None and V arrives rotated.
    key_rot = stack["key_rot"]
    block_table = stack["block_table"]

    # per (layer, loop) inputs of a step, device resident
    q = torch.randn(layers, 4, B, HEADS, HEAD_DIM, device=device).bfloat16()
    live = stack["rows"](B * layers)
    k_live = torch.stack([r.view(layers, B, HEADS, HEAD_DIM) for r in live], dim=1).contiguous()   # [layers, 4, B, H, D]
    live = stack["rows"](B * layers)
    v_live = torch.stack([r.view(layers, B, HEADS, HEAD_DIM) for r in live], dim=1).contiguous()
    out = torch.zeros_like(q)
    qsl = torch.arange(B + 1, dtype=torch.int32, device=device)
    seq_lens = torch.full((B,), L, dtype=torch.int32, device=device)
    slot_mapping = torch.zeros(B, dtype=torch.int64, device=device)
    batch_index = torch.arange(B, device=device)

    def advance():
        # position of the live token = seq_len - 1; its slot is where this step's quantize writes
        position = (seq_lens - 1).long()
        slot_mapping.copy_(block_table[batch_index, position // PAGE].long() * PAGE + position % PAGE)

    gathered = [None]
    # Head sharding: the output projection needs every head.  "fused": the attention kernel stores its rows into every
    # GPU's gathered buffer over NVLink and a barrier kernel follows (graph capturable); "nccl": one all-gather per call.
    fused_gather = sharding.HeadGather(B, heads_total, HEAD_DIM, device) if shard_heads and args.gather == "fused" else None

    def hot_path():
        for layer in range(layers):
            for loop in range(4):
                if fused_gather is not None:
                    _cuda.attention(q[layer, loop], k_live[layer, loop], v_live[layer, loop], caches[layer],
                                    out[layer, loop], qsl, seq_lens, block_table, key_rot, None, None, records,
                                    "anchor", 3, loop, gather=fused_gather, gather_buffer=loop % 2)
                    fused_gather.barrier()
                    continue
                _cuda.attention(q[layer, loop], k_live[layer, loop], v_live[layer, loop], caches[layer], out[layer, loop],
                                qsl, seq_lens, block_table, key_rot, None, None, records, "anchor", 3, loop)
                if shard_heads:
                    gathered[0] = sharding.gather_heads(out[layer, loop], heads_total)
            _cuda.quantize([(k_live[layer, i], v_live[layer, i]) for i in range(4)], caches[layer], slot_mapping,
                           key_rot, None, None, records, "anchor", 3, "ls")

    def step_body():
        advance()
        hot_path()
        seq_lens.add_(1)

    stream = torch.cuda.Stream(device)

    def join_default_stream():
        """Everything queued on the default stream (input tensors, lengths, tables) is complete before the side stream
        reads it: a kernel that saw half-initialised lengths or block ids would read outside the cache."""
        stream.wait_stream(torch.cuda.current_stream(device))

    join_default_stream()
    with torch.cuda.stream(stream):
        step_body()                      # eager warm-up: workspace, per-variant attributes
    stream.synchronize()
    seq_lens.fill_(L)
    if shard_heads and world > 1 and fused_gather is None:
        # The step contains NCCL all-gathers; it is replayed eagerly rather than from a captured graph.
        class _Eager:
            @staticmethod
            def replay():
                step_body()
        graph = _Eager()
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step_body()
    seq_lens.fill_(L)
    torch.cuda.synchronize(device)
    launches_per_step = layers * (9 if fused_gather is not None else 5)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, steps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        join_default_stream()
        with torch.cuda.stream(stream):
            start.record(stream)
            for _ in range(steps):
                fn()
            stop.record(stream)
        stop.synchronize()
        barrier()
        return sharding.max_over_ranks(start.elapsed_time(stop), device)

    sampler = ClockSampler(local_rank)
    # ---------------- device-resident throughput ----------------
    join_default_stream()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            graph.replay()
    if rank == 0:
        sampler.start()
    ms = timed(graph.replay, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    if fused_gather is not None:
        # the gathered rows of the last call must equal an NCCL all-gather of every rank's own output
        fused_gather.check()
        last = out[layers - 1, 3]
        expected = sharding.gather_heads(last, heads_total)
        if not torch.equal(fused_gather.gathered(3 % 2), expected):
            raise RuntimeError("fused head gather differs from the all-gathered outputs")
    value = replicas * B * args.steps / (ms * 1e-3)

    # ---------------- end to end: host rows in, outputs back ----------------
    seq_lens.fill_(L)
    host_q = torch.empty(q.shape, dtype=q.dtype).pin_memory().copy_(q)
    host_k = torch.empty(k_live.shape, dtype=q.dtype).pin_memory().copy_(k_live)
    host_v = torch.empty(v_live.shape, dtype=q.dtype).pin_memory().copy_(v_live)
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    host_lens = torch.full((B,), L, dtype=torch.int32).pin_memory()
    h2d = host_q.numel() * 2 * 3 + host_lens.numel() * 4
    d2h = host_out.numel() * 2

    def e2e_step():
        q.copy_(host_q, non_blocking=True)
        k_live.copy_(host_k, non_blocking=True)
        v_live.copy_(host_v, non_blocking=True)
        seq_lens.copy_(host_lens, non_blocking=True)
        graph.replay()
        host_out.copy_(out, non_blocking=True)
        host_lens.add_(1)

    join_default_stream()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            e2e_step()
    stream.synchronize()
    host_lens.fill_(L)
    ms_e2e = timed(e2e_step, args.steps)
    e2e_value = replicas * B * args.steps / (ms_e2e * 1e-3)

    # ---------------- dominant kernel alone: attention of a residual loop, one launch per layer ----------------
    seq_lens.fill_(L)

    def attention_only(loop):
        def run():
            for layer in range(layers):
                _cuda.attention(q[layer, loop], k_live[layer, loop], v_live[layer, loop], caches[layer], out[layer, loop],
                                qsl, seq_lens, block_table, key_rot, None, None, records, "anchor", 3, loop)
        return run

    def graph_timed(fn, replays):
        """Capture `fn` once (after an eager warm-up) and time `replays` replays: per-kernel device time without
        the Python launch overhead of eager calls."""
        join_default_stream()
        with torch.cuda.stream(stream):
            fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        timed(g.replay, 1)
        return timed(g.replay, replays)

    reps = max(3, 48 // layers)
    ms_res = graph_timed(attention_only(0), reps) / (reps * layers)
    ms_anchor = graph_timed(attention_only(3), reps) / (reps * layers)
    bytes_res = attention_bytes(B, L, args.group, False)
    bytes_anchor = attention_bytes(B, L, args.group, True)
    peak, peak_kind = measured_peak()
    achieved = bytes_res / (ms_res * 1e-3) / 1e9

    def quantize_only():
        for layer in range(layers):
            _cuda.quantize([(k_live[layer, i], v_live[layer, i]) for i in range(4)], caches[layer], slot_mapping,
                           key_rot, None, None, records, "anchor", 3, "ls")
    ms_quant = graph_timed(quantize_only, reps) / (reps * layers)

    # prefill-sized write: two full prompts (2 x context tokens) of layer 0 re-quantized in one call
    prefill_tokens = min(2, B) * L
    pk, pv = stack["rows"](prefill_tokens), stack["rows"](prefill_tokens)
    positions = torch.arange(L, device=device)
    prefill_slots = torch.cat([block_table[b, positions // PAGE].long() * PAGE + positions % PAGE
                               for b in range(min(2, B))])

    def quantize_prefill():
        _cuda.quantize(list(zip(pk, pv)), caches[0], prefill_slots, key_rot, None, None, records, "anchor", 3, "ls")
    ms_prefill = graph_timed(quantize_prefill, 5) / 5
    del pk, pv
    _cuda.attention_status(device)

    bf16 = None
    if args.compare_bf16 and rank == 0:
        # One layer's four loop attentions over BF16 K/V of the same shape (contiguous [B, H, L, D], no paging, library
        # kernel): the comparator the packed path has to beat.  4 loops x (K + V) = 8 tensors of B*H*L*D bf16.
        import torch.nn.functional as F
        kv = [torch.randn(B, HEADS, L, HEAD_DIM, device=device, dtype=torch.bfloat16) for _ in range(8)]
        qb = torch.randn(4, B, HEADS, 1, HEAD_DIM, device=device, dtype=torch.bfloat16)
        ob = torch.empty_like(qb)

        def bf16_layer():
            for loop in range(4):
                ob[loop] = F.scaled_dot_product_attention(qb[loop], kv[2 * loop], kv[2 * loop + 1])
        ms_bf16 = graph_timed(bf16_layer, 5) / 5
        bytes_bf16 = 8 * B * HEADS * L * HEAD_DIM * 2
        packed_layer_ms = 3 * ms_res + ms_anchor + ms_quant
        bf16 = {"kernel": "torch.nn.functional.scaled_dot_product_attention, contiguous BF16 KV, 4 loops of one layer",
                "ms_per_layer": ms_bf16, "gbs": bytes_bf16 / (ms_bf16 * 1e-3) / 1e9,
                "packed_ms_per_layer": packed_layer_ms, "speedup": ms_bf16 / packed_layer_ms,
                "bf16_kv_bytes_per_layer": bytes_bf16}
        del kv

    sweep = None
    if args.sweep and rank == 0:
        sweep = []
        for batch in (1, 8, 32, 64):
            if batch > B:
                continue
            for context in (2048, 4096, 8192):
                if context > L:
                    continue
                lens = torch.full((batch,), context, dtype=torch.int32, device=device)
                starts = torch.arange(batch + 1, dtype=torch.int32, device=device)
                for loop in (0, 3):
                    def run():
                        for layer in range(layers):
                            _cuda.attention(q[layer, loop, :batch], k_live[layer, loop, :batch], v_live[layer, loop, :batch],
                                            caches[layer], out[layer, loop, :batch], starts, lens, block_table[:batch],
                                            key_rot, None, None, records, "anchor", 3, loop)
                    t = graph_timed(run, reps) / (reps * layers)
                    nbytes = attention_bytes(batch, context, args.group, loop == 3)
                    sweep.append({"batch": batch, "context": context, "loop": loop, "us": 1000 * t,
                                  "gbs": nbytes / (t * 1e-3) / 1e9, "frac": nbytes / (t * 1e-3) / 1e9 / peak})

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    line = {
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms / args.steps,
        "higher_is_better": True,
        "scaling": "strong" if shard_heads else "weak",
        "vs_baseline": None,
        "dtype": "f16 dot products and value sums with fp32 softmax/accumulation (attention); f32 (quantizer)",
        "data": "synthetic",
        "config": workload_config(args),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {
            "bound": "hbm", "kernel": "attention_kernel (residual loop: INT4 anchor + INT2 residual)",
            "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
            # DRAM bytes per launch = algorithmic bytes x 1.128, the ratio ncu measured on a smaller launch of the same
            # kernel (profiles/attention_kernel_b32_ctx8192.md); traffic grows in proportion to the tokens read
            "traffic": 1.128 * bytes_res, "algorithmic_bytes_per_launch": bytes_res, "us_per_launch": 1000 * ms_res,
            "anchor_loop": {"us_per_launch": 1000 * ms_anchor, "achieved": bytes_anchor / (ms_anchor * 1e-3) / 1e9,
                            "frac": bytes_anchor / (ms_anchor * 1e-3) / 1e9 / peak},
            "quantize_decode_write": {"us_per_launch": 1000 * ms_quant,
                                      "achieved": quantize_bytes(B, args.group) / (ms_quant * 1e-3) / 1e9},
            "quantize_prefill_write": {"tokens": prefill_tokens, "us_per_launch": 1000 * ms_prefill,
                                       "achieved": quantize_bytes(prefill_tokens, args.group) / (ms_prefill * 1e-3) / 1e9,
                                       "frac": quantize_bytes(prefill_tokens, args.group) / (ms_prefill * 1e-3) / 1e9 / peak},
        },
    }
    if sweep is not None:
        line["sweep"] = sweep
    if bf16 is not None:
        line["bf16_kv_comparator"] = bf16
    if not args.no_cpu_baseline:
        cpu_value, description, _ = cpu_sample(L, args.group, layers, B, sample_context=min(L, 4096))  # 5-20 s of CPU work
        line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": 1, "kind": "port", "sample": description}
    emit(line)
    if world > 1:
        dist.destroy_process_group()


_result_stream = None


def emit(line: dict) -> None:
    """The one JSON line of the run, on the process's real standard output."""
    text = json.dumps(line) + "\n"
    if _result_stream is not None:
        os.write(_result_stream, text.encode())
    else:
        sys.stdout.write(text)
        sys.stdout.flush()


def main():
    global HEADS, HEAD_DIM, PAGE, _result_stream
    args = parse_args()
    HEADS, HEAD_DIM, PAGE = args.heads, args.head_dim, args.page
    # Libraries print to file descriptor 1 on their own (NCCL announces its version there): keep the real standard
    # output for the result line and send everything else to standard error.
    sys.stdout.flush()
    _result_stream = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
