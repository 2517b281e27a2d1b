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
  sweep     attention alone over batch {1, 8, 32, 64} x context {2048, 4096, 8192}, residual and anchor loop
  ragged    a 64-row batch of one 8192-token row and 63 short rows against the time its pages imply at the uniform rate
  other_shapes  the same kernels with INT2 g16 residuals, and at 55 heads x 96 (batch 16 x 4096)
  bf16_kv_comparator  a BF16-KV decode attention (library kernel, contiguous KV) of one layer's four loops
  reference_cuda  the reference's own CUDA kernels on the same GPU, cache and inputs, when oracle/_ref holds its build
  head_sharded  the 55 x 96 shape with the KV heads spread over the ranks and the output gather fused into the
            attention kernel (strong scaling; the one-GPU run gives the curve's first point)
  config2_model_decode  a random-init Ouro-1.4B-shaped looped decoder: decode tokens/s with packed KV against BF16 KV
  cpu_baseline  the reference's PyTorch statement of the path (FP32Chain.reconstruct + probabilities + p @ V) timed on
            this machine's host cores; the numpy restatement when those files are absent

`--impl reference` times that CPU path alone, with every host thread, on the same workload description.
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import statistics
import subprocess
import sys
import time
from dataclasses import dataclass, replace

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
DENSE_ROTATION = False   # --dense-rotation: the stacks hand the operators a dense fp16 matrix
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


@dataclass(frozen=True)
class Shape:
    """One workload: a stack of `layers` KV groups of 4 loops ([2, group] x 3 + [4, 32], anchor last)."""
    batch: int
    context: int
    layers: int
    heads: int = 16
    head_dim: int = 128
    page: int = 16
    group: int = 32

    @property
    def records(self):
        return [[2, self.group]] * 3 + [[4, 32]]

    @property
    def width(self):
        return 3 * record_bytes(2, self.group, self.head_dim) + record_bytes(4, 32, self.head_dim)


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
    p.add_argument("--gather", default="fused", choices=["fused", "complete", "nccl"],
                   help="with --shard heads: fused = the attention kernel stores into every GPU's gathered output over "
                        "NVLink, followed by a barrier kernel per call (captured in the graph); complete = the same stores, "
                        "the kernel itself ends only when every rank's rows have arrived (no barrier launch); nccl = one "
                        "all-gather per call, eager")
    p.add_argument("--splits", type=int, default=0,
                   help="force the number of KV partitions per row (0 = the kernel picks them per row from the lengths)")
    p.add_argument("--dense-rotation", action="store_true",
                   help="give the operators the key rotation as a dense fp16 matrix (the path of a learned rotation) "
                        "instead of the registered signed-Hadamard structure")
    p.add_argument("--quick", action="store_true",
                   help="only the headline numbers: no sweep, other shapes, comparators or CPU baseline")
    p.add_argument("--no-cpu-baseline", action="store_true")
    return p.parse_args()


def record_bytes(bits, group, dim):
    return dim * bits // 8 + 2 * dim // group + 2


def attention_bytes(history_tokens, rows, shape, loop_is_anchor):
    """Algorithmic bytes of one attention launch: every cached token's anchor record without its alpha column,
    plus the loop's own residual record, for K and V; plus q, live k, live v, out in bf16.  `history_tokens` is the sum
    over the rows of their cached tokens."""
    anchor = record_bytes(4, 32, shape.head_dim) - 2
    per_token = anchor if loop_is_anchor else anchor + record_bytes(2, shape.group, shape.head_dim)
    return history_tokens * shape.heads * 2 * per_token + rows * shape.heads * shape.head_dim * 8


def quantize_bytes(tokens, shape):
    return 2 * 4 * tokens * shape.heads * shape.head_dim * 2 + 2 * tokens * shape.heads * shape.width


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own PyTorch statement of the path, timed on this machine's host cores
# ----------------------------------------------------------------------------------------------------------


def reference_python_available():
    return all(os.path.isfile(os.path.join(REF_DIR, "py", "calibration", name))
               for name in ("quantization.py", "rotation_math.py", "rotation_training.py"))


class ReferenceCpuPath:
    """One layer of ONE sequence at the workload's full context, through the reference's own functions
    (scripts/calibration/rotation_training.py:46-62 FP32Chain.reconstruct, rotation_math.py:44-49 probabilities):

      set-up (timed apart): quantize + reconstruct the `context - 1` cached tokens of the four loops, K and V;
      one step:  the four decode attentions (probabilities over the reconstructed keys + the live key, p @ V) and the
                 quantize + reconstruct of the step's new token, K and V.

    The workload's step is `layers x batch` such independent units; nothing is extrapolated along the context."""

    def __init__(self, shape: Shape, threads: int, seed: int = 0):
        import torch

        sys.path.insert(0, os.path.join(REF_DIR, "py"))
        from calibration.rotation_math import hadamard, probabilities
        from calibration.rotation_training import FP32Chain

        torch.set_num_threads(threads)
        torch.set_grad_enabled(False)
        self.torch, self.shape, self.probabilities = torch, shape, probabilities
        H, D, T = shape.heads, shape.head_dim, shape.context
        g = torch.Generator().manual_seed(seed)

        def loops():
            scale = torch.exp(0.5 * torch.randn(H, D, generator=g))
            anchor = torch.randn(T, H, D, generator=g) * scale
            for h in range(H):
                anchor[:, h, torch.randperm(D, generator=g)[:4]] *= 8
            return [(anchor * 0.9 + 0.3 * torch.randn(T, H, D, generator=g)).bfloat16() for _ in range(3)] + [anchor.bfloat16()]

        self.keys, self.values = loops(), loops()
        sign = (torch.randint(0, 2, (H, D), generator=g) * 2 - 1).float()
        self.rotation = (sign[:, :, None] * hadamard("cpu", D)[None]).half().float().contiguous()
        self.chain = FP32Chain([2, 2, 2, 4], "anchor", [shape.group] * 3 + [32], anchor_index=3)
        self.query = torch.randn(1, H, D, generator=g).bfloat16()
        t0 = time.perf_counter()
        history = [{"k": k[: T - 1], "v": v[: T - 1]} for k, v in zip(self.keys, self.values)]
        self.k_hat = self.chain.reconstruct(history, "k", [self.rotation], None)
        self.v_hat = self.chain.reconstruct(history, "v", [self.rotation], None)
        self.setup_seconds = time.perf_counter() - t0
        # the decode contract: cached tokens reconstructed, the last token live (raw bf16)
        self.k_all = [torch.cat([self.k_hat[i], self.keys[i][T - 1:].float()]) for i in range(4)]
        self.v_all = [torch.cat([self.v_hat[i], self.values[i][T - 1:].float()]) for i in range(4)]
        self.last = torch.tensor([T - 1])

    def step(self):
        torch, T = self.torch, self.shape.context
        t0 = time.perf_counter()
        for loop in range(4):
            p = self.probabilities(self.query, self.k_all[loop], self.last, head_dim=self.shape.head_dim)
            torch.bmm(p, self.v_all[loop].transpose(0, 1))
        t1 = time.perf_counter()
        live = [{"k": k[T - 1:], "v": v[T - 1:]} for k, v in zip(self.keys, self.values)]
        self.chain.reconstruct(live, "k", [self.rotation], None)
        self.chain.reconstruct(live, "v", [self.rotation], None)
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1


def cpu_reference(shape: Shape, steps: int, warmup: int):
    """(tokens/s of the workload on the host cores, cpu_baseline dict, seconds of one whole-workload step)."""
    threads = max(1, os.cpu_count() or 1)
    path = ReferenceCpuPath(shape, threads)
    attention, write = [], []
    for i in range(warmup + steps):
        a, w = path.step()
        if i >= warmup:
            attention.append(a)
            write.append(w)
    unit = statistics.median(attention) + statistics.median(write)   # one sequence, one layer
    step_seconds = unit * shape.layers * shape.batch
    value = shape.batch / step_seconds
    sample = (f"the reference's PyTorch path (FP32Chain.reconstruct + probabilities + p@V, torch {path.torch.__version__}, "
              f"{threads} threads) on 1 sequence x 1 layer at the full context {shape.context}: 4 decode attentions "
              f"{1e3 * statistics.median(attention):.1f} ms + write of the new token {1e3 * statistics.median(write):.1f} ms, "
              f"median of {steps}; the step is {shape.layers} layers x {shape.batch} sequences of this unit "
              f"(set-up, not in the step: quantize+reconstruct of the {shape.context - 1} cached tokens "
              f"{path.setup_seconds:.2f} s = {(shape.context - 1) / path.setup_seconds:.0f} tokens/s)")
    baseline = {"value": value, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample,
                "prefill_write_tokens_per_s": (shape.context - 1) / path.setup_seconds}
    return value, baseline, step_seconds


def cpu_port(shape: Shape, sample_context=1024, seed=0):
    """Fallback when the reference's PyTorch files were not placed under oracle/_ref/py: the numpy restatement, one
    sequence, one layer, at a reduced context (it is a scalar port), scaled linearly along the context."""
    from tests import helpers

    case = helpers.make_case(seed, shape.head_dim, shape.heads, [sample_context], shape.group, shape.page)
    t0 = time.perf_counter()
    cache = helpers.oracle_cache(case)
    t1 = time.perf_counter()
    for loop in range(4):
        helpers.oracle_attention(case, cache, loop)
    t2 = time.perf_counter()
    write = (t1 - t0) / max(1, sample_context - 1)
    attention = (t2 - t1) / max(1, sample_context - 1) * (shape.context - 1)
    step_seconds = (attention + write) * shape.layers * shape.batch
    value = shape.batch / step_seconds
    sample = (f"numpy restatement (oracle/rq_oracle.py), 1 sequence x 1 layer x context {sample_context} (quantize "
              f"{t1 - t0:.2f} s, 4 attentions {t2 - t1:.2f} s), scaled linearly to context {shape.context}; the reference's "
              "PyTorch files were not found under oracle/_ref/py")
    return value, {"value": value, "unit": UNIT, "cores": 1, "kind": "port", "sample": sample}, step_seconds


def cpu_baseline(shape: Shape, steps=3, warmup=1):
    """The reference's own PyTorch statement when its files are there (and run); else the numpy port."""
    if reference_python_available():
        try:
            return cpu_reference(shape, steps, warmup)
        except Exception as error:   # noqa: BLE001 -- e.g. the files do not import under this torch: time the port instead
            print(f"reference PyTorch path failed ({type(error).__name__}: {error}); timing the numpy port", file=sys.stderr)
    return cpu_port(shape)


def run_reference(args, shape):
    """`--impl reference`: the CPU path alone.  Rank 0 only; the other ranks have nothing to do."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    value, baseline, step_seconds = cpu_baseline(shape, max(1, args.steps), max(1, args.warmup))
    emit({
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1000.0 * step_seconds,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args, shape),
        "cpu_baseline": baseline,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def workload_config(args, shape):
    return {
        "workload": f"config1 kernel sweep point: batch {shape.batch} x context {shape.context}, INT2 g{shape.group} "
                    f"residuals + INT4 g32 anchor, {shape.layers} layers x 4 loops, {shape.heads} heads x {shape.head_dim}, "
                    f"block {shape.page}, CUDA-graph decode step (4 attention + 1 quantize launch per layer)"
                    + ("; key rotation given as a dense fp16 matrix" if args.dense_rotation else "")
                    + ("" if args.shard != "heads" else
                       "; KV heads sharded over the ranks, output rows stored into every GPU's gathered buffer by the attention "
                       "kernel, captured in the graph" if args.gather != "nccl" else
                       "; KV heads sharded over the ranks, one NCCL all-gather of the output per attention call, eager step"),
        "batch_per_gpu": shape.batch,
        "sharding": args.shard,
        "context": shape.context,
        "layers": shape.layers,
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


class Stack:
    """Packed caches of `layers` layers for `batch` sequences of `context` tokens (+ head room), filled by the
    quantizer kernel from seeded synthetic rows; every layer shares one block table, as under vLLM."""

    def __init__(self, shape: Shape, device, torch, heads_here=None, seed_offset=0):
        from residualquant_b200 import _cuda, rotation, synth

        self.shape, self.device, self.torch = shape, device, torch
        heads = shape.heads if heads_here is None else heads_here   # a head-sharded rank holds only its slice
        self.heads = heads
        D, P = shape.head_dim, shape.page
        self.records = shape.records
        head_room = 128
        blocks_per_seq = (shape.context + head_room + P - 1) // P
        num_blocks = shape.batch * blocks_per_seq + 1
        rng = np.random.default_rng(1234 + seed_offset)
        pool = rng.permutation(num_blocks - 1) + 1          # block 0 stays unused, like vLLM's null block
        self.block_table = torch.from_numpy(pool.reshape(shape.batch, blocks_per_seq).astype(np.int32)).to(device)
        self.key_rot = rotation.signed_hadamard(synth.signs(rng, heads, D), float(synth.fp16_rsqrt(D)), device)
        # what the operators are given: the registered structure (fused Walsh-Hadamard transform), or with --dense-rotation
        # the same rotation as a plain fp16 [heads, D, D] matrix, which takes the learned-rotation path of both kernels
        self.rotation = self.key_rot.dense() if DENSE_ROTATION else self.key_rot

        gen = torch.Generator(device=device)
        gen.manual_seed(99 + seed_offset)
        channel_scale = torch.exp(0.5 * torch.randn(heads, D, device=device, generator=gen))
        outlier = torch.ones(heads, D, device=device)
        for h in range(heads):
            outlier[h, torch.randperm(D, device=device, generator=gen)[:4]] = 8.0
        channel_scale = channel_scale * outlier

        def rows(tokens):
            anchor = torch.randn(tokens, heads, D, device=device, generator=gen) * channel_scale
            loops = [(0.9 * anchor + 0.3 * torch.randn(tokens, heads, D, device=device, generator=gen)).bfloat16()
                     for _ in range(3)]
            return loops + [anchor.bfloat16()]

        self.rows = rows
        self.caches = [torch.zeros((2, num_blocks, heads, P, shape.width), dtype=torch.uint8, device=device)]
        # fill layer 0 sequence by sequence, then clone it into the other layers
        positions = torch.arange(shape.context, device=device)
        for b in range(shape.batch):
            slots = self.block_table[b, positions // P].long() * P + positions % P
            k, v = rows(shape.context), rows(shape.context)
            # The model's weights absorb the value rotation in the served configuration (weights.py:9-37 of the
            # reference), so the kernels see value_rotation=None and V arrives rotated.
            _cuda.quantize(list(zip(k, v)), self.caches[0], slots, self.rotation, None, None, self.records, "anchor", 3, "ls")
        torch.cuda.synchronize(device)
        for _ in range(1, shape.layers):
            self.caches.append(self.caches[0].clone())
        L, B = shape.layers, shape.batch
        # per (layer, loop) inputs of a step, device resident
        self.q = torch.randn(L, 4, B, heads, D, device=device, generator=gen).bfloat16()
        live = rows(B * L)
        self.k_live = torch.stack([r.view(L, B, heads, D) for r in live], dim=1).contiguous()   # [layers, 4, B, H, D]
        live = rows(B * L)
        self.v_live = torch.stack([r.view(L, B, heads, D) for r in live], dim=1).contiguous()
        self.out = torch.zeros_like(self.q)
        self.qsl = torch.arange(B + 1, dtype=torch.int32, device=device)
        self.seq_lens = torch.full((B,), shape.context, dtype=torch.int32, device=device)
        self.slot_mapping = torch.zeros(B, dtype=torch.int64, device=device)
        self.batch_index = torch.arange(B, device=device)

    def advance(self):
        # position of the live token = seq_len - 1; its slot is where this step's quantize writes
        P = self.shape.page
        position = (self.seq_lens - 1).long()
        self.slot_mapping.copy_(self.block_table[self.batch_index, position // P].long() * P + position % P)

    def attention(self, layer, loop, rows=None, seq_lens=None, qsl=None, **extra):
        from residualquant_b200 import _cuda

        rows = self.shape.batch if rows is None else rows
        _cuda.attention(self.q[layer, loop, :rows], self.k_live[layer, loop, :rows], self.v_live[layer, loop, :rows],
                        self.caches[layer], self.out[layer, loop, :rows], self.qsl if qsl is None else qsl,
                        self.seq_lens if seq_lens is None else seq_lens, self.block_table[:rows], self.rotation, None, None,
                        self.records, "anchor", 3, loop, **extra)

    def quantize(self, layer):
        from residualquant_b200 import _cuda

        _cuda.quantize([(self.k_live[layer, i], self.v_live[layer, i]) for i in range(4)], self.caches[layer],
                       self.slot_mapping, self.rotation, None, None, self.records, "anchor", 3, "ls")


class Timer:
    """CUDA-event timing on a side stream, barrier + synchronize on both sides, maximum over the ranks."""

    def __init__(self, torch, dist, device, world):
        self.torch, self.dist, self.device, self.world = torch, dist, device, world
        self.stream = torch.cuda.Stream(device)

    def join_default_stream(self):
        """Everything queued on the default stream (input tensors, lengths, tables) is complete before the side stream
        reads it: a kernel that saw half-initialised lengths or block ids would read outside the cache."""
        self.stream.wait_stream(self.torch.cuda.current_stream(self.device))

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.device)

    def timed(self, fn, steps, collective=True):
        from residualquant_b200 import sharding

        torch = self.torch
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if collective:
            self.barrier()
        else:
            torch.cuda.synchronize(self.device)
        self.join_default_stream()
        with torch.cuda.stream(self.stream):
            start.record(self.stream)
            for _ in range(steps):
                fn()
            stop.record(self.stream)
        stop.synchronize()
        if not collective:
            return start.elapsed_time(stop)
        self.barrier()
        return sharding.max_over_ranks(start.elapsed_time(stop), self.device)

    def capture(self, fn):
        """Eager warm-up, then one CUDA graph of `fn`."""
        torch = self.torch
        self.join_default_stream()
        with torch.cuda.stream(self.stream):
            fn()
        self.stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.stream):
            fn()
        return graph

    def graph_ms(self, fn, replays, collective=False):
        """Capture `fn` and time `replays` replays: per-kernel device time without the Python launch overhead."""
        graph = self.capture(fn)
        self.timed(graph.replay, 1, collective)
        return self.timed(graph.replay, replays, collective) / replays


def kernel_figures(timer, stack, peak, reps):
    """Residual-loop and anchor-loop attention, decode write and prefill-sized write of one stack, each alone."""
    torch, shape = stack.torch, stack.shape
    L, B = shape.layers, shape.batch
    stack.seq_lens.fill_(shape.context)
    sized = replace(shape, heads=stack.heads)
    out = {}
    for name, loop in (("attention_residual_loop", 0), ("attention_anchor_loop", 3)):
        ms = timer.graph_ms(lambda: [stack.attention(layer, loop) for layer in range(L)], reps) / L
        nbytes = attention_bytes(B * (shape.context - 1), B, sized, loop == 3)
        out[name] = {"us_per_launch": 1000 * ms, "algorithmic_bytes_per_launch": nbytes,
                     "achieved": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
    stack.advance()
    ms = timer.graph_ms(lambda: [stack.quantize(layer) for layer in range(L)], reps) / L
    out["quantize_decode_write"] = {"tokens": B, "us_per_launch": 1000 * ms,
                                    "achieved": quantize_bytes(B, sized) / (ms * 1e-3) / 1e9}
    # prefill-sized write: two full prompts (2 x context tokens) of layer 0 re-quantized in one call
    from residualquant_b200 import _cuda

    prompts = min(2, B)
    tokens = prompts * shape.context
    pk, pv = stack.rows(tokens), stack.rows(tokens)
    positions = torch.arange(shape.context, device=stack.device)
    slots = torch.cat([stack.block_table[b, positions // shape.page].long() * shape.page + positions % shape.page
                       for b in range(prompts)])
    ms = timer.graph_ms(lambda: _cuda.quantize(list(zip(pk, pv)), stack.caches[0], slots, stack.rotation, None, None,
                                               stack.records, "anchor", 3, "ls"), 5)
    nbytes = quantize_bytes(tokens, sized)
    out["quantize_prefill_write"] = {"tokens": tokens, "us_per_launch": 1000 * ms, "achieved": nbytes / (ms * 1e-3) / 1e9,
                                     "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
    return out


def sweep_figures(timer, stack, peak, reps):
    """Attention alone over the batch x context grid of the kernel-sweep configuration (one launch per layer, so every
    launch reads a cache that the previous launches pushed out of L2)."""
    torch, shape = stack.torch, stack.shape
    rows_out = []
    for batch in (1, 8, 32, 64):
        if batch > shape.batch:
            continue
        for context in (2048, 4096, 8192):
            if context > shape.context:
                continue
            lens = torch.full((batch,), context, dtype=torch.int32, device=stack.device)
            starts = torch.arange(batch + 1, dtype=torch.int32, device=stack.device)
            for loop in (0, 3):
                ms = timer.graph_ms(lambda: [stack.attention(layer, loop, batch, lens, starts)
                                             for layer in range(shape.layers)], reps) / shape.layers
                nbytes = attention_bytes(batch * (context - 1), batch, shape, loop == 3)
                rows_out.append({"batch": batch, "context": context, "loop": loop, "us": round(1000 * ms, 2),
                                 "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1),
                                 "frac": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4)})
    return rows_out


def decode_step_figures(timer, stack, reps):
    """The latency protocol of the reference's own measurements (batch 1 at 2k / 4k / 8k): one whole decode step of the
    stack (4 attention + 1 write launch per layer) under CUDA-graph replay."""
    torch, shape = stack.torch, stack.shape
    out = []
    for context in (2048, 4096, 8192):
        if context > shape.context:
            continue
        lens = torch.full((1,), context, dtype=torch.int32, device=stack.device)
        starts = torch.arange(2, dtype=torch.int32, device=stack.device)
        slot = (stack.block_table[:1, (context - 1) // shape.page].long() * shape.page + (context - 1) % shape.page)
        from residualquant_b200 import _cuda

        def step():
            for layer in range(shape.layers):
                for loop in range(4):
                    stack.attention(layer, loop, 1, lens, starts)
                _cuda.quantize([(stack.k_live[layer, i, :1], stack.v_live[layer, i, :1]) for i in range(4)],
                               stack.caches[layer], slot, stack.rotation, None, None, stack.records, "anchor", 3, "ls")
        ms = timer.graph_ms(step, reps)
        out.append({"batch": 1, "context": context, "ms_per_step": round(ms, 4), "tokens_per_s": round(1000.0 / ms, 1),
                    "launches": 5 * shape.layers})
    return out


def ragged_figures(timer, stack, peak, reps, uniform_us):
    """One 8192-token row among 63 rows of 17..600 tokens: what length-aware partitioning is for.  `implied_us` is the time
    the batch's cached tokens would take at the rate of the uniform batch (same rows, every row at the full context)."""
    torch, shape = stack.torch, stack.shape
    if shape.batch < 64:
        return None
    rng = np.random.default_rng(7)
    lengths = np.concatenate([[shape.context], rng.integers(17, 601, size=63)]).astype(np.int32)
    lens = torch.from_numpy(lengths).to(stack.device)
    starts = torch.arange(65, dtype=torch.int32, device=stack.device)
    history = int((lengths - 1).sum())
    out = {"rows": 64, "lengths": f"{shape.context} + 63 rows of 17..600 (seed 7), {history} cached tokens in all"}
    from residualquant_b200 import _cuda, _lib

    uniform = _lib.load().rq_attention_default_splits(64, shape.heads, stack.block_table.shape[1], shape.page)
    out["uniform_rule_partitions"] = int(uniform)
    for name, loop in (("residual_loop", 0), ("anchor_loop", 3)):
        def layers():
            for layer in range(shape.layers):
                stack.attention(layer, loop, 64, lens, starts)
        ms = timer.graph_ms(layers, reps) / shape.layers
        # the same call with one partition count for every row, chosen from the widest row (the rule a host-side schedule
        # has to use when the grid must not depend on the lengths)
        _cuda.set_attention_splits(uniform)
        try:
            uniform_ms = timer.graph_ms(layers, reps) / shape.layers
        finally:
            _cuda.set_attention_splits(0)
        implied = uniform_us[name] * history / (64 * (shape.context - 1))
        out[name] = {"us": round(1000 * ms, 2), "uniform_rule_us": round(1000 * uniform_ms, 2),
                     "implied_us": round(implied, 2), "ratio": round(1000 * ms / implied, 3),
                     "frac": round(attention_bytes(history, 64, shape, loop == 3) / (ms * 1e-3) / 1e9 / peak, 4)}
    return out


def bf16_comparator(timer, stack, packed_ms_per_layer):
    """One layer's four loop attentions over BF16 K/V of the same shape (contiguous [B, H, L, D], no paging, library
    kernel): the comparator the packed path has to beat.  4 loops x (K + V) = 8 tensors of B*H*L*D bf16."""
    torch, shape = stack.torch, stack.shape
    import torch.nn.functional as F

    B, H, L, D = shape.batch, shape.heads, shape.context, shape.head_dim
    kv = [torch.randn(B, H, L, D, device=stack.device, dtype=torch.bfloat16) for _ in range(8)]
    qb = torch.randn(4, B, H, 1, D, device=stack.device, dtype=torch.bfloat16)
    ob = torch.empty_like(qb)

    def bf16_layer():
        for loop in range(4):
            ob[loop] = F.scaled_dot_product_attention(qb[loop], kv[2 * loop], kv[2 * loop + 1])
    ms = timer.graph_ms(bf16_layer, 5)
    nbytes = 8 * B * H * L * D * 2
    del kv
    return {"kernel": "torch.nn.functional.scaled_dot_product_attention, contiguous BF16 KV, 4 loops of one layer",
            "ms_per_layer": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "packed_ms_per_layer": packed_ms_per_layer,
            "speedup": ms / packed_ms_per_layer, "bf16_kv_bytes_per_layer": nbytes,
            "bf16_kv_bytes_whole_stack": nbytes * shape.layers}


def reference_cuda_figures(timer, stack):
    """The reference's own CUDA kernels (built from its sources by oracle/build_ref.py into oracle/_ref) beside this
    library's, on one layer of the stack: same GPU, same packed cache, same inputs, CUDA-graph replay.  The reference takes
    its rotation as a dense fp16 matrix (TF32 tensor-core product per call); this library is timed both ways: with the
    same dense matrix ("dense") and with the fused Walsh-Hadamard transform the matrix's structure allows ("fwht")."""
    if not glob.glob(os.path.join(REF_DIR, "_cuda*.so")):
        return {"unavailable": "oracle/_ref holds no build of the reference's extension"}
    torch, shape = stack.torch, stack.shape
    from residualquant_b200 import _cuda

    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        import _cuda as reference   # the reference's module name
    except Exception as error:      # built against another torch, missing symbols, ...
        return {"unavailable": f"import failed: {error}"[:200]}
    B, P = shape.batch, shape.page
    dense = stack.key_rot.dense()
    q, k, v = stack.q[0, 0], stack.k_live[0, 0], stack.v_live[0, 0]
    cache = stack.caches[0]
    stack.seq_lens.fill_(shape.context)
    stack.advance()
    torch.cuda.synchronize(stack.device)
    live_pairs = [(stack.k_live[0, i], stack.v_live[0, i]) for i in range(4)]
    prompts = min(2, B)
    tokens = prompts * (shape.context - 1)
    positions = torch.arange(shape.context - 1, device=stack.device)
    prompt_slots = torch.cat([stack.block_table[b, positions // P].long() * P + positions % P for b in range(prompts)])
    pk, pv = stack.rows(tokens), stack.rows(tokens)
    prompt_pairs = list(zip(pk, pv))
    scratch = cache.clone()
    out_ref, out_ours = torch.zeros_like(q), torch.zeros_like(q)
    figures = {"shape": f"batch {B} x context {shape.context}, one layer, {shape.heads} heads x {shape.head_dim}, g{shape.group}",
               "note": "us per call under CUDA-graph replay; the caches of consecutive replays are the same, larger than L2 "
                       "for batch >= 8"}

    def attention_of(module, rotation, out, loop, rows=B, lens=None):
        lens = stack.seq_lens[:rows] if lens is None else lens
        return lambda: module.attention(q[:rows], k[:rows], v[:rows], cache, out[:rows], stack.qsl[:rows + 1], lens,
                                        stack.block_table[:rows], rotation, None, None, stack.records, "anchor", 3, loop)

    def three_ways(loop, rows=B, lens=None, reps=5):
        return {"reference": round(1000 * timer.graph_ms(attention_of(reference, dense, out_ref, loop, rows, lens), reps), 2),
                "this_dense": round(1000 * timer.graph_ms(attention_of(_cuda, dense, out_ours, loop, rows, lens), reps), 2),
                "this_fwht": round(1000 * timer.graph_ms(attention_of(_cuda, stack.key_rot, out_ours, loop, rows, lens), reps), 2)}

    def quantize_of(module, rotation, pairs, slots):
        return lambda: module.quantize(pairs, scratch, slots, rotation, None, None, stack.records, "anchor", 3, "ls")

    try:
        for name, loop in (("attention_residual_us", 0), ("attention_anchor_us", 3)):
            figures[name] = three_ways(loop)
            figures[name]["outputs_rms_difference"] = float((out_ref.float() - out_ours.float()).pow(2).mean().sqrt())
        # small batches (latency regime) and a ragged batch (one full-context row among short ones), residual loop
        for rows in (1, 8):
            if rows < B:
                figures[f"attention_residual_batch{rows}_us"] = three_ways(0, rows, reps=20)
        if B >= 64:
            rng = np.random.default_rng(7)
            lengths = np.concatenate([[shape.context], rng.integers(17, 601, size=63)]).astype(np.int32)
            ragged = torch.from_numpy(lengths).to(stack.device)
            figures["attention_residual_ragged_us"] = three_ways(0, 64, ragged, reps=20)
            figures["attention_residual_ragged_us"]["lengths"] = f"{shape.context} + 63 rows of 17..600 (seed 7)"
        for name, pairs, slots in (("quantize_decode_us", live_pairs, stack.slot_mapping),
                                   ("quantize_prefill_us", prompt_pairs, prompt_slots)):
            figures[name] = {
                "tokens": int(slots.numel()),
                "reference": round(1000 * timer.graph_ms(quantize_of(reference, dense, pairs, slots), 3), 2),
                "this_dense": round(1000 * timer.graph_ms(quantize_of(_cuda, dense, pairs, slots), 3), 2),
                "this_fwht": round(1000 * timer.graph_ms(quantize_of(_cuda, stack.key_rot, pairs, slots), 3), 2),
            }
    except RuntimeError as error:
        figures["unavailable"] = f"{error}"[:200]
    return figures


def head_sharded_figures(timer, torch, dist, device, rank, world, steps, warmup):
    """BASELINE's largest configuration's kernel shape (55 heads x 96, batch 16 at context 4096, 4 core layers x 8 groups
    = 32 caches, 128 attention calls per step) with the KV heads spread over the ranks: strong scaling.  Every rank
    stores its finished rows into every GPU's gathered output from inside the attention kernel; the whole step is one
    CUDA graph per rank."""
    from residualquant_b200 import sharding

    shape = Shape(batch=16, context=4096, layers=32, heads=55, head_dim=96, page=16, group=32)
    local = sharding.shard_counts(shape.heads, world)[rank]
    stack = Stack(shape, device, torch, heads_here=local, seed_offset=1000 + rank)
    def measure(gather):
        def step():
            # barrier form: one barrier kernel per call, launched as a programmatic dependent.  complete form: every
            # attention call ends only when all ranks' rows of that call are in this GPU's gathered buffer (its last CTA
            # publishes and waits), so nothing sits between the calls.  No gather at all: what the rank's own work costs.
            for layer in range(shape.layers):
                for loop in range(4):
                    if gather is None:
                        stack.attention(layer, loop)
                        continue
                    stack.attention(layer, loop, gather=gather, gather_buffer=loop % 2)
                    gather.barrier()
                stack.quantize(layer)
            stack.seq_lens.add_(1)
            stack.advance()

        stack.seq_lens.fill_(shape.context - 1)
        stack.advance()
        graph = timer.capture(step)    # one eager step, then the capture
        stack.seq_lens.fill_(shape.context)
        stack.advance()
        timer.join_default_stream()
        with torch.cuda.stream(timer.stream):
            for _ in range(warmup):
                graph.replay()
        ms = timer.timed(graph.replay, steps)
        if gather is None:
            del graph
            return ms, True
        gather.check()
        expected = sharding.gather_heads(stack.out[shape.layers - 1, 3], shape.heads)
        equal = bool(torch.equal(gather.gathered(3 % 2), expected))
        flags = torch.tensor([1 if equal else 0], device=device)
        if world > 1:
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        del graph
        return ms, bool(flags.item() == 1)

    gather = sharding.HeadGather(shape.batch, shape.heads, shape.head_dim, device)
    ms, equal = measure(gather)
    complete = sharding.HeadGather(shape.batch, shape.heads, shape.head_dim, device, complete=True)
    complete_ms, complete_equal = measure(complete)
    alone_ms, _ = measure(None)
    result = {"shape": "55 heads x 96, batch 16 x context 4096, 32 (layer, group) caches, 128 attention + 128 barrier + 32 "
                       "write launches per step, INT2 g32 + INT4 g32; output rows stored into every GPU's gathered buffer by the "
                       "attention kernel, one barrier kernel per call (programmatic dependent)",
              "n": world, "heads_per_rank": sharding.shard_counts(shape.heads, world),
              "tokens_per_s": shape.batch * steps / (ms * 1e-3), "ms_per_step": ms / steps,
              "gathered_equal_nccl": equal, "scaling": "strong",
              # the same step with the barrier folded into the attention kernel (its last CTA publishes and waits for
              # every rank), and with no gather at all (this rank's share of the work alone: the bound of the scaling)
              "complete_form": {"ms_per_step": complete_ms / steps, "gathered_equal_nccl": complete_equal,
                                "launches": "128 attention + 32 write"},
              "without_gather_ms_per_step": alone_ms / steps}
    del stack, gather, complete
    torch.cuda.empty_cache()
    return result


class LoopedDecoder:
    """Random-init Ouro-1.4B-shaped looped decoder for the model-level comparison (BASELINE configuration 2): 24 layers
    shared by 4 loops, hidden 2048, 16 heads x 128, SwiGLU FFN 5632, vocabulary 49152, bf16 weights N(0, 0.02).  The
    projections are library GEMMs (they are outside the two hot paths); rotary embedding is left out (an elementwise
    kernel that both arms would share).  Layer order and KV grouping follow the reference's adapter
    (plugins/looped_transformers/src/looped_transformers/ouro.py:141-158, 231-241): `for loop: for layer:`, one KV group
    of 4 loops per physical layer, written by the last loop."""

    def __init__(self, torch, device, batch, layers=24, hidden=2048, heads=16, head_dim=128, ffn=5632, vocab=49152):
        self.torch, self.device, self.batch = torch, device, batch
        self.layers, self.hidden, self.heads, self.head_dim, self.ffn = layers, hidden, heads, head_dim, ffn
        gen = torch.Generator(device=device)
        gen.manual_seed(2024)

        def weight(*shape):
            return (0.02 * torch.randn(*shape, device=device, generator=gen)).bfloat16()

        self.embed = weight(vocab, hidden)
        self.lm_head = weight(hidden, vocab)
        self.qkv = [weight(hidden, 3 * heads * head_dim) for _ in range(layers)]
        self.out = [weight(heads * head_dim, hidden) for _ in range(layers)]
        self.gate_up = [weight(hidden, 2 * ffn) for _ in range(layers)]
        self.down = [weight(ffn, hidden) for _ in range(layers)]
        self.norms = [[torch.ones(hidden, device=device, dtype=torch.bfloat16) for _ in range(3)] for _ in range(layers)]
        self.final_norm = torch.ones(hidden, device=device, dtype=torch.bfloat16)
        self.tokens = torch.randint(100, 10000, (batch,), device=device, generator=gen)

    def weight_bytes_per_step(self, loops=4):
        per_layer = sum(w[0].numel() for w in (self.qkv, self.out, self.gate_up, self.down)) * 2
        return loops * self.layers * per_layer + self.lm_head.numel() * 2

    def step(self, attention, end_of_layer, loops=4):
        """One decode step.  `attention(layer, loop, q, k, v) -> [B, H, D]`; `end_of_layer(layer)` after the last loop."""
        torch, F = self.torch, self.torch.nn.functional
        B, H, D = self.batch, self.heads, self.head_dim
        x = self.embed[self.tokens]
        for loop in range(loops):
            for layer in range(self.layers):
                n1, n2, n3 = self.norms[layer]
                qkv = (F.rms_norm(x, (self.hidden,), n1) @ self.qkv[layer]).view(B, 3, H, D)
                o = attention(layer, loop, qkv[:, 0], qkv[:, 1], qkv[:, 2])
                x = x + F.rms_norm(o.reshape(B, H * D) @ self.out[layer], (self.hidden,), n2)
                gate_up = F.rms_norm(x, (self.hidden,), n3) @ self.gate_up[layer]
                x = x + (F.silu(gate_up[:, : self.ffn]) * gate_up[:, self.ffn:]) @ self.down[layer]
                if loop == loops - 1:
                    end_of_layer(layer)
            x = F.rms_norm(x, (self.hidden,), self.final_norm)
        self.tokens.copy_((x @ self.lm_head).argmax(-1))


def model_decode_figures(timer, torch, device, batch=32, prompt=2048, generated=128, steps=24):
    """BASELINE configuration 2: decode tokens/s of the looped decoder with the packed KV path against the same decoder
    with BF16 KV, same GPU, same GEMMs, CUDA-graph replay, prefill and the first token excluded (the reference's
    protocol, experiments/kv_memory_latency/measure.py:347-360).  Both arms run at the mean context of the generated
    tokens (prompt + generated / 2): the BF16 arm is a library attention call whose KV length is baked into the captured
    graph, so neither arm's context grows during the timed steps (the packed arm's lengths are reset between replays)."""
    from residualquant_b200 import _cuda

    context = prompt + generated // 2
    shape = Shape(batch=batch, context=context, layers=24)
    stack = Stack(shape, device, torch, seed_offset=31)
    model = LoopedDecoder(torch, device, batch)
    F = torch.nn.functional
    B, H, D = batch, shape.heads, shape.head_dim
    _cuda.set_stable_metadata(True)
    pending = [[] for _ in range(shape.layers)]
    outputs = torch.zeros(shape.layers, 4, B, H, D, device=device, dtype=torch.bfloat16)

    def packed_attention(layer, loop, q, k, v):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out = outputs[layer, loop]
        _cuda.attention(q, k, v, stack.caches[layer], out, stack.qsl, stack.seq_lens, stack.block_table, stack.rotation, None,
                        None, stack.records, "anchor", 3, loop)
        pending[layer].append((k, v))
        return out

    def packed_end_of_layer(layer):
        _cuda.quantize(pending[layer], stack.caches[layer], stack.slot_mapping, stack.rotation, None, None, stack.records,
                       "anchor", 3, "ls")
        pending[layer].clear()

    def packed_step():
        model.step(packed_attention, packed_end_of_layer)
        # the next replay starts from the same context: lengths and slots are left as they are

    stack.seq_lens.fill_(context)
    stack.advance()
    packed_ms = timer.graph_ms(packed_step, steps)

    # BF16 KV: [layer][loop] K and V, contiguous [B, H, context, D]; the new token overwrites the last position
    kv = torch.empty(shape.layers, 4, 2, B, H, context, D, device=device, dtype=torch.bfloat16)
    for layer in range(shape.layers):
        kv[layer].normal_()

    def bf16_attention(layer, loop, q, k, v):
        cache_k, cache_v = kv[layer, loop, 0], kv[layer, loop, 1]
        cache_k[:, :, context - 1] = k
        cache_v[:, :, context - 1] = v
        return F.scaled_dot_product_attention(q.unsqueeze(2), cache_k, cache_v).squeeze(2)

    bf16_ms = timer.graph_ms(lambda: model.step(bf16_attention, lambda layer: None), steps)
    packed_kv = shape.layers * 2 * shape.heads * (context - 1) * B * (3 * (record_bytes(4, 32, D) - 2 + record_bytes(2, 32, D))
                                                                        + record_bytes(4, 32, D) - 2)
    figures = {
        "model": "random-init Ouro-1.4B shape: 24 layers x 4 loops, hidden 2048, 16 heads x 128, SwiGLU 5632, vocab 49152, bf16",
        "batch": B, "context": context, "note": f"decode at the mean context of {generated} generated tokens after a {prompt}-token "
                                                "prompt; cuBLAS projections and torch elementwise kernels in both arms, rotary embedding omitted",
        "packed_kv": {"ms_per_token": packed_ms, "tokens_per_s": B * 1000.0 / packed_ms, "kv_bytes_read_per_step": packed_kv},
        "bf16_kv": {"ms_per_token": bf16_ms, "tokens_per_s": B * 1000.0 / bf16_ms,
                    "kv_bytes_read_per_step": int(kv.numel() * 2), "attention": "torch scaled_dot_product_attention, contiguous KV"},
        "speedup": bf16_ms / packed_ms,
        "weight_bytes_per_step": model.weight_bytes_per_step(),
    }
    del kv, stack, model
    torch.cuda.empty_cache()
    return figures


def run_gpu(args, shape):
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

    shard_heads = args.shard == "heads"
    heads_here = None
    if shard_heads:
        heads_here = sharding.shard_counts(shape.heads, world)[rank]   # this rank's slice of every cache and of q/k/v
        if heads_here == 0:
            raise RuntimeError("more ranks than KV heads")
    replicas = 1 if shard_heads else world                          # independent copies of the batch in the job
    B, L, layers = shape.batch, shape.context, shape.layers
    _cuda.set_attention_splits(args.splits)
    timer = Timer(torch, dist, device, world)
    stack = Stack(shape, device, torch, heads_here, seed_offset=rank)
    peak, peak_kind = measured_peak()

    gathered = [None]
    # Head sharding: the output projection needs every head.  "fused": the attention kernel stores its rows into every
    # GPU's gathered buffer over NVLink (graph capturable); "nccl": one all-gather per call.
    fused_gather = (sharding.HeadGather(B, shape.heads, shape.head_dim, device, complete=args.gather == "complete")
                    if shard_heads and args.gather != "nccl" else None)

    def hot_path():
        for layer in range(layers):
            for loop in range(4):
                if fused_gather is not None:
                    stack.attention(layer, loop, gather=fused_gather, gather_buffer=loop % 2)
                    fused_gather.barrier()
                    continue
                stack.attention(layer, loop)
                if shard_heads:
                    gathered[0] = sharding.gather_heads(stack.out[layer, loop], shape.heads)
            stack.quantize(layer)

    # The engine's promise of RQ_FLAG_STABLE_METADATA: lengths, tables and slots are written once per step, never by the
    # kernel right in front of an attention call -- here at the END of the captured step, for the next replay.
    _cuda.set_stable_metadata(True)

    def step_body():
        hot_path()
        stack.seq_lens.add_(1)
        stack.advance()

    def rewind():
        stack.seq_lens.fill_(L)
        stack.advance()

    rewind()

    if shard_heads and world > 1 and fused_gather is None:
        # The step contains NCCL all-gathers; it is replayed eagerly rather than from a captured graph.
        timer.join_default_stream()
        with torch.cuda.stream(timer.stream):
            step_body()
        timer.stream.synchronize()

        class _Eager:
            @staticmethod
            def replay():
                step_body()
        graph = _Eager()
    else:
        graph = timer.capture(step_body)
    rewind()
    torch.cuda.synchronize(device)
    launches_per_step = layers * (9 if fused_gather is not None and not fused_gather.complete else 5)

    sampler = ClockSampler(local_rank)
    # ---------------- device-resident throughput ----------------
    timer.join_default_stream()
    with torch.cuda.stream(timer.stream):
        for _ in range(args.warmup):
            graph.replay()
    if rank == 0:
        sampler.start()
    ms = timer.timed(graph.replay, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    if fused_gather is not None:
        # the gathered rows of the last call must equal an NCCL all-gather of every rank's own output
        fused_gather.check()
        expected = sharding.gather_heads(stack.out[layers - 1, 3], shape.heads)
        if not torch.equal(fused_gather.gathered(3 % 2), expected):
            raise RuntimeError("fused head gather differs from the all-gathered outputs")
    value = replicas * B * args.steps / (ms * 1e-3)

    # ---------------- end to end: host rows in, outputs back ----------------
    rewind()
    q, k_live, v_live, out = stack.q, stack.k_live, stack.v_live, stack.out
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
        stack.seq_lens.copy_(host_lens, non_blocking=True)
        stack.advance()
        graph.replay()
        host_out.copy_(out, non_blocking=True)
        host_lens.add_(1)

    timer.join_default_stream()
    with torch.cuda.stream(timer.stream):
        for _ in range(args.warmup):
            e2e_step()
    timer.stream.synchronize()
    host_lens.fill_(L)
    ms_e2e = timer.timed(e2e_step, args.steps)
    e2e_value = replicas * B * args.steps / (ms_e2e * 1e-3)
    del host_q, host_k, host_v, host_out

    # ---------------- every kernel alone ----------------
    reps = max(3, 48 // layers)
    kernels = kernel_figures(timer, stack, peak, reps)
    residual, anchor = kernels["attention_residual_loop"], kernels["attention_anchor_loop"]
    _cuda.attention_status(device)

    extras = {}

    def side(name, measure):
        """A side measurement must never cost the result line: on an error its entry says what went wrong."""
        try:
            figures = measure()
        except Exception as error:   # noqa: BLE001 -- anything: the headline figures above are already measured
            figures = {"error": f"{type(error).__name__}: {error}"[:300]}
            try:
                torch.cuda.synchronize(device)
            except Exception as later:   # noqa: BLE001
                figures["error"] += f"; then {later}"[:200]
        if figures is not None:
            extras[name] = figures

    full = not args.quick and not shard_heads
    if full and rank == 0 and world == 1:
        # Only the single-GPU run carries the side measurements; a multi-GPU launch reports scaling.
        side("sweep", lambda: sweep_figures(timer, stack, peak, reps))
        side("decode_step_batch1", lambda: decode_step_figures(timer, stack, reps))
        side("ragged", lambda: ragged_figures(timer, stack, peak, reps, {"residual_loop": residual["us_per_launch"],
                                                                        "anchor_loop": anchor["us_per_launch"]}))
        packed_layer_ms = (3 * residual["us_per_launch"] + anchor["us_per_launch"]
                           + kernels["quantize_decode_write"]["us_per_launch"]) / 1000.0
        side("reference_cuda", lambda: reference_cuda_figures(timer, stack))
        if shape.batch * shape.heads * shape.context * shape.head_dim * 16 < 40e9:
            side("bf16_kv_comparator", lambda: bf16_comparator(timer, stack, packed_layer_ms))
    if full and world > 1:
        # every rank takes part; rank 0 reports.  (Not wrapped: a rank that skipped a collective would hang the others.)
        del stack
        stack = None
        torch.cuda.empty_cache()
        extras["head_sharded"] = head_sharded_figures(timer, torch, dist, device, rank, world, args.steps, args.warmup)
    if full and rank == 0 and world == 1:
        del stack
        stack = None
        torch.cuda.empty_cache()
        def other_shapes():
            other = {}
            for name, variant in (("g16", replace(shape, group=16, layers=min(4, layers))),
                                  ("huginn_55x96", Shape(batch=16, context=4096, layers=8, heads=55, head_dim=96, page=16, group=32))):
                s = Stack(variant, device, torch, seed_offset=17)
                figures = kernel_figures(timer, s, peak, 3)
                figures["shape"] = (f"batch {variant.batch} x context {variant.context}, {variant.heads} heads x "
                                    f"{variant.head_dim}, g{variant.group}, {variant.layers} layers")
                other[name] = figures
                del s
                torch.cuda.empty_cache()
            return other

        side("other_shapes", other_shapes)
        # the one-GPU point of the head-sharded strong-scaling curve (same step, every head on this GPU)
        side("head_sharded", lambda: head_sharded_figures(timer, torch, dist, device, rank, world, args.steps, args.warmup))
        side("config2_model_decode", lambda: model_decode_figures(timer, torch, device))

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    achieved = residual["achieved"]
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
        "config": workload_config(args, shape),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {
            "bound": "hbm", "kernel": "attention_kernel (residual loop: INT4 anchor + INT2 residual)",
            "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
            # DRAM bytes per launch = algorithmic bytes x 1.128, the ratio ncu measured on a smaller launch of the same
            # kernel (profiles/attention_kernel_b32_ctx8192.md); traffic grows in proportion to the tokens read
            "traffic": 1.128 * residual["algorithmic_bytes_per_launch"],
            "algorithmic_bytes_per_launch": residual["algorithmic_bytes_per_launch"],
            "us_per_launch": residual["us_per_launch"],
            "anchor_loop": {k: anchor[k] for k in ("us_per_launch", "achieved", "frac")},
            "quantize_decode_write": kernels["quantize_decode_write"],
            "quantize_prefill_write": kernels["quantize_prefill_write"],
        },
    }
    line.update(extras)
    if not args.no_cpu_baseline and not args.quick:
        try:
            _, line["cpu_baseline"], _ = cpu_baseline(shape)
        except Exception as error:   # noqa: BLE001 -- the line is printed whatever happens to the host-side leg
            line["cpu_baseline"] = {"error": f"{type(error).__name__}: {error}"[:300]}
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
    global _result_stream, DENSE_ROTATION
    args = parse_args()
    DENSE_ROTATION = args.dense_rotation
    shape = Shape(batch=args.batch, context=args.context, layers=args.layers, heads=args.heads, head_dim=args.head_dim,
                  page=args.page, group=args.group)
    # Libraries print to file descriptor 1 on their own (NCCL announces its version there): keep the real standard
    # output for the result line and send everything else to standard error.
    sys.stdout.flush()
    _result_stream = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args, shape)
    else:
        run_gpu(args, shape)


if __name__ == "__main__":
    main()
