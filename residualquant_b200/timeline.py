"""Where a small attention call's time goes: per-phase timestamps from inside the kernel.

    python -m residualquant_b200.build --timeline
    RQ_B200_LIBRARY=residualquant_b200/librq_b200_timeline.so \
        python -m residualquant_b200.timeline --batch 1 --context 8192 [--heads 16] [--head-dim 128] [--ragged]

Needs the timeline build of the library (phase timestamps compiled into the attention kernels, see
csrc/rq_attention_impl.cuh) and a GPU.  It fills one layer's packed cache with synthetic rows, captures a CUDA graph of
twelve attention calls that alternate between loop 0 and loop 1 (both residual loops: the same kernel), replays it, and
reads back the timestamps of the last two launches.  Per phase it prints the median and the maximum over the CTAs that
had work, in microseconds (cycle counts divided by the SM clock that nvidia-smi reports), and from the global timer how
the two launches overlap: when the second launch's CTAs entered relative to the first one's end, and the period from
one launch's end to the next's.  Time per call under replay is measured with CUDA events around the graph.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import subprocess

import numpy as np
import torch

from . import _cuda, _lib, rotation, synth

SLOTS = ("entry_global_ns", "entry", "after_lookup", "after_staging", "after_wait", "after_query", "after_pages",
         "after_warp_fold", "after_ticket", "after_partitions", "exit", "exit_global_ns", "lookup_loads_issued",
         "lookup_loads_arrived", "lookup_chosen", "query_rotated", "query_shared", "sm_id_plus_one")
TIMELINE_CTAS = 4096
PHASES = (  # name, from slot, to slot
    ("work lookup", "entry", "after_lookup"),
    ("  loads issued", "entry", "lookup_loads_issued"),
    ("  loads arrived", "lookup_loads_issued", "lookup_loads_arrived"),
    ("  partition choice", "lookup_loads_arrived", "lookup_chosen"),
    ("  item -> (row, part), barrier", "lookup_chosen", "after_lookup"),
    ("block table + first stage fetches", "after_lookup", "after_staging"),
    ("wait for the previous kernel", "after_staging", "after_wait"),
    ("query: rotate (warp 0)", "after_wait", "query_rotated"),
    ("query: barrier", "query_rotated", "query_shared"),
    ("query: integer operands", "query_shared", "after_query"),
    ("page loop", "after_query", "after_pages"),
    ("warp fold", "after_pages", "after_warp_fold"),
    ("CTA fold + ticket", "after_warp_fold", "after_ticket"),
    ("last CTA: fold the partitions", "after_ticket", "after_partitions"),
    ("epilogue", "after_partitions", "exit"),
)


def sm_clock_mhz(device_index: int) -> float:
    out = subprocess.run(["nvidia-smi", f"--id={device_index}", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits"],
                         capture_output=True, text=True)
    try:
        return float(out.stdout.strip().splitlines()[0])
    except (ValueError, IndexError):
        return 1965.0


def build_case(batch, lengths, heads, head_dim, page, device, seed=5):
    """One layer's packed cache ([2,2,2,4] g32, anchor last) filled with synthetic rows through `quantize`."""
    rng = np.random.default_rng(seed)
    records = [[2, 32], [2, 32], [2, 32], [4, 32]]
    width = sum(head_dim * b // 8 + 2 * (head_dim // g) + 2 for b, g in records)
    table, blocks = synth.paging(rng, [n + page for n in lengths], page)
    cache = torch.zeros((2, blocks, heads, page, width), dtype=torch.uint8, device=device)
    key_rotation = rotation.signed_hadamard(synth.signs(rng, heads, head_dim), float(synth.fp16_rsqrt(head_dim)), device)
    block_table = torch.from_numpy(table).to(device)
    for request, length in enumerate(lengths):
        done = 0
        while done < length - 1:                       # the last token of every sequence is the live one
            count = min(2048, length - 1 - done)
            rows_k = [torch.from_numpy(r).to(device).bfloat16() for r in synth.loop_rows(rng, count, heads, head_dim)]
            rows_v = [torch.from_numpy(r).to(device).bfloat16() for r in synth.loop_rows(rng, count, heads, head_dim)]
            positions = np.arange(done, done + count)
            slots = torch.from_numpy(synth.slots_for(table, request, positions, page)).to(device)
            _cuda.quantize(list(zip(rows_k, rows_v)), cache, slots, key_rotation, None, None, records, "anchor", 3, "ls")
            done += count
    return cache, block_table, key_rotation, records


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--context", type=int, default=8192)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--head-dim", type=int, default=128, choices=[96, 128])
    parser.add_argument("--page", type=int, default=16)
    parser.add_argument("--ragged", action="store_true", help="row 0 at --context, the others 17..600 tokens")
    parser.add_argument("--plain", action="store_true", help="without the stable-metadata promise (no early start)")
    parser.add_argument("--json", action="store_true")
    args = parser.parse_args()

    lib = _lib.load()
    name = f"rq_timeline_d{args.head_dim}"
    if not hasattr(lib, name):
        raise SystemExit("this is not a timeline build of the library: `python -m residualquant_b200.build --timeline`, then set "
                         "RQ_B200_LIBRARY=residualquant_b200/librq_b200_timeline.so")
    read_back = getattr(lib, name)
    read_back.argtypes, read_back.restype = [ctypes.c_void_p, ctypes.c_size_t], ctypes.c_int

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    lengths = [args.context] * args.batch
    if args.ragged:
        lengths[1:] = [int(v) for v in np.random.default_rng(7).integers(17, 601, size=args.batch - 1)]
    cache, block_table, key_rotation, records = build_case(args.batch, lengths, args.heads, args.head_dim, args.page, device)
    rows = args.batch
    q, k, v = (torch.randn(rows, args.heads, args.head_dim, device=device).bfloat16() for _ in range(3))
    out = torch.zeros_like(q)
    qsl = torch.arange(rows + 1, dtype=torch.int32, device=device)
    seq = torch.tensor(lengths, dtype=torch.int32, device=device)
    _cuda.set_stable_metadata(not args.plain)

    def calls():
        for _ in range(6):
            for loop in (0, 1):
                _cuda.attention(q, k, v, cache, out, qsl, seq, block_table, key_rotation, None, None, records, "anchor", 3, loop)

    stream = torch.cuda.Stream(device)
    stream.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(stream):
        calls()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            calls()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            graph.replay()
        begin.record(stream)
        for _ in range(10):
            graph.replay()
        end.record(stream)
        stream.synchronize()
    us_per_call = 1000.0 * begin.elapsed_time(end) / 120.0
    _cuda.attention_status(device)

    stamps = np.zeros((2, TIMELINE_CTAS, len(SLOTS)), dtype=np.uint64)
    if read_back(stamps.ctypes.data_as(ctypes.c_void_p), stamps.nbytes) != 0:
        raise SystemExit("reading the timeline back failed")
    ghz = sm_clock_mhz(0) / 1000.0
    index = {slot: i for i, slot in enumerate(SLOTS)}
    report = {"us_per_call": round(us_per_call, 2), "sm_clock_mhz": round(1000.0 * ghz), "launches": []}
    for half in (0, 1):
        t = stamps[half].astype(np.int64)
        launched = t[:, index["entry_global_ns"]] > 0
        worked = launched & (t[:, index["after_query"]] > 0)
        phases = {}
        for label, start, stop in PHASES:
            lo, hi = t[worked, index[start]], t[worked, index[stop]]
            ok = (lo > 0) & (hi > 0)
            if ok.any():
                us = (hi[ok] - lo[ok]) / ghz / 1000.0
                phases[label] = [round(float(np.median(us)), 2), round(float(us.max()), 2)]
        sms = t[worked, index["sm_id_plus_one"]] - 1
        per_sm = np.bincount(sms, minlength=1)
        histogram = {int(n): int(c) for n, c in zip(*np.unique(per_sm, return_counts=True))}
        report["launches"].append({"ctas_launched": int(launched.sum()), "ctas_with_work": int(worked.sum()), "phases": phases,
                                   "working_ctas_per_sm": histogram,
                                   "sm_of_first_ctas": [int(v) for v in (t[:12, index["sm_id_plus_one"]] - 1)],
                                   "first_entry_ns": int(t[launched, index["entry_global_ns"]].min()),
                                   "last_exit_ns": int(t[:, index["exit_global_ns"]].max())})
    first, second = report["launches"]
    report["overlap"] = {"second_enters_before_first_ends_us": round((first["last_exit_ns"] - second["first_entry_ns"]) / 1000.0, 2),
                         "end_to_end_period_us": round((second["last_exit_ns"] - first["last_exit_ns"]) / 1000.0, 2)}
    if args.json:
        print(json.dumps(report))
        return
    print(f"batch {args.batch} x context {args.context}{' (ragged)' if args.ragged else ''}, {args.heads} heads x {args.head_dim}: "
          f"{report['us_per_call']} us per call under graph replay, SM clock {report['sm_clock_mhz']} MHz")
    print(f"CTAs launched {second['ctas_launched']}, with work {second['ctas_with_work']}; the next launch's CTAs enter "
          f"{report['overlap']['second_enters_before_first_ends_us']} us before this one ends; period "
          f"{report['overlap']['end_to_end_period_us']} us")
    print(f"SMs by number of working CTAs they ran {second['working_ctas_per_sm']}; SMs of CTAs 0..11: {second['sm_of_first_ctas']}")
    print(f"{'phase (second of two consecutive launches)':46s} {'median us':>10s} {'max us':>8s}")
    for label, (median, worst) in second["phases"].items():
        print(f"{label:46s} {median:10.2f} {worst:8.2f}")


if __name__ == "__main__":
    main()
