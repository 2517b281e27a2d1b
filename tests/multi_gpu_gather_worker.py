"""One rank of the two-GPU head-gather test (launched by tests/test_gpu_head_gather_multi.py under torchrun).

KV heads are split unevenly over the ranks (5 = 3 + 2).  All three forms of the fused gather run several calls with the two
gathered buffers alternating: the barrier form (`HeadGather.barrier()` after every call), the signalled form (the
kernel publishes, the next call waits) and the complete form (the kernel publishes and stays until every rank has).
After every form the gathered rows must equal an NCCL all-gather of the ranks' own outputs bit for bit, the state block
must show no timeout, and in the barrier and complete forms a copy queued right behind every call must already hold
every rank's rows of that call.  Peer stores are plain stores; no multicast."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from residualquant_b200 import _cuda, sharding  # noqa: E402
from tests import gpu_helpers as G  # noqa: E402
from tests import helpers  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    device = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=device)
    heads = 5
    begin, end = sharding.shard_range(heads, world, rank)
    full = helpers.make_case(91, 128, heads, [260, 33, 1, 120], 32, 16)      # the same case on every rank
    cache = torch.from_numpy(np.ascontiguousarray(helpers.oracle_cache(full)[:, :, begin:end])).to(device)
    rows = len(full.seq_lens)
    from residualquant_b200 import rotation

    kr = rotation.signed_hadamard(full.key_signs[begin:end], float(full.rscale), device)
    vr = rotation.signed_hadamard(full.value_signs[begin:end], float(full.rscale), device)
    q = G.bf16(full.query[:, begin:end], device)
    qsl = torch.arange(rows + 1, dtype=torch.int32, device=device)
    seq = torch.from_numpy(full.seq_lens).to(device)
    table = torch.from_numpy(full.block_table).to(device)
    records = [list(r) for r in full.layout.records]
    failures = []
    for form in ("barrier", "signalled", "complete"):
        gather = sharding.HeadGather(rows, heads, 128, device, buffers=2, signalled=form == "signalled",
                                     complete=form == "complete")
        outs, snapshots = [], []
        for call, loop in enumerate((0, 1, 2, 3, 1, 0, 3)):
            k = G.bf16(full.keys[loop][full.live_rows][:, begin:end], device)
            v = G.bf16(full.values[loop][full.live_rows][:, begin:end], device)
            out = torch.zeros_like(q)
            _cuda.attention(q, k, v, cache, out, qsl, seq, table, kr, vr, None, records, "anchor", 3, loop,
                            gather=gather, gather_buffer=call % 2)
            if form == "barrier":
                gather.barrier()
            if form != "signalled":
                # what a consumer queued right behind the call (and its barrier) reads: every rank's rows of THIS call
                snapshots.append(gather.gathered(call % 2).clone())
            outs.append((loop, call % 2, out))
        if form == "signalled":
            gather.barrier()     # the consumer's wait
        gather.check()
        torch.cuda.synchronize(device)
        for index, (loop, buffer, out) in enumerate(outs):
            expected = sharding.gather_heads(out, heads)
            if snapshots and not torch.equal(snapshots[index], expected):
                failures.append(f"{form} call {index}: the rows read behind the call differ from the all-gather")
            if index < len(outs) - 2:
                continue
            if not torch.equal(gather.gathered(buffer), expected):
                failures.append(f"{form} loop {loop}: gathered rows differ from the all-gather")
            want = helpers.oracle_attention(full, helpers.oracle_cache(full), loop)
            got = expected.float().cpu().numpy()
            if not np.all(np.abs(got - want) <= 2e-2 + 1e-2 * np.abs(want)):
                failures.append(f"{form} loop {loop}: outside the tolerance of the oracle")
        state = gather.state[:3].tolist()
        if state[1] != 0 or state[0] != 7:
            failures.append(f"{form}: state {state}")
        gather.close()
    flag = torch.tensor([len(failures)], device=device)
    dist.all_reduce(flag)
    dist.destroy_process_group()
    if failures:
        print("\n".join(failures), file=sys.stderr)
    sys.exit(1 if int(flag.item()) else 0)


if __name__ == "__main__":
    main()
