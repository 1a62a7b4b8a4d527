"""NVLink / NVSwitch probe on the library's symmetric heap: correctness of peer and multicast access, and the copy
bandwidths that the rooflines of the fused kernels use.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N -m unillm_b200.dist.probe_links [--mb 256] [--json PATH]

Per rank and message size it times (CUDA events around one kernel, best of 10 after a warm-up; the reported figure is
the minimum over ranks, i.e. the slowest rank):

  * ``peer_store``  : plain 16-byte stores of local data into the next rank's block (what the reduce-scatter epilogue
                      and the all-gather producer do without multicast);
  * ``peer_load``   : plain loads from the next rank's block into local memory;
  * ``multimem_st`` : one ``multimem.st`` per 16 bytes to the multicast address (the switch writes every rank's copy);
  * ``multimem_ld_reduce`` : ``multimem.ld_reduce`` (bf16x2 add, fp32 accumulation) of the multicast address into local
                      memory -- every rank pulls a different 1/N of the buffer, like the reduce-scatter consumer.

Before timing, every path is checked for values: a peer sees what its neighbour wrote, a multicast store lands on all
ranks, a multicast load returns the sum of the ranks' copies.  All ranks run the same kernel at the same time, so the
numbers are what a rank gets while its peers do the same, not a single-sender best case.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    import torch
    import torch.distributed as dist

    from .symm_heap import SymmetricHeap, probe

    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256, help="largest message in MiB (sizes go 1, 4, 16, ... up to this)")
    ap.add_argument("--json", default=None)
    ap.add_argument("--no-multicast", action="store_true")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    big = a.mb << 20
    heap = SymmetricHeap.create(2 * big, rank, world, dist.group.WORLD, dev, multicast=False if a.no_multicast else None)
    buf = heap.tensor()
    nxt = (rank + 1) % world
    out = {"world": world, "multicast": bool(heap.mc_ptr), "heap_bytes": heap.nbytes, "checks": {}, "gbs": {}}
    # ---- values: peer store / peer load ----
    n = 1 << 20
    src = torch.full((n,), rank + 1, dtype=torch.uint8, device=dev)
    probe(0, src.data_ptr(), heap.peer_ptrs[nxt], n, dev, iters=1)          # my pattern into the first MiB of my neighbour
    torch.cuda.synchronize()
    dist.barrier()
    prv = (rank - 1) % world
    ok_store = bool((buf[:n] == prv + 1).all())
    dst = torch.zeros(n, dtype=torch.uint8, device=dev)
    probe(0, heap.peer_ptrs[nxt], dst.data_ptr(), n, dev, iters=1)          # read my neighbour's first MiB
    torch.cuda.synchronize()
    ok_load = bool((dst == rank + 1).all())
    out["checks"]["peer_store"], out["checks"]["peer_load"] = ok_store, ok_load
    dist.barrier()
    # ---- values: multicast store / reduce ----
    if heap.mc_ptr:
        seg = 4096
        mine = torch.full((seg,), 10 + rank, dtype=torch.uint8, device=dev)
        probe(1, mine.data_ptr(), heap.mc_ptr + big + rank * seg, seg, dev, iters=1)   # my segment, on every rank
        torch.cuda.synchronize()
        dist.barrier()
        got = buf[big:big + world * seg].view(world, seg)
        out["checks"]["multimem_st"] = bool(all((got[r] == 10 + r).all() for r in range(world)))
        vals = torch.full((seg // 2,), float(rank + 1), dtype=torch.bfloat16, device=dev)
        buf[:seg].copy_(vals.view(torch.uint8))
        torch.cuda.synchronize()
        dist.barrier()
        red = torch.zeros(seg // 2, dtype=torch.bfloat16, device=dev)
        probe(2, heap.mc_ptr, red.data_ptr(), seg, dev, iters=1)
        torch.cuda.synchronize()
        out["checks"]["multimem_ld_reduce"] = bool((red.float() == world * (world + 1) / 2).all())
        dist.barrier()
    # ---- bandwidth ----
    sizes = []
    s = 1 << 20
    while s <= big:
        sizes.append(s)
        s *= 4
    local_src = torch.empty(big, dtype=torch.uint8, device=dev).random_(0, 255)
    local_dst = torch.empty(big, dtype=torch.uint8, device=dev)
    for sz in sizes:
        row = {}
        dist.barrier()
        row["peer_store"] = probe(0, local_src.data_ptr(), heap.peer_ptrs[nxt], sz, dev)
        dist.barrier()
        row["peer_load"] = probe(0, heap.peer_ptrs[nxt], local_dst.data_ptr(), sz, dev)
        if heap.mc_ptr:
            dist.barrier()
            row["multimem_st"] = probe(1, local_src.data_ptr(), heap.mc_ptr + big, sz, dev)
            dist.barrier()
            part = max(sz // world // 16 * 16, 16)
            row["multimem_ld_reduce"] = probe(2, heap.mc_ptr + rank * part, local_dst.data_ptr(), part, dev)
        t = torch.tensor([row[k] for k in sorted(row)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        out["gbs"][str(sz)] = {k: round(float(v), 1) for k, v in zip(sorted(row), t.tolist())}
    torch.cuda.synchronize()
    ok = all(out["checks"].values())
    flag = torch.tensor([int(ok)], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    out["all_ranks_ok"] = bool(int(flag[0]))
    heap.close()
    if rank == 0:
        line = json.dumps(out)
        print(line)
        if a.json:
            os.makedirs(os.path.dirname(a.json) or ".", exist_ok=True)
            with open(a.json, "w") as f:
                f.write(line + "\n")
    dist.destroy_process_group()
    return 0 if out["all_ranks_ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
