"""Peer-memory datapath probe: what one GPU reaches of another's HBM over NVLink / NVSwitch, measured.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m stkernel_b200.bench.peer_probe [--bytes 268435456] [--out FILE]

Every rank maps every peer's symmetric region (CUDA IPC) and times, with CUDA events on its own device:
  * stores to one peer and loads from one peer (16-byte accesses, one kernel), for every peer in turn;
  * stores to all peers at once and loads from all peers at once (one kernel, blocks spread over the peers);
  * a local copy of the same size (the HBM reference point);
  * the 8-byte flag round trip with every peer (release-store, remote acquire-poll, store back), 2000 rounds inside
    one kernel per side.
Rank 0 prints one JSON object: per-direction GB/s as the minimum, median and maximum over (rank, peer) pairs, the
all-peer aggregate per GPU, and the round-trip latency in microseconds.  The fused-collective rooflines in
`profiles/` and `tests/multigpu/symm_check.py` divide by these numbers (the counterpart of the reference's datapath
probe, probes/uma_datapath.cu:42-107).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics

import torch
import torch.distributed as dist


def _time_us(fn, iters: int = 5) -> float:
    fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3)
    return best


def probe(nbytes: int) -> dict:
    from ..ops import _lib
    from ..parallel.communicator import Communicator
    from ..parallel.symm import SymmetricHeap
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    comm = Communicator(device=dev, use_symm=False)
    heap = SymmetricHeap(comm, 2 * nbytes + 4096)           # [receive area | send area | flags]
    L = _lib.lib()
    st = _lib.status_buffer()
    local_src = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    local_dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    arr = lambda xs: (ctypes.c_longlong * len(xs))(*xs)
    peers = [p for p in range(world) if p != rank]
    stream = lambda: _lib.stream()

    def copy(dsts, srcs, per_peer_bytes, blocks=64):
        rc = L.stk_peer_copy(arr(dsts), arr(srcs), len(dsts), per_peer_bytes, blocks, stream())
        assert rc == 0, rc

    out = {"store_gbs": [], "load_gbs": [], "rtt_us": []}
    dist.barrier()
    # one peer at a time, one active pair per step so that a pair has the fabric to itself: step s pairs r with r ^ ... is
    # not defined for every world size, so ranks simply take turns
    for turn in range(world):
        if turn == rank:
            for p in peers:
                us = _time_us(lambda: copy([heap.bases[p]], [local_src.data_ptr()], nbytes))
                out["store_gbs"].append(nbytes / us * 1e-3)
                us = _time_us(lambda: copy([local_dst.data_ptr()], [heap.bases[p] + nbytes], nbytes))
                out["load_gbs"].append(nbytes / us * 1e-3)
        torch.cuda.synchronize()
        dist.barrier()
    # all peers at once, every rank at the same time (the pattern of an all-gather / all-to-all)
    share = (nbytes // max(1, len(peers))) // 16 * 16
    dist.barrier()
    us = _time_us(lambda: copy([heap.bases[p] + rank * 0 for p in peers], [local_src.data_ptr() + i * share for i, p in enumerate(peers)],
                               share, blocks=32))
    out["all_peer_store_gbs"] = share * len(peers) / us * 1e-3
    dist.barrier()
    us = _time_us(lambda: copy([local_dst.data_ptr() + i * share for i, p in enumerate(peers)], [heap.bases[p] + nbytes for p in peers],
                               share, blocks=32))
    out["all_peer_load_gbs"] = share * len(peers) / us * 1e-3
    dist.barrier()
    us = _time_us(lambda: copy([local_dst.data_ptr()], [local_src.data_ptr()], nbytes, blocks=296))
    out["local_copy_gbs"] = 2 * nbytes / us * 1e-3         # read + write bytes, as the HBM peak is quoted
    # flag round trips: pairs (a, b) one after the other; both sides launch, the initiator's device time is the figure
    rounds, base = 2000, 0
    flag_off = 2 * nbytes
    for a in range(world):
        for b in range(a + 1, world):
            base += rounds + 8
            if rank in (a, b):
                other = b if rank == a else a
                my_flag = heap.bases[rank] + flag_off + 8 * other
                peer_flag = heap.bases[other] + flag_off + 8 * rank
                torch.cuda.synchronize()
            dist.barrier()
            if rank in (a, b):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                rc = L.stk_peer_pingpong(ctypes.c_void_p(my_flag), ctypes.c_void_p(peer_flag), 1 if rank == a else 0, rounds, base,
                                         4_000_000, st.data_ptr(), stream())
                assert rc == 0
                e1.record()
                torch.cuda.synchronize()
                if rank == a:
                    out["rtt_us"].append(e0.elapsed_time(e1) * 1e3 / rounds)
            dist.barrier()
    _lib.check_status()
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    res = None
    if rank == 0:
        def stats(key):
            xs = [v for g in gathered for v in g[key]]
            return {"min": min(xs), "median": statistics.median(xs), "max": max(xs), "n": len(xs)} if xs else None
        res = {"world": world, "bytes": nbytes, "peer_store_gbs": stats("store_gbs"), "peer_load_gbs": stats("load_gbs"),
               "flag_round_trip_us": stats("rtt_us"),
               "all_peer_store_gbs_per_gpu": {"min": min(g["all_peer_store_gbs"] for g in gathered),
                                              "median": statistics.median(g["all_peer_store_gbs"] for g in gathered)},
               "all_peer_load_gbs_per_gpu": {"min": min(g["all_peer_load_gbs"] for g in gathered),
                                             "median": statistics.median(g["all_peer_load_gbs"] for g in gathered)},
               "local_copy_gbs": statistics.median(g["local_copy_gbs"] for g in gathered),
               "nominal_link_gbs_per_direction": 900.0}
    torch.cuda.synchronize()
    dist.barrier()
    heap.close()
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    res = probe(a.bytes // 16 * 16)
    if res is not None:
        print(json.dumps(res), flush=True)
        if a.out:
            with open(a.out, "w") as f:
                f.write(json.dumps(res) + "\n")
    os._exit(0)


if __name__ == "__main__":
    main()
