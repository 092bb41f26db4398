"""Run under torchrun on 2+ GPUs: symmetric-memory all-reduce kernels and the GEMM-fused
all-reduce against the NCCL collective, with device-timed comparisons (max over ranks)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from stkernel_b200.ops import _lib                              # noqa: E402
from stkernel_b200.ops import functional as Fn                  # noqa: E402
from stkernel_b200.ops import reference as R                    # noqa: E402
from stkernel_b200.parallel.communicator import Communicator    # noqa: E402


def timed(fn, iters=20, warm=3):
    """Device time per call in us, from a CUDA graph holding `iters` calls (no host launch cost),
    max over ranks."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def measured_peer_store_bps(comm) -> float:
    """Bytes per second of 16-byte stores from this rank into the next rank's symmetric region (64 MiB, best of 5),
    minimum over ranks: the measured link figure the rooflines below divide by."""
    import ctypes
    L = _lib.lib()
    n = 64 << 20
    src = torch.empty(n, dtype=torch.uint8, device="cuda")
    heap = comm.symm.heap
    peer = (comm.rank + 1) % comm.world_size
    dst = heap.bases[peer] + comm.symm.layout["off_ag"]          # the two-shot all-gather buffer: >= 64 MiB, idle here
    one = lambda xs: (ctypes.c_longlong * 1)(*xs)
    best = float("inf")
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        assert L.stk_peer_copy(one([dst]), one([src.data_ptr()]), 1, n, 64, _lib.stream()) == 0
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e-3)
    dist.barrier()
    t = torch.tensor([n / best], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return float(t.item())


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    comm = Communicator(device=dev, use_symm=True, ag_bytes=4096 * 8192 * 2)
    out = {"world": world, "symm": comm.symm is not None, "disabled_reason": comm.disabled_reason, "allreduce": [], "gemm_ar": [],
           "ag_gemm": []}
    assert comm.symm is not None, comm.disabled_reason
    link_bps = measured_peer_store_bps(comm)
    out["peer_store_gbs_measured"] = link_bps * 1e-9
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    for numel in (4096, 6 * 4096, 64 * 4096, 256 * 4096, 4096 * 4096):
        x = torch.randn(numel, device=dev, generator=g).to(torch.bfloat16)
        ref = x.float()
        dist.all_reduce(ref)
        y = x.clone()
        comm.all_reduce(y)
        torch.cuda.synchronize()
        _lib.check_status()
        err = (y.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
        assert err < 2e-2, (numel, err)
        buf = x.clone()
        ours = timed(lambda: comm.all_reduce(buf))
        nccl = timed(lambda: dist.all_reduce(buf))
        nb = numel * 2
        # bytes this rank sends: one-shot pushes the whole buffer to every peer, two-shot 2 x (world-1)/world of it
        sent = nb * (world - 1) if nb <= comm.symm.oneshot_max else 2 * nb * (world - 1) // world
        roof = sent / link_bps * 1e6
        out["allreduce"].append({"bytes": nb, "ours_us": ours, "nccl_us": nccl, "rel_err": err, "nvlink_bytes_sent": sent,
                                 "achieved_nvlink_gbs": sent / ours * 1e-3, "frac_of_measured_link": roof / ours,
                                 "frac_of_900gbs": sent / 900e9 * 1e6 / ours})
    # ---- reduce-scatter / all-gather along dim 0 (sequence-parallel prefill), interleaved with all-reduces ----
    out["rs_ag"] = []
    for rows, hdim in ((world * 8, 4096), (1024, 4096), (4096, 4096)):
        rows = rows // world * world
        x = torch.randn(rows, hdim, device=dev, generator=g).to(torch.bfloat16)
        ref_rs = torch.empty(rows // world, hdim, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(ref_rs, x.float())
        shard = x[: rows // world].contiguous()
        ref_ag = torch.empty(rows, hdim, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(ref_ag, shard)
        for rep in range(3):                                   # back to back and around an all-reduce: the shared staging areas
            got_rs = comm.symm.reduce_scatter(x)
            comm.all_reduce(x.clone())
            got_ag = comm.symm.all_gather(shard)
            got_rs2 = comm.symm.reduce_scatter(x)
            got_ag2 = comm.symm.all_gather(shard)
            torch.cuda.synchronize()
            _lib.check_status()
            assert got_rs is not None and got_ag is not None
            e = ((got_rs.float() - ref_rs).norm() / ref_rs.norm()).item()
            assert e < 1e-2 and torch.equal(got_rs, got_rs2), ("reduce_scatter", rows, e)
            assert torch.equal(got_ag, ref_ag) and torch.equal(got_ag2, ref_ag), ("all_gather", rows)
        nb = rows * hdim * 2
        o_rs = torch.empty(rows // world, hdim, dtype=torch.bfloat16, device=dev)
        o_ag = torch.empty(rows, hdim, dtype=torch.bfloat16, device=dev)
        out["rs_ag"].append({"bytes": nb, "own_reduce_scatter_us": timed(lambda: comm.symm.reduce_scatter(x)),
                             "nccl_reduce_scatter_us": timed(lambda: dist.reduce_scatter_tensor(o_rs, x)),
                             "own_all_gather_us": timed(lambda: comm.symm.all_gather(shard)),
                             "nccl_all_gather_us": timed(lambda: dist.all_gather_into_tensor(o_ag, shard)),
                             "rs_rel_err": e})
    # ---- GEMM fused with the all-reduce (row-parallel layer) ----
    K_total, N = 8192, 4096
    k = K_total // world
    for dtype in ("bf16", "fp8"):
        for T in (1, 8, 64, 128):
            gw = torch.Generator(device=dev).manual_seed(7 + rank)
            x = torch.randn(T, k, device=dev, generator=gw).to(torch.bfloat16)
            w = torch.randn(N, k, device=dev, generator=gw) * 0.05
            lw = Fn.LinearWeight.from_master(w, dtype, dev)
            if dtype == "fp8":
                xq, xs = R.quant_fp8_group128_act(x)
                ref = R.dequant_fp8_group128_act(xq, xs) @ lw.dequant().t()
            else:
                ref = x.float() @ lw.dequant().t()
            dist.all_reduce(ref)
            ctx = comm.symm.gemm_ctx(T, N)
            assert ctx is not None
            y = None
            for _ in range(3):
                y = Fn.linear(x, lw, ar_ctx=ctx)
            torch.cuda.synchronize()
            _lib.check_status()
            err = ((y.float() - ref).norm() / ref.norm()).item()
            assert err < 2e-2, (dtype, T, err)
            fused = timed(lambda: Fn.linear(x, lw, ar_ctx=ctx))

            def base():
                o = Fn.linear(x, lw)
                dist.all_reduce(o)
            def base_symm():
                o = Fn.linear(x, lw)
                comm.all_reduce(o)
            def base_torch():
                o = x @ lw.w.t() if dtype == "bf16" else Fn.linear(x, lw)
                dist.all_reduce(o)
            out["gemm_ar"].append({"dtype": dtype, "T": T, "fused_us": fused, "gemm_then_nccl_us": timed(base),
                                   "gemm_then_oneshot_us": timed(base_symm),
                                   "cublas_then_nccl_us": timed(base_torch) if dtype == "bf16" else None, "rel_err": err})
    # ---- all-gather fused with the column-parallel GEMM (sequence-sharded activations) ----
    K, N_total = 8192, 4096
    n_loc = N_total // world
    for T in (8, 64, 256, 4096):
        if T % world:
            continue
        rows = T // world
        gw = torch.Generator(device=dev).manual_seed(31 + rank)
        xs = torch.randn(rows, K, device=dev, generator=gw).to(torch.bfloat16)
        w = (torch.randn(n_loc, K, device=dev, generator=gw) * 0.05).to(torch.bfloat16)
        full = torch.empty(T, K, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(full, xs)
        ref = full.float() @ w.float().t()
        y = None
        for _ in range(3):                       # odd count on purpose: both buffers get used
            y = comm.symm.ag_gemm(xs, w)
        torch.cuda.synchronize()
        _lib.check_status()
        err = ((y.float() - ref).norm() / ref.norm()).item()
        assert err < 2e-2, ("ag_gemm", T, err)
        comm.symm.ag_gemm(xs, w)                 # back to an even call count before graph capture
        fused = timed(lambda: comm.symm.ag_gemm(xs, w))
        lw = Fn.LinearWeight(w)

        def base_own():
            dist.all_gather_into_tensor(full, xs)
            Fn.linear(full, lw)
        def base_torch():
            dist.all_gather_into_tensor(full, xs)
            torch.matmul(full, w.t())
        flops = 2.0 * T * n_loc * K
        nvl = rows * K * 2 * (world - 1)         # bytes this rank receives
        roof = max(flops / 1613.6e12, nvl / link_bps) * 1e6
        roof900 = max(flops / 1613.6e12, nvl / 900e9) * 1e6
        out["ag_gemm"].append({"T": T, "fused_us": fused, "nccl_ag_then_own_gemm_us": timed(base_own),
                               "nccl_ag_then_cublas_us": timed(base_torch), "roofline_us": roof, "frac_of_roofline": roof / fused,
                               "frac_of_roofline_at_900gbs": roof900 / fused, "achieved_nvlink_gbs": nvl / fused * 1e-3,
                               "rel_err": err})
    if rank == 0:
        print("SYMM_OK " + json.dumps(out), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
