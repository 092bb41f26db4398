"""Device-timed decode / prefill benchmark of the Flash-shaped model (used by the top-level bench.py)."""
from __future__ import annotations

import time
from typing import Dict, List

import torch
import torch.distributed as dist

from ..config import CacheConfig, EngineConfig, ParallelConfig, SchedulerConfig, flash_config
from ..models.dsv4 import RandomSource, build_model_weights
from ..ops import _lib
from ..ops import cache as C
from ..ops.cache import PAGE
from ..runtime.engine import Engine, Request, SamplingParams


def _max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _sync(world: int) -> None:
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def fill_caches_synthetic(eng: Engine, seed: int = 0) -> None:
    """Write random (finite) rows into every page of every cache, through the same insert kernel
    the model uses for latent rows; indexer-K pages get random e4m3 values with unit scales."""
    dev = eng.device
    g = torch.Generator(device=dev).manual_seed(seed)
    cfg = eng.cfg.model
    inv = eng.model.inv
    for group in (eng.kv.swa_cache, eng.kv.comp_cache):
        for li, cache in group.items():
            n = cache.num_slots
            step = 1 << 16
            for s0 in range(0, n, step):
                m = min(step, n - s0)
                kv = torch.randn(m, cache.dim, device=dev, generator=g).to(torch.bfloat16)
                pos = torch.arange(s0, s0 + m, device=dev, dtype=torch.int64) % 100000
                slots = torch.arange(s0, s0 + m, device=dev, dtype=torch.int64)
                C.kv_rope_quant_insert(kv, pos, slots, inv, cache)
    for li, cache in eng.kv.idx_cache.items():
        d = cache.dim
        vals = torch.randn(cache.num_pages, PAGE * d, device=dev, generator=g)
        if cache.fp8:
            cache.buf[:, :PAGE * d] = vals.to(torch.float8_e4m3fn).view(torch.uint8)
            ones = torch.ones(cache.num_pages, PAGE, device=dev).view(torch.uint8).view(cache.num_pages, PAGE * 4)
            cache.buf[:, PAGE * d:PAGE * d + PAGE * 4] = ones
        else:
            cache.buf[:, :PAGE * d * 2] = vals.to(torch.bfloat16).view(torch.uint8).view(cache.num_pages, -1)
    torch.cuda.synchronize()


def _adopt_context(eng: Engine, row: int, ctx: int) -> None:
    """Allocate the pages a request with `ctx` computed tokens holds: all compressed rows, the SWA window."""
    if ctx // 4 > 0:
        eng.kv.c4.ensure(row, 0, (ctx // 4 - 1) // PAGE)
    eng.kv.prepare(row, ctx, 1)


def add_synthetic_requests(eng: Engine, n: int, ctx: int, max_tokens: int, vocab: int, seed: int) -> List[int]:
    """Admit `n` requests whose first `ctx` tokens count as already computed (their pages are
    allocated and hold the synthetic rows written by `fill_caches_synthetic`)."""
    ids = []
    g = torch.Generator().manual_seed(seed)
    for i in range(n):
        prompt = torch.randint(0, vocab, (ctx + 1,), generator=g).tolist()
        rid = eng.add_request(prompt, SamplingParams(temperature=0.0, seed=i, max_tokens=max_tokens))
        req = eng.sched.waiting.pop()
        req.row = eng.kv.alloc_row()
        _adopt_context(eng, req.row, ctx)
        req.num_computed = ctx
        eng.sched.running.append(req)
        ids.append(rid)
    return ids


def timed_steps(eng: Engine, steps: int, world: int, forced_vocab: int, n_rows: int, host_roundtrip: bool):
    """-> (ms per step by CUDA events, ms per step by wall clock), max over ranks."""
    g = torch.Generator().manual_seed(123)
    forced = [torch.randint(0, forced_vocab, (n_rows,), generator=g).tolist() for _ in range(steps)]
    _sync(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        eng.step(None if host_roundtrip else forced[i])
    e1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3 / steps
    dev_ms = e0.elapsed_time(e1) / steps
    _sync(world)
    return _max_over_ranks(dev_ms, world, eng.device), _max_over_ranks(wall, world, eng.device)


def run_bench(n_gpus: int, rank: int, local: int, steps: int, warmup: int, ctx: int, layers_per_gpu: int,
              extra: bool = True, fused: bool = True, conc_extra: int = 64, real_prefill: bool = True) -> Dict:
    dev = torch.device(f"cuda:{local}")
    layers = layers_per_gpu * n_gpus
    mcfg = flash_config(num_layers=layers)
    total_steps = warmup * 3 + steps * 2 + 64
    ecfg = EngineConfig(
        model=mcfg, parallel=ParallelConfig(tp_size=n_gpus, ep_size=n_gpus, fused_collectives=fused),
        sched=SchedulerConfig(max_model_len=ctx + total_steps + 64, max_num_seqs=conc_extra, max_num_batched_tokens=4096,
                              graph_cap=conc_extra)).validate()
    comm = None
    if n_gpus > 1:
        from ..parallel.communicator import Communicator
        comm = Communicator(device=dev, use_symm=fused)
    t0 = time.time()
    weights = build_model_weights(mcfg, RandomSource(0), dev, rank, n_gpus, head_fp8=True)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    eng = Engine(ecfg, weights, dev, comm, rank, max_context=ctx + total_steps + 64)
    res: Dict = {"layers": layers, "build_s": build_s}
    vocab = mcfg.vocab_size
    g = torch.Generator().manual_seed(1)

    # ---- prefill of one 32K-token prompt (real), chunked 4096 ----
    prompt = torch.randint(0, vocab, (ctx,), generator=g).tolist()
    rid = eng.add_request(prompt, SamplingParams(temperature=0.0, seed=0, max_tokens=total_steps))
    if real_prefill:
        # warm the prefill kernels on a short throw-away request first
        _sync(n_gpus)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        n_chunks = 0
        while eng.requests[rid].in_prefill:
            eng.step()
            n_chunks += 1
        e1.record()
        torch.cuda.synchronize()
        pre_ms = _max_over_ranks(e0.elapsed_time(e1), n_gpus, dev)
        res["extra"] = {"prefill_32k_tok_s_first_pass": ctx / pre_ms * 1e3, "prefill_chunks": n_chunks}
        res["context_fill"] = "real chunked prefill of the 32K prompt"
    else:
        fill_caches_synthetic(eng)
        req = eng.sched.waiting.pop()
        req.row = eng.kv.alloc_row()
        _adopt_context(eng, req.row, ctx)
        req.num_computed = ctx
        req.prompt = req.prompt + [1]
        eng.sched.running.append(req)
        res["extra"] = {}
        res["context_fill"] = "synthetic random rows in every cache page"
    _lib.check_status()

    # ---- decode, C = 1 ----
    timed_steps(eng, warmup, n_gpus, vocab, 1, False)
    l0 = _lib.launch_count
    dev_ms, _ = timed_steps(eng, steps, n_gpus, vocab, 1, False)
    res["gpu_launches"] = _lib.launch_count - l0
    res["decode_c1_ms"] = dev_ms
    res["decode_c1_tok_s"] = 1e3 / dev_ms
    timed_steps(eng, warmup, n_gpus, vocab, 1, True)
    ev_ms, wall_ms = timed_steps(eng, steps, n_gpus, vocab, 1, True)
    res["e2e_ms"] = wall_ms
    res["e2e_tok_s"] = 1e3 / wall_ms
    res["h2d_bytes"] = eng.h2d_bytes_last
    res["d2h_bytes"] = eng.d2h_bytes_last
    _lib.check_status()

    if extra:
        # ---- second prefill pass (kernels warm) for the prefill figure ----
        if real_prefill:
            rid2 = eng.add_request(torch.randint(0, vocab, (ctx,), generator=g).tolist(),
                                   SamplingParams(temperature=0.0, seed=1, max_tokens=1))
            # keep request 0 out of the way: finish it
            eng.sched.retire(eng.requests[rid])
            _sync(n_gpus)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            while eng.requests[rid2].in_prefill:
                eng.step()
            e1.record()
            torch.cuda.synchronize()
            pre_ms = _max_over_ranks(e0.elapsed_time(e1), n_gpus, dev)
            res["extra"]["prefill_32k_tok_s"] = ctx / pre_ms * 1e3
            res["extra"]["prefill_32k_ms"] = pre_ms
            while eng.has_work():
                eng.step()
        else:
            eng.sched.retire(eng.requests[rid])
        # ---- decode, C = 64 over synthetic 32K contexts ----
        fill_caches_synthetic(eng)
        add_synthetic_requests(eng, conc_extra, ctx, warmup + max(8, steps // 4) + 8, vocab, 7)
        timed_steps(eng, warmup, n_gpus, vocab, conc_extra, False)
        k2 = max(8, steps // 4)
        dev_ms64, _ = timed_steps(eng, k2, n_gpus, vocab, conc_extra, False)
        res["extra"][f"decode_c{conc_extra}_ms_per_step"] = dev_ms64
        res["extra"][f"decode_c{conc_extra}_tok_s"] = conc_extra * 1e3 / dev_ms64
        res["extra"]["decode_c64_context_fill"] = "synthetic random rows in every cache page"
        _lib.check_status()
    res["extra"]["weights_build_s"] = build_s
    if comm is not None:
        res["extra"]["collective_calls"] = dict(comm.calls)
        res["extra"]["symm_disabled_reason"] = comm.disabled_reason
    return res
