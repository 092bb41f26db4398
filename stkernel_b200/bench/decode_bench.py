"""Device-timed decode / prefill benchmark of the Flash-shaped model (used by the top-level bench.py).

Phases (each its own engine where the cache geometry differs):
  1. 32K context: real chunked prefill of one prompt, decode at C=1 (device-timed and end to end through
     `Engine.step()`), a second (warm) prefill pass, decode at C=64 over synthetic 32K contexts;
  2. 128K context: decode at C=1 and C=64 over synthetic contexts;
  3. DSpark speculative decoding at C=1 and C=16: cost of the speculative step against the plain step, and the
     accept path driven by a replay drafter at the reference's published per-position acceptance.

Every timed figure is the median of R repeats of exactly K steps, each repeat bracketed by a barrier and a device
synchronisation, timed with CUDA events, maximum over ranks; R is chosen so that a phase runs for about half a second.
"""
from __future__ import annotations

import random
import time
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..config import EngineConfig, ParallelConfig, SchedulerConfig, SpecConfig, flash_config
from ..models.dsv4 import RandomSource, build_model_weights
from ..ops import _lib
from ..ops import cache as C
from ..ops.cache import PAGE
from ..runtime.engine import Engine, Request, SamplingParams

# cumulative per-position acceptance of the reference's trained drafter (MEASUREMENTS.md:49-51)
REFERENCE_ACCEPTANCE = (0.785, 0.564, 0.396, 0.286, 0.215)


def _max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _min_over_ranks(x: float, world: int, device) -> float:
    return -_max_over_ranks(-x, world, device)


def _sync(world: int) -> None:
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def fill_caches_synthetic(eng: Engine, seed: int = 0) -> None:
    """Write random (finite) rows into every page of every cache, through the same insert kernel
    the model uses for latent rows; indexer-K pages get random e4m3 values with unit scales."""
    dev = eng.device
    g = torch.Generator(device=dev).manual_seed(seed)
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
        step = 4096
        for p0 in range(0, cache.num_pages, step):
            m = min(step, cache.num_pages - p0)
            vals = torch.randn(m, PAGE * d, device=dev, generator=g)
            if cache.fp8:
                cache.buf[p0:p0 + m, :PAGE * d] = vals.to(torch.float8_e4m3fn).view(torch.uint8)
                ones = torch.ones(m, PAGE, device=dev).view(torch.uint8).view(m, PAGE * 4)
                cache.buf[p0:p0 + m, PAGE * d:PAGE * d + PAGE * 4] = ones
            else:
                cache.buf[p0:p0 + m, :PAGE * d * 2] = vals.to(torch.bfloat16).view(torch.uint8).view(m, -1)
    torch.cuda.synchronize()


def _adopt_context(eng: Engine, row: int, ctx: int) -> None:
    """Allocate the pages a request with `ctx` computed tokens holds: all compressed rows, the SWA window."""
    if ctx // 4 > 0:
        eng.kv.c4.ensure(row, 0, (ctx // 4 - 1) // PAGE)
    eng.kv.prepare(row, ctx, 1)


def add_synthetic_requests(eng: Engine, n: int, ctx: int, max_tokens: int, vocab: int, seed: int,
                           temperature: float = 0.0) -> List[int]:
    """Admit `n` requests whose first `ctx` tokens count as already computed (their pages are
    allocated and hold the synthetic rows written by `fill_caches_synthetic`)."""
    ids = []
    g = torch.Generator().manual_seed(seed)
    for i in range(n):
        prompt = torch.randint(0, vocab, (ctx + 1,), generator=g).tolist()
        rid = eng.add_request(prompt, SamplingParams(temperature=temperature, seed=i, max_tokens=max_tokens))
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
    # third value: the fastest rank's device time (the ranks run the same step; the gap to the maximum is rank skew)
    return (_max_over_ranks(dev_ms, world, eng.device), _max_over_ranks(wall, world, eng.device),
            _min_over_ranks(dev_ms, world, eng.device))


def timed_repeats(eng: Engine, steps: int, world: int, vocab: int, n_rows: int, host_roundtrip: bool,
                  min_seconds: float = 0.5, max_repeats: int = 40) -> Dict:
    """Repeats of exactly `steps` steps until the phase has run for `min_seconds` (at least 3, at most `max_repeats`;
    the count follows the first repeat's time, which every rank knows as the same max-over-ranks number)."""
    first = timed_steps(eng, steps, world, vocab, n_rows, host_roundtrip)
    per = max(first[0], first[1]) * steps / 1e3
    reps = int(min(max_repeats, max(3, -(-min_seconds // max(per, 1e-6)))))
    runs = [first] + [timed_steps(eng, steps, world, vocab, n_rows, host_roundtrip) for _ in range(reps - 1)]
    dev = sorted(r[0] for r in runs)
    wall = sorted(r[1] for r in runs)
    mid = sorted(runs, key=lambda r: r[0])[len(runs) // 2]
    return {"dev_ms": dev[len(dev) // 2], "wall_ms": wall[len(wall) // 2], "repeats": len(runs),
            "dev_ms_min": dev[0], "dev_ms_max": dev[-1], "wall_ms_min": wall[0], "wall_ms_max": wall[-1],
            "dev_ms_fastest_rank": mid[2], "dev_ms_slowest_rank": mid[0]}


def _engine(mcfg, n_gpus: int, rank: int, dev, comm, weights, fused: bool, max_ctx: int, max_seqs: int, graph_cap: int,
            spec: Optional[SpecConfig] = None, draft_weights=None) -> Engine:
    ecfg = EngineConfig(
        model=mcfg, parallel=ParallelConfig(tp_size=n_gpus, ep_size=n_gpus, fused_collectives=fused),
        sched=SchedulerConfig(max_model_len=max_ctx, max_num_seqs=max_seqs, max_num_batched_tokens=4096, graph_cap=graph_cap),
        spec=spec or SpecConfig()).validate()
    return Engine(ecfg, weights, dev, comm, rank, max_context=max_ctx, draft_weights=draft_weights)


def multi_gpu_self_check(comm, dev) -> Dict:
    """A one-second correctness check of the own collectives against the library's, run before anything is timed:
    relative errors of the one-shot / two-shot all-reduce and of the all-reduce folded into a projection and the
    mHC pre-mix, maximum over ranks."""
    from ..ops import functional as Fn
    out: Dict = {}
    world = comm.world_size
    g = torch.Generator(device=dev).manual_seed(77 + comm.rank)

    def rel(a, b):
        e = ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()
        return _max_over_ranks(e, world, dev)

    for name, numel in (("oneshot_8KiB", 4096), ("twoshot_8MiB", 4096 * 1024)):
        x = torch.randn(numel, device=dev, generator=g).to(torch.bfloat16)
        ref = x.float()
        dist.all_reduce(ref)
        y = comm.all_reduce(x.clone())
        out[name] = rel(y, ref)
    ll = comm.symm.ll_exchange(2, 4096) if comm.symm is not None else None
    if ll is not None:
        x = torch.randn(2, 1024, device=dev, generator=g).to(torch.bfloat16)
        w = Fn.LinearWeight((torch.randn(4096, 1024, device=dev, generator=g) * 0.05).to(torch.bfloat16))
        ref = Fn.linear(x, w).float()
        dist.all_reduce(ref)
        got = Fn.ll_reduce(Fn.linear(x, w, ll=ll))
        out["folded_allreduce_projection"] = rel(got, ref)
    torch.cuda.synchronize()
    _lib.check_status()
    out["symm_enabled"] = comm.symm is not None and comm.symm.enabled
    return out


def run_bench(n_gpus: int, rank: int, local: int, steps: int, warmup: int, ctx: int, layers_per_gpu: int,
              extra: bool = True, fused: bool = True, conc_extra: int = 64, real_prefill: bool = True,
              long_ctx: int = 131072, spec: bool = True) -> Dict:
    dev = torch.device(f"cuda:{local}")
    layers = layers_per_gpu * n_gpus
    mcfg = flash_config(num_layers=layers)
    headroom = 7168                     # decode steps a request may take before its compressed-row graph bucket changes
    comm = None
    res: Dict = {"layers": layers, "extra": {}}
    if n_gpus > 1:
        from ..parallel.communicator import Communicator
        comm = Communicator(device=dev, use_symm=fused)
        res["extra"]["multi_gpu_self_check"] = multi_gpu_self_check(comm, dev)
    t0 = time.time()
    weights = build_model_weights(mcfg, RandomSource(0), dev, rank, n_gpus, head_fp8=True)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    res["build_s"] = build_s
    vocab = mcfg.vocab_size
    g = torch.Generator().manual_seed(1)

    # ================= phase 1: 32K context =================
    eng = _engine(mcfg, n_gpus, rank, dev, comm, weights, fused, ctx + headroom + 64, conc_extra, conc_extra)
    prompt = torch.randint(0, vocab, (ctx,), generator=g).tolist()
    rid = eng.add_request(prompt, SamplingParams(temperature=0.0, seed=0, max_tokens=headroom))
    if real_prefill:
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
        res["extra"].update({"prefill_32k_tok_s_first_pass": ctx / pre_ms * 1e3, "prefill_chunks": n_chunks})
        res["context_fill"] = "real chunked prefill of the 32K prompt"
    else:
        fill_caches_synthetic(eng)
        req = eng.sched.waiting.pop()
        req.row = eng.kv.alloc_row()
        _adopt_context(eng, req.row, ctx)
        req.num_computed = ctx
        req.prompt = req.prompt + [1]
        eng.sched.running.append(req)
        res["context_fill"] = "synthetic random rows in every cache page"
    _lib.check_status()

    # ---- decode, C = 1 ----
    timed_steps(eng, warmup, n_gpus, vocab, 1, False)
    l0 = _lib.launch_count
    r1 = timed_repeats(eng, steps, n_gpus, vocab, 1, False)
    res["gpu_launches"] = (_lib.launch_count - l0) // r1["repeats"]
    res["decode_c1_ms"] = r1["dev_ms"]
    res["decode_c1_tok_s"] = 1e3 / r1["dev_ms"]
    res["decode_c1_repeats"] = r1
    timed_steps(eng, warmup, n_gpus, vocab, 1, True)
    r2 = timed_repeats(eng, steps, n_gpus, vocab, 1, True)
    res["e2e_ms"] = r2["wall_ms"]
    res["e2e_tok_s"] = 1e3 / r2["wall_ms"]
    res["e2e_repeats"] = r2
    res["h2d_bytes"] = eng.h2d_bytes_last
    res["d2h_bytes"] = eng.d2h_bytes_last
    _lib.check_status()

    if extra:
        # ---- second prefill pass (kernels warm) for the prefill figure ----
        if real_prefill:
            rid2 = eng.add_request(torch.randint(0, vocab, (ctx,), generator=g).tolist(),
                                   SamplingParams(temperature=0.0, seed=1, max_tokens=1))
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
        add_synthetic_requests(eng, conc_extra, ctx, headroom, vocab, 7)
        timed_steps(eng, warmup, n_gpus, vocab, conc_extra, False)
        r64 = timed_repeats(eng, max(8, steps // 4), n_gpus, vocab, conc_extra, False)
        res["extra"][f"decode_c{conc_extra}_ms_per_step"] = r64["dev_ms"]
        res["extra"][f"decode_c{conc_extra}_tok_s"] = conc_extra * 1e3 / r64["dev_ms"]
        res["extra"]["decode_c64_context_fill"] = "synthetic random rows in every cache page"
        _lib.check_status()
    del eng
    torch.cuda.empty_cache()

    # ================= phase 2: 128K context (synthetic cache rows) =================
    if extra and long_ctx > ctx:
        eng = _engine(mcfg, n_gpus, rank, dev, comm, weights, fused, long_ctx + headroom + 64, conc_extra, conc_extra)
        fill_caches_synthetic(eng)
        ids = add_synthetic_requests(eng, 1, long_ctx, headroom, vocab, 11)
        timed_steps(eng, warmup, n_gpus, vocab, 1, False)
        rl1 = timed_repeats(eng, steps, n_gpus, vocab, 1, False)
        res["extra"]["decode_c1_ctx128k"] = {"ms_per_step": rl1["dev_ms"], "tok_s": 1e3 / rl1["dev_ms"],
                                             "context_fill": "synthetic random rows in every cache page"}
        eng.sched.retire(eng.requests[ids[0]])
        add_synthetic_requests(eng, conc_extra, long_ctx, headroom, vocab, 13)
        timed_steps(eng, warmup, n_gpus, vocab, conc_extra, False)
        rl64 = timed_repeats(eng, max(8, steps // 4), n_gpus, vocab, conc_extra, False)
        res["extra"]["decode_c64_ctx128k"] = {"ms_per_step": rl64["dev_ms"], "tok_s": conc_extra * 1e3 / rl64["dev_ms"],
                                              "kv_bytes_per_rank": eng.kv.bytes_allocated(),
                                              "context_fill": "synthetic random rows in every cache page"}
        _lib.check_status()
        del eng
        torch.cuda.empty_cache()

    # ================= phase 3: DSpark speculative decoding =================
    if extra and spec:
        res["extra"]["spec"] = run_spec_phase(n_gpus, rank, dev, comm, fused, layers, ctx, warmup, steps)
    res["extra"]["weights_build_s"] = build_s
    if comm is not None:
        res["extra"]["collective_calls"] = dict(comm.calls)
        res["extra"]["symm_disabled_reason"] = comm.disabled_reason
    return res


class ReplayDrafter:
    """Stands in for a trained drafter when the weights are random: proposes the tokens the same engine emitted in an
    earlier pass over the same request (same seeds, same kernels, hence the same text), corrupting position j with
    the probability that gives the published cumulative acceptance.  Only the proposals are replaced on the host;
    the draft block still runs on the device every step.

    The replayed text is only a valid oracle while this pass still emits it: an accepted draft row is computed beside
    other rows than in the recording pass, and one rounding-level flip of a sampled token changes everything after it.
    The drafter therefore checks, at every call, that the request's output is still a prefix of the recording, and
    counts steps and emitted tokens only while it is (`steps_in_sync`, `tokens_in_sync`)."""

    def __init__(self, recorded: Dict[int, List[int]], vocab: int, acceptance=REFERENCE_ACCEPTANCE, seed: int = 0):
        self.rec, self.vocab = recorded, vocab
        self.cond = [acceptance[0]] + [acceptance[j] / acceptance[j - 1] for j in range(1, len(acceptance))]
        self.rng = random.Random(seed)
        self.in_sync: Dict[int, bool] = {}
        self.last_len: Dict[int, int] = {}
        self.steps_in_sync = 0
        self.tokens_in_sync = 0
        self.counting = False

    def __call__(self, req: Request, device_drafts: List[int]) -> List[int]:
        key = req.params.seed
        rec = self.rec.get(key)
        have = len(req.output)
        ok = rec is not None and self.in_sync.get(key, True) and have + len(device_drafts) < len(rec) \
            and list(req.output) == rec[:have]
        if self.counting and key in self.last_len and self.in_sync.get(key, True):
            # the step that just ended was drafted from a valid oracle
            self.steps_in_sync += 1
            self.tokens_in_sync += have - self.last_len[key]
        self.in_sync[key] = ok
        self.last_len[key] = have
        if not ok:
            return list(device_drafts)
        out = []
        for j in range(len(device_drafts)):
            tok = rec[have + j]
            c = self.cond[min(j, len(self.cond) - 1)]
            out.append(tok if self.rng.random() < c else (tok + 1) % self.vocab)
        return out


def run_spec_phase(n_gpus: int, rank: int, dev, comm, fused: bool, layers: int, ctx: int, warmup: int, steps: int,
                   n_spec: int = 5, temperature: float = 0.6) -> Dict:
    from ..spec.dspark import build_draft_weights
    mcfg = flash_config(layers, n_mtp_layers=3, dspark_target_layer_ids=(layers // 4, layers // 2, layers - 1))
    src = RandomSource(0)
    w = build_model_weights(mcfg, src, dev, rank, n_gpus, head_fp8=True)
    dw = build_draft_weights(mcfg, src, w, dev, rank, n_gpus)
    vocab = mcfg.vocab_size
    out: Dict = {"num_speculative_tokens": n_spec, "temperature": temperature,
                 "drafter": "random-init drafter (acceptance at chance) and replay drafter (reference acceptance profile)"}
    k = max(8, steps // 2)
    for conc in (1, 16):
        row: Dict = {}
        # plain decode on the same model (no drafts)
        eng = _engine(mcfg, n_gpus, rank, dev, comm, w, fused, ctx + 4096, max(conc, 2), 256)
        fill_caches_synthetic(eng)
        add_synthetic_requests(eng, conc, ctx, 4000, vocab, 7, temperature)
        timed_steps(eng, warmup, n_gpus, vocab, conc, True)
        rp = timed_repeats(eng, k, n_gpus, vocab, conc, True, min_seconds=0.3)
        row["plain_ms_per_step"] = rp["dev_ms"]
        row["plain_tok_s"] = conc * 1e3 / rp["wall_ms"]
        del eng
        torch.cuda.empty_cache()
        spec_cfg = SpecConfig(method="dspark", num_speculative_tokens=n_spec, markov_topk=512, temperature=temperature)

        def spec_engine():
            e = _engine(mcfg, n_gpus, rank, dev, comm, w, fused, ctx + 4096, max(conc, 2), 256, spec_cfg, dw)
            fill_caches_synthetic(e)
            add_synthetic_requests(e, conc, ctx, 4000, vocab, 7, temperature)
            return e

        # pass 1: the device drafter's own proposals (random weights: accepted at chance); records the emitted text
        eng = spec_engine()
        timed_steps(eng, warmup, n_gpus, vocab, conc, True)
        m0 = (eng.metrics.spec_num_drafts, eng.metrics.spec_num_accepted_tokens)
        rs = timed_repeats(eng, k, n_gpus, vocab, conc, True, min_seconds=0.3)
        drafts = eng.metrics.spec_num_drafts - m0[0]
        row["spec_ms_per_step"] = rs["dev_ms"]
        row["random_drafter_accepted_per_step"] = (eng.metrics.spec_num_accepted_tokens - m0[1]) / max(drafts, 1)
        row["break_even_accepted_tokens"] = rs["dev_ms"] / rp["dev_ms"] - 1.0
        # keep decoding (untimed) until the recorded text is long enough for a replay whose mean acceptance is not noise:
        # 48 drafted steps per request at C=1, 16 at C=16
        want_rep = 48 if conc == 1 else 16
        need = (want_rep + warmup + 2) * (n_spec + 1)
        guard = 0
        while min(len(r.output) for r in eng.requests.values()) < need and guard < 2 * need:
            eng.step()
            guard += 1
        recorded = {r.params.seed: list(r.output) for r in eng.requests.values()}
        del eng
        torch.cuda.empty_cache()
        # pass 2: the same requests again, proposals replayed from pass 1 at the reference's acceptance profile
        eng = spec_engine()
        eng.draft_override = ReplayDrafter(recorded, vocab)
        n_rep = max(8, min(len(v) for v in recorded.values()) // (n_spec + 1) - warmup - 2)
        for _ in range(warmup):
            eng.step()
        eng.draft_override.counting = True
        g0 = eng.metrics.generation_tokens_total
        m0 = (eng.metrics.spec_num_drafts, eng.metrics.spec_num_accepted_tokens, list(eng.metrics.spec_accepted_per_pos))
        _sync(n_gpus)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(n_rep):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        wall = _max_over_ranks(time.perf_counter() - t0, n_gpus, dev)
        toks = eng.metrics.generation_tokens_total - g0
        drafts = eng.metrics.spec_num_drafts - m0[0]
        per = [a - (m0[2][i] if i < len(m0[2]) else 0) for i, a in enumerate(eng.metrics.spec_accepted_per_pos)]
        rd = eng.draft_override
        row["replay_steps"] = n_rep
        row["replay_ms_per_step"] = _max_over_ranks(e0.elapsed_time(e1) / n_rep, n_gpus, dev)
        row["replay_wall_ms_per_step"] = wall * 1e3 / n_rep
        row["replay_accepted_per_step_all_steps"] = (eng.metrics.spec_num_accepted_tokens - m0[1]) / max(drafts, 1)
        row["replay_per_position_acceptance_all_steps"] = [round(a / max(drafts, 1), 4) for a in per]
        # steps drafted from a valid oracle (the request still emitted the recorded text): the acceptance of those
        # steps is the reference's profile; a step costs the same whatever it accepts, so tokens/s over those steps
        # is tokens per step / measured time per step
        row["replay_request_steps_in_sync"] = rd.steps_in_sync
        row["replay_tokens_per_step_in_sync"] = rd.tokens_in_sync / max(rd.steps_in_sync, 1)
        tps = conc * row["replay_tokens_per_step_in_sync"] / (row["replay_wall_ms_per_step"] * 1e-3)
        row["replay_tok_s"] = tps
        row["replay_tok_s_all_steps"] = toks / wall
        row["replay_speedup_vs_plain"] = tps / row["plain_tok_s"]
        _lib.check_status()
        del eng
        torch.cuda.empty_cache()
        out[f"c{conc}"] = row
    return out
