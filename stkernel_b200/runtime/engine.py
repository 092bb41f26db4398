"""The serving engine: continuous batching with chunked prefill over the paged caches.

One `Engine` per rank (one process per GPU).  `step()` schedules decode rows first,
then prefill chunks up to the token budget (the reference's serving mode:
4096-token chunks, decode-first ordering, launchers/start-hy4-tp4.sh:370-391), builds
the per-step metadata on the device, runs the model, samples with seeded Gumbel
noise keyed by (seed, position) and appends the new tokens.  Pure-decode steps
replay a CUDA graph per batch-size bucket.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..config import EngineConfig
from ..models.dsv4 import DSV4Model, ModelWeights, StepMeta
from ..ops import attention as A
from ..ops import sampling as S
from ..ops.cache import PAGE
from .kv import KVManager, OutOfPages, memory_pool_tokens, size_pools
from .metrics import Metrics


class DeviceStatusError(RuntimeError):
    """A kernel of the step recorded a non-zero status (a bounded wait ran out, or an index was out of range)."""

    NAMES = {1: "mbarrier wait timed out", 2: "peer flag wait timed out", 3: "index out of range",
             4: "local flag wait timed out"}

    def __init__(self, code: int, detail: int):
        super().__init__(f"device status {code} ({self.NAMES.get(code, '?')}), detail {detail}")
        self.code, self.detail = code, detail


@dataclass
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0
    max_tokens: int = 16
    min_tokens: int = 0
    ignore_eos: bool = False
    eos_token_id: Optional[int] = None
    top_k: int = 0                  # <= 0: off
    top_p: float = 1.0              # >= 1: off
    logprobs: Optional[int] = None  # report the sampled token's log-probability and this many most likely alternatives

    @property
    def truncates(self) -> bool:
        return self.top_k > 0 or self.top_p < 1.0


@dataclass
class Request:
    req_id: int
    prompt: List[int]
    params: SamplingParams
    row: int = -1
    num_computed: int = 0               # tokens whose KV is in the cache
    output: List[int] = field(default_factory=list)
    finished: bool = False
    arrival: float = field(default_factory=time.time)
    first_token_time: Optional[float] = None
    finish_reason: Optional[str] = None   # "stop" (EOS), "length" (token or context limit), "abort"
    drafts: List[int] = field(default_factory=list)   # proposals awaiting verification (speculative decoding)
    logprobs: List[Tuple[float, List[Tuple[int, float]]]] = field(default_factory=list)   # per output token, when asked for

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def token_span(self, start: int, n: int) -> List[int]:
        """tokens[start:start+n] without concatenating the prompt and the output."""
        lp = len(self.prompt)
        if start >= lp:
            return self.output[start - lp:start - lp + n]
        if start + n <= lp:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.output[:start + n - lp]

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def in_prefill(self) -> bool:
        return self.num_computed < len(self.prompt)


@dataclass
class ScheduledSeq:
    req: Request
    start: int          # first position computed this step
    n: int              # tokens computed this step
    samples: bool       # the last token of this span produces a new token
    n_sample: int = 1   # trailing rows that sample (1 + drafts for a verifying decode row)


class Scheduler:
    """Decode-first continuous batching with chunked prefill and page-aware admission."""

    def __init__(self, cfg: EngineConfig, kv: KVManager, prefix_cache=None):
        self.cfg = cfg
        self.kv = kv
        self.prefix_cache = prefix_cache
        self.waiting: List[Request] = []
        self.running: List[Request] = []

    def add(self, req: Request) -> None:
        self.waiting.append(req)

    def schedule(self) -> List[ScheduledSeq]:
        sc = self.cfg.sched
        budget = sc.max_num_batched_tokens
        out: List[ScheduledSeq] = []
        # 1) decode rows first
        for r in self.running:
            if r.finished or r.in_prefill:
                continue
            if len(r.output) >= r.params.max_tokens or r.total_len >= sc.max_model_len:
                continue             # its last token is still in flight (asynchronous scheduling); nothing more to run
            if budget <= 0:
                break
            k = min(len(r.drafts), budget - 1)
            out.append(ScheduledSeq(r, r.num_computed, 1 + k, True, 1 + k))
            budget -= 1 + k
        # 2) running prefills continue, chunked
        for r in self.running:
            if r.finished or not r.in_prefill or budget <= 0:
                continue
            n = min(budget, len(r.prompt) - r.num_computed)
            out.append(ScheduledSeq(r, r.num_computed, n, r.num_computed + n == len(r.prompt)))
            budget -= n
        # 3) admit waiting requests while rows, pages and budget allow
        while self.waiting and budget > 0 and len(self.running) < sc.max_num_seqs:
            r = self.waiting[0]
            ctx = min(len(r.prompt) + r.params.max_tokens, sc.max_model_len)
            if not self.kv.can_admit(min(budget, len(r.prompt)), ctx):
                if self.prefix_cache is None or not self.prefix_cache.entries:
                    break
                # cached prefixes hold pages too: give them up, oldest first, before refusing a request
                need_swa, need_c4 = self.kv.admit_needs(min(budget, len(r.prompt)), ctx)
                self.prefix_cache.make_room(need_swa, need_c4 + self.kv.promised())
                if not self.kv.can_admit(min(budget, len(r.prompt)), ctx):
                    break
            self.waiting.pop(0)
            r.row = self.kv.alloc_row()
            self.kv.reserve(r.row, ctx)
            self.running.append(r)
            start = 0
            if self.prefix_cache is not None:
                start, entry = self.prefix_cache.match(r.prompt)
                if entry is not None:
                    self.prefix_cache.adopt(r.row, entry)
                    r.num_computed = start
            n = min(budget, len(r.prompt) - start)
            out.append(ScheduledSeq(r, start, n, start + n == len(r.prompt)))
            budget -= n
        return out

    def retire(self, req: Request) -> None:
        req.finished = True
        if req in self.running:
            self.kv.free_row(req.row)
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)

    @property
    def num_running(self) -> int:
        return len(self.running)

    @property
    def num_waiting(self) -> int:
        return len(self.waiting)


class HostStage:
    """One set of pinned staging buffers with numpy views (cheap element writes from Python)."""

    def __init__(self, max_tokens: int, max_reqs: int, pin: bool, max_samples: Optional[int] = None):
        mk = lambda n, dt: torch.zeros(n, dtype=dt, pin_memory=pin)
        self.h_tokens = mk(max_tokens, torch.int64)
        self.h_qstart = mk(max_reqs + 1, torch.int32)
        self.h_rows = mk(max_reqs, torch.int32)
        self.h_start = mk(max_reqs, torch.int32)
        ms = max_samples or max_reqs
        self.h_logit_rows = mk(ms, torch.int64)
        self.h_temp = mk(ms, torch.float32)
        self.h_seed = mk(ms, torch.int64)
        self.h_pos = mk(ms, torch.int64)
        self.h_topk = mk(ms, torch.int32)
        self.h_topp = mk(ms, torch.float32)
        self.n_topk, self.n_topp = self.h_topk.numpy(), self.h_topp.numpy()
        self.n_tokens, self.n_qstart, self.n_rows, self.n_start = (self.h_tokens.numpy(), self.h_qstart.numpy(),
                                                                   self.h_rows.numpy(), self.h_start.numpy())
        self.n_logit_rows, self.n_temp, self.n_seed, self.n_pos = (self.h_logit_rows.numpy(), self.h_temp.numpy(),
                                                                   self.h_seed.numpy(), self.h_pos.numpy())
        self.event = None           # recorded after the uploads that read this set


class StepBuffers:
    """Two pinned host staging sets (the host may prepare step k+1 while the copies of step k are
    still queued) + fixed-address device tensors for the step description."""

    def __init__(self, max_tokens: int, max_reqs: int, device, max_samples: Optional[int] = None):
        pin = torch.device(device).type == "cuda"
        self.stages = [HostStage(max_tokens, max_reqs, pin, max_samples) for _ in range(2)]
        self.parity = 0
        h = self.stages[0]
        dv = lambda x: torch.zeros_like(x, device=device)
        self.d_tokens, self.d_qstart, self.d_rows, self.d_start = dv(h.h_tokens), dv(h.h_qstart), dv(h.h_rows), dv(h.h_start)
        self.d_logit_rows, self.d_temp, self.d_seed, self.d_pos = dv(h.h_logit_rows), dv(h.h_temp), dv(h.h_seed), dv(h.h_pos)
        self.d_topk, self.d_topp = dv(h.h_topk), dv(h.h_topp)
        self.truncating = False         # whether any sampling row of the staged step asks for top-k / top-p
        self.h_out = torch.zeros(3 * (max_samples or max_reqs) + max_reqs, dtype=torch.int64, pin_memory=pin)
        self.cuda = pin

    def next_stage(self) -> HostStage:
        """The staging set for the next step, once no earlier upload still reads it."""
        self.parity ^= 1
        st = self.stages[self.parity]
        if st.event is not None:
            st.event.synchronize()
        return st

    def h2d_bytes(self, t: int, n: int) -> int:
        return t * 8 + (n + 1) * 4 + n * 4 * 2 + n * 8 * 3 + n * 4


class Engine:
    def __init__(self, cfg: EngineConfig, weights: ModelWeights, device, comm=None, tp_rank: int = 0,
                 max_context: Optional[int] = None, draft_weights=None, mask_token_id: int = 0, pipe=None):
        """pipe: a `parallel.pipeline.PipeStage` when this engine is one pipeline stage (its `weights` then hold the
        stage's layers only, `build_model_weights(layer_range=pipe.layer_range(...))`).  Every stage runs the same
        scheduler on the same requests; the last stage samples and the tokens are broadcast."""
        cfg.validate()
        self.cfg = cfg
        self.device = torch.device(device)
        sc = cfg.sched
        ctx = max_context or sc.max_model_len
        # decode context parallel: the ranks of the tensor-parallel group each store 1/dcp of the ratio-4 caches
        dcp = cfg.parallel.dcp_size
        if dcp > 1 and (dcp != cfg.parallel.tp_size or comm is None):
            raise ValueError("dcp_size must be 1 or tp_size (the context-parallel ranks are the tensor-parallel group)")
        pool_tokens = cfg.cache.kv_pool_tokens
        if pool_tokens is None and cfg.cache.size_by_memory and self.device.type == "cuda":
            free, total = torch.cuda.mem_get_info(self.device)
            lo_hi = pipe.layer_range(cfg.model.num_hidden_layers) if pipe is not None else (0, cfg.model.num_hidden_layers)
            pool_tokens = memory_pool_tokens(cfg.model, cfg.cache.gpu_memory_utilization, free, total, ctx,
                                             list(range(*lo_hi)), dcp)
            if comm is not None or pipe is not None:
                # every rank (and every stage) runs the same scheduler: they must agree on the pool, so take the smallest
                import torch.distributed as dist
                seen = [None] * dist.get_world_size()
                dist.all_gather_object(seen, pool_tokens)
                pool_tokens = min(seen)
        pools = size_pools(cfg.model, sc.max_num_seqs, ctx, sc.max_num_batched_tokens, dcp, pool_tokens)
        if cfg.cache.num_pages is not None:
            pools["swa_pages"] = max(pools["swa_pages"], cfg.cache.num_pages)
        has_c128 = any(cfg.model.layer_kind(i) == "c128a" for i in range(cfg.model.num_hidden_layers))
        spec_on = cfg.spec.method == "dspark"
        n_spec = cfg.spec.num_speculative_tokens if spec_on else 0
        if spec_on and draft_weights is None:
            raise ValueError("speculative decoding needs the draft weights")
        # a verify step touches N positions past the accepted prefix and the draft block N more
        self.spec_lookahead = 2 * n_spec + 1 if spec_on else 0
        if pipe is not None:
            if pipe.pp_size != cfg.parallel.pp_size:
                raise ValueError("pipeline stage and ParallelConfig.pp_size disagree")
            if spec_on:
                raise ValueError("speculative decoding is not available across pipeline stages")
            lo, hi = pipe.layer_range(cfg.model.num_hidden_layers)
            if weights.layer_offset != lo or len(weights.layers) != hi - lo:
                raise ValueError(f"stage {pipe.pp_rank} expects layers [{lo}, {hi}), the weights hold "
                                 f"[{weights.layer_offset}, {weights.layer_offset + len(weights.layers)})")
        elif cfg.parallel.pp_size > 1:
            raise ValueError("ParallelConfig.pp_size > 1 needs a PipeStage")
        stage_layers = list(range(*pipe.layer_range(cfg.model.num_hidden_layers))) if pipe is not None else None
        self.kv = KVManager(cfg.model, self.device, sc.max_num_seqs, ctx + 64, pools["swa_pages"] + (sc.max_num_seqs if spec_on else 0),
                            pools["c4_pages"], pools["c128_pages"] if has_c128 else 0, sc.max_num_batched_tokens,
                            layers=stage_layers, extra_swa_layers=cfg.model.n_mtp_layers if spec_on else 0, spec_tokens=n_spec,
                            dcp_rank=tp_rank if dcp > 1 else 0, dcp_size=dcp)
        self.model = DSV4Model(cfg.model, weights, self.kv, comm, tp_rank, cfg.parallel.tp_size)
        self.model.pipe = pipe
        self.prefix_cache = None
        if cfg.cache.enable_prefix_caching:
            from .prefix_cache import PrefixCache
            pc = PrefixCache(self.kv)
            self.prefix_cache = pc if pc.enabled else None
            if self.prefix_cache is not None:
                self.kv.swa.on_pressure = pc.evict_one
                self.kv.c4.on_pressure = pc.evict_one
        self.sched = Scheduler(cfg, self.kv, self.prefix_cache)
        self.buf = StepBuffers(sc.max_num_batched_tokens + sc.max_num_seqs * (1 + n_spec), sc.max_num_seqs, self.device,
                               sc.max_num_seqs * (1 + n_spec))
        self.drafter = None
        if spec_on:
            pin = self.device.type == "cuda"
            self.h_spec_host = torch.zeros(sc.max_num_seqs, 5 + n_spec, dtype=torch.int64, pin_memory=pin)
            self.h_spec_temp = torch.zeros(sc.max_num_seqs, dtype=torch.float32, pin_memory=pin)
            self.d_spec_host = torch.zeros(sc.max_num_seqs, 5 + n_spec, dtype=torch.int64, device=self.device)
            self.d_spec_temp = torch.zeros(sc.max_num_seqs, dtype=torch.float32, device=self.device)
            self._spec_cols = torch.arange(n_spec + 1, device=self.device)
            from ..spec.dspark import DSparkDrafter
            self.model.aux_layers = tuple(cfg.model.dspark_target_layer_ids)
            self.drafter = DSparkDrafter(cfg.model, cfg.spec, draft_weights, self.kv, comm, tp_rank, cfg.parallel.tp_size,
                                         mask_token_id)
        self.weight_source = None            # set by the caller when experts are to be re-placed at run time
        if cfg.parallel.eplb_record or cfg.parallel.eplb_redundant > 0:
            from ..parallel.eplb import LoadRecorder
            self.model.load_recorder = LoadRecorder(cfg.model.num_hidden_layers, cfg.model.n_routed_experts, self.device)
        self.metrics = Metrics()
        self.async_scheduling = sc.async_scheduling and not spec_on and pipe is None
        self._inflight = None                # asynchronous scheduling: the step that is launched and not read yet
        self._async_parity = 0
        self._h_async = ([torch.zeros(sc.max_num_seqs * (1 + n_spec), dtype=torch.int64, pin_memory=True) for _ in range(2)]
                         if self.async_scheduling and self.device.type == "cuda" else [])
        self._feed_parity = 0
        self._h_feed = ([torch.zeros(2, sc.max_num_seqs, dtype=torch.int64, pin_memory=True) for _ in range(2)]
                        if self.async_scheduling and self.device.type == "cuda" else [])
        self._d_feed = (torch.zeros(2, sc.max_num_seqs, dtype=torch.int64, device=self.device)
                        if self.async_scheduling and self.device.type == "cuda" else None)
        self._next_id = 0
        self.requests: Dict[int, Request] = {}
        self._graphs: Dict[tuple, object] = {}
        # a captured step cannot hold the stage-to-stage sends and receives: pipeline stages run eagerly; so do steps
        # under decode context parallelism (their staging buffers are allocated as block sizes first appear)
        self.use_graphs = self.device.type == "cuda" and sc.graph_cap > 0 and pipe is None and dcp == 1
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self._placements: Dict[int, object] = {}
        self._h_status: Optional[torch.Tensor] = None
        self._d_agreed: Optional[torch.Tensor] = None
        # Optional host hook (request, device-drafted tokens) -> tokens to verify next step: benchmarks replace the
        # drafter's proposals by a replayed sequence to exercise the accept path at a chosen acceptance rate (the
        # draft block still runs on the device, so the step cost is the real one).
        self.draft_override = None

    # ---- public API ------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        rid = self._next_id
        self._next_id += 1
        req = Request(rid, list(prompt), params or SamplingParams())
        if len(req.prompt) + req.params.max_tokens > self.cfg.sched.max_model_len + 64:
            raise ValueError("request exceeds max_model_len")
        if req.params.logprobs is not None and not self.supports_logprobs:
            raise ValueError("log-probabilities are not available with speculative decoding, asynchronous scheduling or "
                             "pipeline stages")
        if not self.kv.fits(min(len(req.prompt) + req.params.max_tokens, self.cfg.sched.max_model_len)):
            raise ValueError("request needs more compressed-KV pages than the pool holds")
        self.requests[rid] = req
        self.sched.add(req)
        self.metrics.requests_total += 1
        return rid

    @property
    def supports_logprobs(self) -> bool:
        return self.drafter is None and not self.async_scheduling and self.model.pipe is None

    def has_work(self) -> bool:
        return bool(self.sched.waiting or self.sched.running) or self._inflight is not None

    def abort(self, req_id: int) -> bool:
        """Drop a request between steps (client went away, stop string hit); frees its pages."""
        r = self.requests.get(req_id)
        if r is None or r.finished:
            return False
        r.finish_reason = "abort"
        self.sched.retire(r)
        self.metrics.requests_finished += 1
        return True

    def release(self, req_id: int) -> None:
        """Forget a finished request (the server calls this once the response is out)."""
        r = self.requests.get(req_id)
        if r is not None and r.finished:
            del self.requests[req_id]

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None) -> List[List[int]]:
        ids = [self.add_request(p, params) for p in prompts]
        while self.has_work():
            self.step()
        return [self.requests[i].output for i in ids]

    # ---- device status ---------------------------------------------------------------
    def _agreed_status(self) -> Optional[torch.Tensor]:
        """Under tensor parallelism the sampling exchange carries every rank's status word; the largest lands here, so
        that all ranks fail the same step when any of them saw a wait run out."""
        if self.device.type != "cuda" or self.cfg.parallel.tp_size == 1:
            return None
        if self._d_agreed is None:
            self._d_agreed = torch.zeros(2, dtype=torch.int32, device=self.device)
        return self._d_agreed

    def _queue_status_read(self) -> None:
        """Queue the copy of the kernels' status word behind the step, next to the sampled tokens: the host reads
        both after the one synchronisation the step already has."""
        if self.device.type != "cuda":
            return
        from ..ops import _lib
        if self._h_status is None:
            self._h_status = torch.zeros(4, dtype=torch.int32, pin_memory=True)
        self._h_status[:2].copy_(_lib.status_buffer(), non_blocking=True)
        if self._d_agreed is not None:
            self._h_status[2:].copy_(self._d_agreed, non_blocking=True)

    def _read_status(self) -> Tuple[int, int]:
        """(code, detail) of the step just synchronised; (0, 0) = every bounded wait and index check passed."""
        if self._h_status is None:
            return 0, 0
        code, detail = int(self._h_status[0]), int(self._h_status[1])
        if code == 0 and int(self._h_status[2]) != 0:
            return int(self._h_status[2]), -1          # another rank's code: no detail of our own
        return code, detail

    def _check_device_status(self) -> None:
        """A kernel that gave up a bounded wait (peer flag, mbarrier) or met an out-of-range index skipped its work,
        so this step's tokens are not to be trusted: count it, switch the symmetric-memory collectives off for good
        (later all-reduces take the NCCL path, as overlay/dsv4_oneshot_shim.py:153-162 does after a failed
        heartbeat) and fail the step.  Under lock-step tensor-parallel serving the raising rank ends the job
        (`serve/tp_worker.py`), which the supervisor restarts."""
        code, detail = self._read_status()
        if code == 0:
            return
        self.metrics.device_status_errors += 1
        if self.device.type == "cuda":
            from ..ops import _lib
            _lib.status_buffer().zero_()
        comm = self.model.comm
        symm = getattr(comm, "symm", None) if comm is not None else None
        if symm is not None:
            symm.disable(f"device status {code} (detail {detail}) in step {self.metrics.steps_total}")
        raise DeviceStatusError(code, detail)

    # ---- one step -----------------------------------------------------------------
    def _stage(self, seqs: List[ScheduledSeq]) -> Tuple[int, int, int]:
        """Fill the pinned staging buffers; returns (T, n_req, n_samples)."""
        b = self.buf.next_stage()
        t = 0
        ns = 0
        trunc = False
        for i, s in enumerate(seqs):
            r = s.req
            self.kv.prepare(r.row, s.start, s.n + self.spec_lookahead)
            if s.n_sample > 1:
                b.n_tokens[t:t + s.n] = r.token_span(s.start, 1) + r.drafts[:s.n - 1]
            else:
                b.n_tokens[t:t + s.n] = r.token_span(s.start, s.n)
            b.n_qstart[i] = t
            b.n_rows[i] = r.row
            b.n_start[i] = s.start
            t += s.n
            if s.samples:
                for j in range(s.n - s.n_sample, s.n):
                    b.n_logit_rows[ns] = t - s.n + j
                    b.n_temp[ns] = r.params.temperature
                    b.n_seed[ns] = r.params.seed
                    b.n_pos[ns] = s.start + j + 1    # position of the token being sampled
                    b.n_topk[ns] = r.params.top_k
                    b.n_topp[ns] = r.params.top_p
                    trunc = trunc or r.params.truncates
                    ns += 1
        b.n_qstart[len(seqs)] = t
        self.buf.truncating = trunc
        return t, len(seqs), ns

    def _upload(self, t: int, n: int, ns: int) -> None:
        d = self.buf
        b = d.stages[d.parity]
        nb = True
        d.d_tokens[:t].copy_(b.h_tokens[:t], non_blocking=nb)
        d.d_qstart[:n + 1].copy_(b.h_qstart[:n + 1], non_blocking=nb)
        d.d_rows[:n].copy_(b.h_rows[:n], non_blocking=nb)
        d.d_start[:n].copy_(b.h_start[:n], non_blocking=nb)
        if ns:
            d.d_logit_rows[:ns].copy_(b.h_logit_rows[:ns], non_blocking=nb)
            d.d_temp[:ns].copy_(b.h_temp[:ns], non_blocking=nb)
            d.d_seed[:ns].copy_(b.h_seed[:ns], non_blocking=nb)
            d.d_pos[:ns].copy_(b.h_pos[:ns], non_blocking=nb)
            if d.truncating:
                d.d_topk[:ns].copy_(b.h_topk[:ns], non_blocking=nb)
                d.d_topp[:ns].copy_(b.h_topp[:ns], non_blocking=nb)
        self.kv.sync(d.parity)
        if d.cuda:
            if b.event is None:
                b.event = torch.cuda.Event()
            b.event.record()
        self.h2d_bytes_last = d.h2d_bytes(t, n)

    def _build_meta(self, t_pad: int, n_req: int, max_comp_rows: int, pure_decode: bool = False) -> StepMeta:
        b = self.buf
        cfg = self.cfg.model
        tok_req, positions, first, last, sm = A.token_maps(b.d_qstart, b.d_rows, b.d_start, n_req, t_pad,
                                                           self.kv.swa.table_dev)
        swa_slots, swa_lens = A.swa_indices(positions, tok_req, self.kv.swa.table_dev, cfg.sliding_window)
        return StepMeta(b.d_tokens[:t_pad], tok_req, positions, first, last, sm, swa_slots, swa_lens, max_comp_rows,
                        pure_decode=pure_decode)

    def _run_model(self, t_pad: int, n_req: int, ns: int, max_comp_rows: int, identity_rows: bool = False) -> torch.Tensor:
        """-> sampled tokens [ns] (device).

        identity_rows: token i is the sampling row of request i (a pure-decode step).  The staged row list is then
        not read at all: a padded decode bucket has more rows than the step uploaded, and the entries past them still
        hold an earlier (possibly much larger) step's row numbers."""
        b = self.buf
        meta = self._build_meta(t_pad, n_req, max_comp_rows, pure_decode=identity_rows)
        trunc = b.truncating and not identity_rows
        return self.model.forward_sample(meta, None if identity_rows else b.d_logit_rows[:ns], b.d_temp[:ns], b.d_seed[:ns],
                                         b.d_pos[:ns], b.d_topk[:ns] if trunc else None, b.d_topp[:ns] if trunc else None,
                                         self._agreed_status())

    def step(self, forced: Optional[Sequence[int]] = None) -> List[Tuple[int, int]]:
        """Run one scheduler step.  Returns [(req_id, new_token)] for requests that produced a token.

        `forced` (benchmarking / teacher forcing): use these tokens as the sampled ones and skip the
        device->host read, so consecutive steps queue on the device without a host round trip."""
        if self.drafter is not None:
            return self._step_spec()
        if self.async_scheduling:
            if forced is not None:
                raise ValueError("forced tokens need a step whose tokens are read before the next one is scheduled")
            return self._step_async()
        ticket = self.step_begin()
        return self.step_finish(ticket, forced) if ticket is not None else []

    # ---- asynchronous scheduling ---------------------------------------------------------------------------------
    PENDING = -1                      # placeholder in Request.output for a token that is sampled but not read yet

    def _step_async(self) -> List[Tuple[int, int]]:
        """Begin step k+1, then read step k.  Returns the tokens of step k."""
        prev, self._inflight = self._inflight, None
        if prev is not None:
            # prefill spans that ended on a block boundary: their state is kept before the next step changes it
            self._offer_prefixes(prev[0])

        def feed(seqs: List[ScheduledSeq]) -> None:
            # decode rows whose input token is still on the device: copy it from the previous step's samples
            if prev is None or prev[2] is None:
                return
            where = {id(s.req): k for k, s in enumerate(x for x in prev[0] if x.samples)}
            src: List[int] = []           # sample index in the previous step ...
            dst: List[int] = []           # ... -> token row of the step being begun
            t = 0
            for s in seqs:
                r = s.req
                if s.n == 1 and r.output and r.output[-1] == self.PENDING and s.start == r.total_len - 1:
                    src.append(where[id(r)])
                    dst.append(t)
                t += s.n
            if not src:
                return
            m = len(src)
            if self.device.type == "cuda":
                # the two index lists go up through pinned memory without blocking the host (a pageable copy would wait
                # for the step that is running); the pinned pair alternates, as the copy of the step before may be queued
                host = self._h_feed[self._feed_parity]
                self._feed_parity ^= 1
                host[0, :m] = torch.tensor(dst, dtype=torch.int64)
                host[1, :m] = torch.tensor(src, dtype=torch.int64)
                self._d_feed[0, :m].copy_(host[0, :m], non_blocking=True)        # contiguous rows: plain asynchronous copies
                self._d_feed[1, :m].copy_(host[1, :m], non_blocking=True)
                d_dst, d_src = self._d_feed[0, :m], self._d_feed[1, :m]
            else:
                d_dst, d_src = torch.tensor(dst, dtype=torch.int64), torch.tensor(src, dtype=torch.int64)
            self.buf.d_tokens.index_copy_(0, d_dst, prev[2].index_select(0, d_src))

        nxt = self.step_begin(after_upload=feed)
        if nxt is not None:
            seqs, ns, toks_dev = nxt
            host, ready = None, None
            if toks_dev is not None and self.device.type == "cuda":
                # start this step's device->host copy now, ahead of the kernels of the step after it
                host = self._h_async[self._async_parity]
                self._async_parity ^= 1
                host[:ns].copy_(toks_dev[:ns], non_blocking=True)
                self._queue_status_read()
                ready = torch.cuda.Event()
                ready.record()
            nxt = (seqs, ns, toks_dev, host, ready)
            # provisional bookkeeping, so that the step after this one can be scheduled before this one is read
            for s in seqs:
                s.req.num_computed = s.start + s.n
                if s.samples:
                    s.req.output.append(self.PENDING)
        out = self._finish_async(prev) if prev is not None else []
        self._inflight = nxt
        return out

    def _finish_async(self, ticket) -> List[Tuple[int, int]]:
        seqs, ns, toks_dev, host, ready = ticket
        new_tokens: List[int] = []
        if toks_dev is not None:
            if ready is not None:
                ready.synchronize()                                # this step's copy only, not the step begun since
                new_tokens = host[:ns].tolist()
            else:
                new_tokens = toks_dev[:ns].tolist()
            self.d2h_bytes_last = ns * 8 + 8
            self._check_device_status()
        out: List[Tuple[int, int]] = []
        k = 0
        now = time.time()
        for s in seqs:
            r = s.req
            if s.start < len(r.prompt):
                self.metrics.prompt_tokens_total += s.n
            if not s.samples:
                continue
            tok = new_tokens[k]
            k += 1
            if r.finished:
                continue                                           # ended one step earlier (EOS) or aborted: a surplus row
            n_out = s.start + s.n - len(r.prompt) + 1
            r.output[n_out - 1] = tok                              # the placeholder of this step
            if r.first_token_time is None:
                r.first_token_time = now
                self.metrics.ttft_sum += now - r.arrival
                self.metrics.ttft_count += 1
            self.metrics.generation_tokens_total += 1
            out.append((r.req_id, tok))
            p = r.params
            hit_eos = (p.eos_token_id is not None and tok == p.eos_token_id and not p.ignore_eos and n_out >= p.min_tokens)
            if n_out >= p.max_tokens or hit_eos or len(r.prompt) + n_out >= self.cfg.sched.max_model_len:
                del r.output[n_out:]                               # the placeholder of the step in flight, if any
                r.finish_reason = "stop" if hit_eos else "length"
                self.sched.retire(r)
                self.metrics.requests_finished += 1
        self._refresh_gauges()
        self.metrics.steps_total += 1
        return out

    def step_begin(self, after_upload=None):
        """First half of a step: schedule, stage, upload and queue the model.  Returns a ticket for `step_finish`, or
        None when nothing was scheduled.  A pipeline stage whose model defers the token exchange
        (`parallel.pipeline.MicroBatchPipeline`) can begin another engine's step before this one is finished."""
        seqs = self.sched.schedule()
        if not seqs:
            return None
        t, n_req, ns = self._stage(seqs)
        self._upload(t, n_req, ns)
        if after_upload is not None:
            after_upload(seqs)
        max_end = max(s.start + s.n for s in seqs)
        max_comp_rows = max(1, max_end // 4)
        pure_decode = all(s.n == 1 and s.samples for s in seqs)
        want_lp = max((s.req.params.logprobs for s in seqs if s.samples and s.req.params.logprobs is not None), default=None)
        if ns == 0:
            # prefill chunk that samples nothing: run the body only
            meta = self._build_meta(t, n_req, max_comp_rows)
            self.model.forward_hidden(meta)
            toks_dev = None
        elif want_lp is not None:
            # a step that reports log-probabilities runs outside the captured graphs and gathers whole logit rows
            self.model.want_logprobs, self.model.last_logprobs = want_lp, None
            try:
                toks_dev = self._run_model(t, n_req, ns, max_comp_rows)
            finally:
                self.model.want_logprobs = None
        elif self.use_graphs and pure_decode and n_req <= self.cfg.sched.graph_cap and not self.buf.truncating:
            toks_dev = self._decode_graph(n_req, max_comp_rows).replay()
        else:
            toks_dev = self._run_model(t, n_req, ns, max_comp_rows)
        return seqs, ns, toks_dev

    def step_finish(self, ticket, forced: Optional[Sequence[int]] = None) -> List[Tuple[int, int]]:
        """Second half: read the sampled tokens (after the deferred exchange between pipeline stages, if any) and update
        the requests."""
        seqs, ns, toks_dev = ticket
        if toks_dev is not None and self.model.pipe is not None and self.model.pipe_defer:
            toks_dev = self.model.pipe.broadcast_from_last(toks_dev)
        out: List[Tuple[int, int]] = []
        new_tokens: List[int] = []
        if toks_dev is not None and forced is not None:
            new_tokens = list(forced)[:ns]
            self.d2h_bytes_last = 0
        elif toks_dev is not None:
            if self.device.type == "cuda":
                self.buf.h_out[:ns].copy_(toks_dev[:ns], non_blocking=True)
                self._queue_status_read()
                torch.cuda.current_stream().synchronize()
                new_tokens = self.buf.h_out[:ns].tolist()
            else:
                new_tokens = toks_dev[:ns].tolist()
            self.d2h_bytes_last = ns * 8 + 8
            self._check_device_status()
        lps = None
        if toks_dev is not None and self.model.last_logprobs is not None:
            tok_lp, top_lp, top_ids = (x[:ns].tolist() for x in self.model.last_logprobs)
            self.model.last_logprobs = None
            lps = list(zip(tok_lp, top_lp, top_ids))
        k = 0
        now = time.time()
        for s in seqs:
            r = s.req
            r.num_computed = s.start + s.n
            if s.start < len(r.prompt):
                self.metrics.prompt_tokens_total += s.n
            if s.samples:
                tok = new_tokens[k]
                if lps is not None and r.params.logprobs is not None:
                    lp, vals, ids_ = lps[k]
                    r.logprobs.append((lp, list(zip(ids_, vals))[:r.params.logprobs]))
                k += 1
                r.output.append(tok)
                if r.first_token_time is None:
                    r.first_token_time = now
                    self.metrics.ttft_sum += now - r.arrival
                    self.metrics.ttft_count += 1
                self.metrics.generation_tokens_total += 1
                out.append((r.req_id, tok))
                p = r.params
                hit_eos = (p.eos_token_id is not None and tok == p.eos_token_id and not p.ignore_eos
                           and len(r.output) >= p.min_tokens)
                if len(r.output) >= p.max_tokens or hit_eos or r.total_len >= self.cfg.sched.max_model_len:
                    r.finish_reason = "stop" if hit_eos else "length"
                    self.sched.retire(r)
                    self.metrics.requests_finished += 1
        self._offer_prefixes(seqs)
        self._refresh_gauges()
        self.metrics.steps_total += 1
        return out

    def _refresh_gauges(self) -> None:
        m = self.metrics
        m.num_requests_running = self.sched.num_running
        m.num_requests_waiting = self.sched.num_waiting
        m.kv_cache_usage = self.kv.c4.pages_in_use / max(1, self.kv.c4.num_pages)
        pc = self.prefix_cache
        if pc is not None:
            m.prefix_cache_queries, m.prefix_cache_hits, m.prefix_cache_hit_tokens = pc.queries, pc.hits, pc.hit_tokens

    def _offer_prefixes(self, seqs: List[ScheduledSeq]) -> None:
        """After a step: a prefill span that ended on a block boundary leaves its state to the prefix cache."""
        pc = self.prefix_cache
        if pc is None:
            return
        for s in seqs:
            end = s.start + s.n
            if s.start < len(s.req.prompt) and end <= len(s.req.prompt) and end % pc.block == 0 and not s.req.finished:
                pc.offer(s.req.row, s.req.prompt, end)

    # ---- expert load balancing ---------------------------------------------------------------
    def expert_load(self):
        """Tokens routed to every logical expert of every layer since the last call ([layers, experts], CPU)."""
        rec = self.model.load_recorder
        if rec is None:
            raise RuntimeError("expert load is not being recorded (ParallelConfig.eplb_record / eplb_redundant)")
        return rec.take()

    def rebalance_experts(self, load=None) -> List[float]:
        """Between steps: recompute every layer's expert placement from the recorded (or given) load and rebuild that
        layer's experts from `weight_source`.  All ranks must call it with the same load (the recorded counts are
        identical on every rank: routing is replicated).  Returns the per-layer ratio of the most loaded rank's
        expected tokens after / before; captured decode graphs are dropped (the expert tensors changed)."""
        from ..models.dsv4 import build_experts
        from ..parallel.eplb import Placement, rank_loads, rebalance
        if self.weight_source is None:
            raise RuntimeError("rebalance_experts needs Engine.weight_source")
        if load is None:
            load = self.expert_load()
        par, mc = self.cfg.parallel, self.cfg.model
        gains = []
        for li, lw in enumerate(self.model.w.layers):
            row = [float(x) for x in load[li]]
            old = self._placements.get(li) or Placement(mc.n_routed_experts, par.tp_size, list(range(mc.n_routed_experts)))
            new = rebalance(row, par.eplb_redundant, par.tp_size)
            before, after = max(rank_loads(old, row)), max(rank_loads(new, row))
            gains.append(after / before if before > 0 else 1.0)
            if new.phys_to_logical != old.phys_to_logical:
                lw.experts, lw.eplb = build_experts(mc, self.weight_source, f"layers.{li}", self.device, self.model.tp_rank,
                                                    par.tp_size, new)
                self._placements[li] = new
        self._graphs.clear()
        return gains

    def reset_prefix_cache(self) -> int:
        return self.prefix_cache.reset() if self.prefix_cache is not None else 0

    # ---- speculative step ---------------------------------------------------------------
    def _finish_if_done(self, r: Request, tok: int) -> bool:
        p = r.params
        hit_eos = (p.eos_token_id is not None and tok == p.eos_token_id and not p.ignore_eos
                   and len(r.output) >= p.min_tokens)
        if len(r.output) >= p.max_tokens or hit_eos or r.total_len >= self.cfg.sched.max_model_len:
            r.finish_reason = "stop" if hit_eos else "length"
            self.sched.retire(r)
            self.metrics.requests_finished += 1
            return True
        return False

    def _spec_device(self, t: int, n_req: int, ns: int, nb: int, max_comp_rows: int) -> Optional[torch.Tensor]:
        """Device work of a speculative step over the staged inputs: target forward, context-KV insert, coupled
        verify, next draft block.  Returns [n_acc (nb) | verifier tokens (nb x (1+N)) | new drafts (nb x N)] int64.
        Reads fixed-address buffers only, so a pure-decode step can be captured into a CUDA graph."""
        n_spec = self.drafter.n
        meta = self._build_meta(t, n_req, max_comp_rows)
        X = self.model.forward_hidden(meta)
        aux = self.model.aux_out[0] if len(self.model.aux_out) == 1 else torch.cat(self.model.aux_out, -1)
        self.drafter.insert_context(aux, meta.positions, meta.swa_slot_mapping)
        if nb == 0:
            return None
        b = self.buf
        trunc = b.truncating
        toks = self.model.sample(self.model.head_hidden(X.index_select(0, b.d_logit_rows[:ns])), b.d_temp[:ns], b.d_seed[:ns],
                                 b.d_pos[:ns], b.d_topk[:ns] if trunc else None, b.d_topp[:ns] if trunc else None,
                                 self._agreed_status())
        hd, td = self.d_spec_host[:nb], self.d_spec_temp[:nb]
        idx = (hd[:, 0:1] + self._spec_cols[None, :]).clamp_(max=ns - 1)
        ver = toks[idx]
        n_acc, _ = S.coupled_accept(ver, hd[:, 5:].contiguous())
        anchor = ver.gather(1, n_acc[:, None]).squeeze(1)
        anchor_pos = hd[:, 1] + n_acc + 1
        new_drafts, _ = self.drafter.draft(anchor, anchor_pos, hd[:, 2], td, hd[:, 3])
        return torch.cat([n_acc, ver.reshape(-1), new_drafts.reshape(-1)])

    def _step_spec(self) -> List[Tuple[int, int]]:
        """Target step over [last token, drafts...] rows + prefill chunks, coupled verify, context-KV
        insert for the draft layers, next draft block; one device->host read for all of it."""
        seqs = self.sched.schedule()
        if not seqs:
            return []
        n_spec = self.drafter.n
        t, n_req, ns = self._stage(seqs)
        self._upload(t, n_req, ns)
        max_end = max(s.start + s.n for s in seqs)
        max_comp_rows = max(1, max_end // 4)
        now = time.time()
        out: List[Tuple[int, int]] = []
        samp = [s for s in seqs if s.samples]
        nb = len(samp)
        if nb:
            host, temps = self.h_spec_host, self.h_spec_temp
            row0 = 0
            for i, s in enumerate(samp):
                k = s.n_sample - 1
                host[i, 0], host[i, 1], host[i, 2], host[i, 3] = row0, s.start + s.n - s.n_sample, s.req.row, s.req.params.seed
                host[i, 5:] = -1
                if k:
                    host[i, 5:5 + k] = torch.tensor(s.req.drafts[:k], dtype=torch.int64)
                temps[i] = s.req.params.temperature
                row0 += s.n_sample
            self.d_spec_host[:nb].copy_(host[:nb], non_blocking=True)
            self.d_spec_temp[:nb].copy_(temps[:nb], non_blocking=True)
        full = nb == len(seqs) and all(s.n_sample == 1 + n_spec for s in seqs)
        if self.use_graphs and full and t <= self.cfg.sched.graph_cap and not self.buf.truncating:
            rows_bucket = ((max_comp_rows + 64) // 2048 + 1) * 2048
            key = ("spec", n_req, rows_bucket)
            g = self._graphs.get(key)
            if g is None:
                g = SpecGraph(self, t, n_req, ns, nb, rows_bucket)
                self._graphs[key] = g
            packed = g.replay()
        else:
            packed = self._spec_device(t, n_req, ns, nb, max_comp_rows)
        if nb:
            n_out = packed.numel()
            if self.device.type == "cuda":
                self.buf.h_out[:n_out].copy_(packed, non_blocking=True)
                self._queue_status_read()
                torch.cuda.current_stream().synchronize()
                res = self.buf.h_out[:n_out].tolist()
            else:
                res = packed.tolist()
            self.d2h_bytes_last = n_out * 8 + 8
            self._check_device_status()
            acc_h = res[:nb]
            ver_h = res[nb:nb + nb * (n_spec + 1)]
            dr_h = res[nb + nb * (n_spec + 1):]
        si = 0
        for s in seqs:
            r = s.req
            if s.start < len(r.prompt):
                self.metrics.prompt_tokens_total += min(s.n, len(r.prompt) - s.start)
            if not s.samples:
                r.num_computed = s.start + s.n
                continue
            a = acc_h[si]
            if s.n_sample > 1:
                self.metrics.record_spec(s.n_sample - 1, a)
            base = s.start + s.n - s.n_sample
            for j in range(a + 1):
                tok = ver_h[si * (n_spec + 1) + j]
                r.output.append(tok)
                if r.first_token_time is None:
                    r.first_token_time = now
                    self.metrics.ttft_sum += now - r.arrival
                    self.metrics.ttft_count += 1
                self.metrics.generation_tokens_total += 1
                out.append((r.req_id, tok))
                if self._finish_if_done(r, tok):
                    break
            r.num_computed = base + a + 1
            r.drafts = dr_h[si * n_spec:(si + 1) * n_spec]
            if self.draft_override is not None and not r.finished:
                r.drafts = list(self.draft_override(r, r.drafts))[:n_spec]
            si += 1
        self._offer_prefixes(seqs)
        self._refresh_gauges()
        self.metrics.steps_total += 1
        return out

    # ---- CUDA graphs -----------------------------------------------------------------
    def _decode_graph(self, n_req: int, max_comp_rows: int) -> "DecodeGraph":
        bucket = 1
        while bucket < n_req:
            bucket *= 2
        # compressed-row bound baked into the graph: next multiple of 2048 with 64 rows of headroom,
        # so a sequence crosses into a new graph only every 8192 tokens
        rows_bucket = ((max_comp_rows + 64) // 2048 + 1) * 2048
        key = (bucket, rows_bucket)
        if n_req < bucket:
            # padding rows: empty query ranges => request -1, nothing is read or written for them
            self.buf.d_qstart[n_req + 1:bucket + 1].fill_(n_req)
        g = self._graphs.get(key)
        if g is None:
            g = DecodeGraph(self, bucket, rows_bucket)
            self._graphs[key] = g
        return g


_CAPTURE_STREAMS: Dict[int, "torch.cuda.Stream"] = {}


def _capture_stream(device) -> "torch.cuda.Stream":
    """The stream decode steps are captured on: high priority, so that in the replayed graph the kernels of the
    step's critical chain are scheduled ahead of the side branches (which the model runs on a default-priority
    stream) whenever both have thread blocks waiting for an SM."""
    idx = torch.device(device).index or 0
    if idx not in _CAPTURE_STREAMS:
        _CAPTURE_STREAMS[idx] = torch.cuda.Stream(device, priority=-1)
    return _CAPTURE_STREAMS[idx]


def _after_capture_rendezvous(eng: "Engine") -> None:
    """Capturing a step takes a rank-dependent amount of host time (hundreds of milliseconds for a deep model).  The
    kernels of the first replay poll their peers with a bounded budget, so the ranks meet on the host before any of
    them replays: a rank that is still capturing is not mistaken for a dead one."""
    comm = eng.model.comm
    if comm is not None and getattr(comm, "world_size", 1) > 1 and eng.device.type == "cuda":
        comm.barrier()


class SpecGraph:
    """A captured speculative pure-decode step: every request verifies 1 + N rows and drafts its next block."""

    def __init__(self, eng: "Engine", t: int, n_req: int, ns: int, nb: int, rows_bucket: int):
        from ..ops import _lib
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                eng._spec_device(t, n_req, ns, nb, rows_bucket)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = _lib.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=_capture_stream(eng.device)):
            self.out = eng._spec_device(t, n_req, ns, nb, rows_bucket)
        self.launches_per_replay = _lib.launch_count - before
        _after_capture_rendezvous(eng)

    def replay(self) -> torch.Tensor:
        from ..ops import _lib
        self.graph.replay()
        _lib.launch_count += self.launches_per_replay
        return self.out


class DecodeGraph:
    """A captured pure-decode step for `bucket` rows (token i belongs to request i)."""

    def __init__(self, eng: Engine, bucket: int, rows_bucket: int):
        self.eng = eng
        self.bucket = bucket
        # warm-up outside capture (allocates scratch, configures kernels), then capture
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.out = eng._run_model(bucket, bucket, bucket, rows_bucket, identity_rows=True)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..ops import _lib
        before = _lib.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=_capture_stream(eng.device)):
            self.out = eng._run_model(bucket, bucket, bucket, rows_bucket, identity_rows=True)
        self.launches_per_replay = _lib.launch_count - before
        _after_capture_rendezvous(eng)

    def replay(self) -> torch.Tensor:
        from ..ops import _lib
        self.graph.replay()
        _lib.launch_count += self.launches_per_replay
        return self.out
