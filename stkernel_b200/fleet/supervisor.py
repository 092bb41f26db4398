"""Boot-start and crash recovery for the serving stack on one node.

    python -m stkernel_b200.fleet.supervisor [--base http://127.0.0.1:8000] [--once]

A polling state machine with every side effect injected (HTTP, clock, launch, forensics), so the
policy is testable without a server.  Policy (reference: launchers/dsv4-tp4-supervisor.sh:29-153):

* ready = `/v1/models` lists the served model AND a real 4-token chat completes -- the model list
  alone stays 200 when the engine is a corpse; the chat probe outlasts a long-context ingest (300 s);
* adopt an already healthy stack instead of restarting it;
* 3 consecutive failed health checks -> forensics, then relaunch; boot grace 3600 s polled every
  15 s, ended early when the API answers or the process dies;
* wedge watchdog: requests running while `generation_tokens_total` is static for 30 cycles of 30 s
  -> forensics + relaunch (a legitimate long generation always advances the counter);
* once a day, in a chosen hour, when nothing runs or waits on two looks 20 s apart:
  POST /reset_prefix_cache.

GPU settings are read for forensics (`nvidia-smi -q`) and never written.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

from ..runtime.metrics import parse_prometheus


@dataclass
class Policy:
    model: str = "deepseek-v4-flash"
    chat_timeout: float = 300.0
    fails_needed: int = 3
    boot_grace: float = 3600.0
    boot_poll: float = 15.0
    period: float = 30.0
    wedge_cycles: int = 30
    cache_reset_hour: Optional[int] = 4
    idle_recheck: float = 20.0
    forensics_keep: int = 10


class IO:
    """Side effects of the supervisor; tests replace this object."""

    def __init__(self, base: str, launcher: List[str], forensics_dir: str, log_path: Optional[str] = None):
        self.base, self.launcher, self.forensics_dir, self.log_path = base.rstrip("/"), launcher, forensics_dir, log_path
        self.child: Optional[subprocess.Popen] = None

    # -- time ---------------------------------------------------------------------------------
    def now(self) -> float:
        return time.time()

    def sleep(self, s: float) -> None:
        time.sleep(s)

    def localtime(self) -> time.struct_time:
        return time.localtime()

    def log(self, msg: str) -> None:
        print(time.strftime("%F %T"), msg, flush=True)

    # -- HTTP -----------------------------------------------------------------------------------
    def get(self, path: str, timeout: float) -> Optional[str]:
        try:
            with urllib.request.urlopen(self.base + path, timeout=timeout) as r:
                return r.read().decode("utf-8", "replace")
        except (urllib.error.URLError, OSError, ValueError):
            return None

    def post(self, path: str, body: Optional[dict], timeout: float) -> Optional[str]:
        data = json.dumps(body).encode() if body is not None else b""
        req = urllib.request.Request(self.base + path, data=data, method="POST", headers={"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=timeout) as r:
                return r.read().decode("utf-8", "replace")
        except (urllib.error.URLError, OSError, ValueError):
            return None

    # -- process --------------------------------------------------------------------------------
    def start(self) -> bool:
        self.stop()
        out = open(self.log_path, "ab") if self.log_path else subprocess.DEVNULL
        try:
            self.child = subprocess.Popen(self.launcher, stdout=out, stderr=subprocess.STDOUT, start_new_session=True)
        except OSError:
            return False
        return True

    def alive(self) -> bool:
        return self.child is not None and self.child.poll() is None

    def stop(self) -> None:
        """Ends exactly the process group this supervisor started."""
        if self.child is not None and self.child.poll() is None:
            import signal
            try:
                os.killpg(self.child.pid, signal.SIGTERM)
                self.child.wait(timeout=60)
            except (ProcessLookupError, subprocess.TimeoutExpired):
                try:
                    os.killpg(self.child.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
        self.child = None

    def forensics(self, keep: int) -> Optional[str]:
        d = os.path.join(self.forensics_dir, time.strftime("%Y%m%d-%H%M%S"))
        try:
            os.makedirs(d, exist_ok=True)
        except OSError:
            return None
        if self.log_path and os.path.isfile(self.log_path):
            with open(self.log_path, "rb") as f:
                f.seek(max(0, os.path.getsize(self.log_path) - 200_000))
                open(os.path.join(d, "serve-tail.log"), "wb").write(f.read())
        for name, cmd in (("free.txt", ["free", "-m"]), ("nvidia-smi.txt", ["nvidia-smi", "-q"])):
            try:
                out = subprocess.run(cmd, capture_output=True, timeout=30).stdout
                open(os.path.join(d, name), "wb").write(out)
            except (OSError, subprocess.TimeoutExpired):
                pass
        m = self.get("/metrics", 5)
        if m:
            open(os.path.join(d, "metrics.txt"), "w").write(m)
        old = sorted(x for x in os.listdir(self.forensics_dir) if os.path.isdir(os.path.join(self.forensics_dir, x)))
        for x in old[:-keep]:
            shutil.rmtree(os.path.join(self.forensics_dir, x), ignore_errors=True)
        return d


def metric_sum(metrics_text: str, name: str) -> float:
    return sum(v for k, v in parse_prometheus(metrics_text).items() if k.split("{")[0] == name)


@dataclass
class Supervisor:
    io: IO
    policy: Policy = field(default_factory=Policy)
    fails: int = 0
    wedge: int = 0
    gen_last: float = -1.0
    reset_day: str = ""
    launches: int = 0
    events: List[str] = field(default_factory=list)

    def _note(self, msg: str) -> None:
        self.events.append(msg)
        self.io.log(msg)

    # -- probes ---------------------------------------------------------------------------------
    def api_up(self) -> bool:
        body = self.io.get("/v1/models", 5)
        return body is not None and self.policy.model in body

    def chat_ok(self) -> bool:
        body = self.io.post("/v1/chat/completions", {"model": self.policy.model, "max_tokens": 4,
                                                     "messages": [{"role": "user", "content": "ping"}]},
                            self.policy.chat_timeout)
        return body is not None and '"choices"' in body

    def healthy(self) -> bool:
        return self.api_up() and self.chat_ok()

    # -- actions --------------------------------------------------------------------------------
    def launch(self) -> bool:
        self._note("launching serving stack")
        self.io.forensics(self.policy.forensics_keep)
        self.fails = 0
        self.launches += 1
        if not self.io.start():
            self._note("launcher failed to start")
            return False
        waited = 0.0
        while waited < self.policy.boot_grace:
            if self.api_up():
                self._note(f"API up after {int(waited)}s")
                return True
            if not self.io.alive():
                self._note("serving process died during boot")
                return False
            self.io.sleep(self.policy.boot_poll)
            waited += self.policy.boot_poll
        self._note(f"boot grace exceeded ({int(self.policy.boot_grace)}s)")
        return False

    def wedge_check(self) -> bool:
        """True when a wedge was detected and the stack recycled."""
        m = self.io.get("/metrics", 5)
        if m is None:
            self.wedge = 0
            return False
        running = metric_sum(m, "vllm:num_requests_running")
        gen = metric_sum(m, "vllm:generation_tokens_total")
        if running > 0 and gen == self.gen_last:
            self.wedge += 1
            if self.wedge >= self.policy.wedge_cycles:
                self._note(f"WEDGE: {int(running)} request(s) running, generation static for "
                           f"{int(self.policy.wedge_cycles * self.policy.period)}s - recycling")
                if not self.launch():
                    self._note("wedge relaunch failed; health loop will retry")
                self.wedge, self.gen_last = 0, -1.0
                return True
        else:
            self.wedge = 0
        self.gen_last = gen
        return False

    def _idle(self) -> bool:
        m = self.io.get("/metrics", 5)
        if m is None:
            return False
        return metric_sum(m, "vllm:num_requests_running") + metric_sum(m, "vllm:num_requests_waiting") == 0

    def maybe_cache_reset(self) -> bool:
        if self.policy.cache_reset_hour is None:
            return False
        lt = self.io.localtime()
        day = time.strftime("%Y%m%d", lt)
        if lt.tm_hour != self.policy.cache_reset_hour or self.reset_day == day:
            return False
        if not self._idle():
            return False
        self.io.sleep(self.policy.idle_recheck)
        if not self._idle():
            return False
        if self.io.post("/reset_prefix_cache", None, 15) is not None:
            self.reset_day = day
            self._note("daily idle prefix-cache reset done")
            return True
        return False

    # -- loop -----------------------------------------------------------------------------------
    def start(self) -> None:
        self._note("=== supervisor start ===")
        if self.healthy():
            self._note("existing stack healthy - adopting")
        elif not self.launch():
            self._note("initial launch failed; will retry via health loop")

    def tick(self) -> None:
        """One health-loop cycle (the caller sleeps `policy.period` between ticks)."""
        if self.healthy():
            if self.fails:
                self._note("recovered (fails reset)")
            self.fails = 0
            self.wedge_check()
            self.maybe_cache_reset()
            return
        self.fails += 1
        self._note(f"health check failed ({self.fails}/{self.policy.fails_needed})")
        if self.fails >= self.policy.fails_needed:
            if not self.launch():
                self._note("relaunch failed; retrying next cycle")

    def run(self, cycles: Optional[int] = None) -> None:
        self.start()
        n = 0
        while cycles is None or n < cycles:
            self.io.sleep(self.policy.period)
            self.tick()
            n += 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="deepseek-v4-flash")
    ap.add_argument("--forensics-dir", default=os.path.expanduser("~/stk-forensics"))
    ap.add_argument("--log", default=os.path.expanduser("~/stk-serve.log"))
    ap.add_argument("--cycles", type=int, default=None)
    ap.add_argument("--cache-reset-hour", default="4", help="local hour of the daily idle reset; empty disables")
    a = ap.parse_args(argv)
    io = IO(a.base, [sys.executable, "-m", "stkernel_b200.fleet.launcher"], a.forensics_dir, a.log)
    pol = Policy(model=a.model, cache_reset_hour=int(a.cache_reset_hour) if a.cache_reset_hour else None,
                 wedge_cycles=int(os.environ.get("WEDGE_CYCLES", "30")))
    sup = Supervisor(io, pol)
    try:
        sup.run(a.cycles)
    finally:
        io.stop()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
