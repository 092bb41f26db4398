"""Fleet tooling: fail-closed knobs (exit 2 before anything starts), manifest invariants, supervisor
policy against fake I/O, release watcher, host-audit parsers, guard audit, deploy gates."""
import json
import os
import subprocess
import sys
import time

import pytest

from stkernel_b200.fleet import audit_guards, deploy, fabric, host_audit, launcher, release_watch
from stkernel_b200.fleet import manifest as M
from stkernel_b200.fleet.knobs import KnobError, parse_knobs
from stkernel_b200.fleet.supervisor import IO, Policy, Supervisor, metric_sum

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---- knobs ---------------------------------------------------------------------------------
@pytest.mark.parametrize("env,needle", [
    ({"FP8HEAD": "2"}, "FP8HEAD must be 0 or 1"),
    ({"REFINE": "yes"}, "REFINE must be 0 or 1"),
    ({"MARKOV_TOPK": "-1"}, "MARKOV_TOPK must be 0 or an integer"),
    ({"MARKOV_TOPK": "129281"}, "exceeds model vocab"),
    ({"MARKOV_TOPK": "0512"}, "MARKOV_TOPK must be 0 or an integer"),
    ({"MARKOV_TOPK": "9999999"}, "MARKOV_TOPK must be 0 or an integer"),
    ({"MARKOV_SIDELOAD": "/etc/passwd"}, "must be an absolute path under /models"),
    ({"MARKOV_SIDELOAD": "/models/../etc/x.pt"}, "unsafe character"),
    ({"MARKOV_SIDELOAD": "/models/a b.pt"}, "unsafe character"),
    ({"TP_SIZE": "3"}, "TP_SIZE must be 1, 2, 4 or 8"),
    ({"GPU_MEM": "1.5"}, "GPU_MEM must be a number"),
    ({"SPEC_TOKENS": "0", "REFINE": "1"}, "require speculative decoding"),
    ({"SPEC_TOKENS": "1", "REFINE": "1"}, "SPEC_TOKENS >= 2"),
    ({"ONESHOT": "0", "FUSED": "1"}, "needs the symmetric-memory path"),
    ({"MAX_NUM_SEQS": "64", "MAX_NUM_BATCHED": "128"}, "MAX_NUM_BATCHED must hold"),
    ({"EFFORT": "extreme"}, "EFFORT must be one of"),
    ({"TEMP": "hot"}, "TEMP must be a number"),
    ({"DCP": "1", "TP_SIZE": "1", "SPEC_TOKENS": "0"}, "TP_SIZE >= 2"),
    ({"PP_SIZE": "2"}, "TP_SIZE x PP_SIZE must fit"),
    ({"ASYNC_SCHED": "1"}, "ASYNC_SCHED=1 is not available with speculative decoding"),
    ({"PP_SIZE": "2", "TP_SIZE": "4"}, "not available with speculative decoding"),
])
def test_launcher_fails_closed_with_exit_2(env, needle):
    """Run the real entry point in a child process: a bad knob ends it with exit code 2 and an ABORT
    line, before attestation, preflight or any launch."""
    e = {k: v for k, v in os.environ.items() if not k.isupper() or k in ("PATH", "HOME", "PYTHONPATH", "VIRTUAL_ENV")}
    e.update(env)
    e["PYTHONPATH"] = ROOT
    p = subprocess.run([sys.executable, "-m", "stkernel_b200.fleet.launcher", "--dry-run", "--no-attest"], env=e,
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 2, (p.returncode, p.stdout, p.stderr)
    assert p.stdout.startswith("ABORT:") and needle in p.stdout


def test_good_knobs_dry_run_and_command():
    k = parse_knobs({"TP_SIZE": "8", "MODEL_PATH": "/models/DeepSeek-V4-Flash", "MARKOV_TOPK": "512", "EFFORT": "high"})
    assert k.tp_size == 8 and k.spec_tokens == 5 and k.markov_topk == 512
    cmd = launcher.serve_command(k, python="python")
    assert "--nproc-per-node=8" in cmd and "127.0.0.1" in cmd and "stkernel_b200.serve.tp_worker" in cmd
    spec = json.loads(cmd[cmd.index("--speculative-config") + 1])
    assert spec == {"method": "dspark", "num_speculative_tokens": 5, "draft_sample_method": "probabilistic", "markov_topk": 512}
    env = k.to_env()
    assert env["STK_DRAFT_TOPK"] == "512" and env["MASTER_ADDR"] == "127.0.0.1"
    assert launcher.main(["--dry-run", "--no-attest"], env={"MODEL_PATH": "/models/x"}) == 0
    k2 = parse_knobs({"MAX_NUM_SEQS": "64", "MAX_NUM_BATCHED": "4096"})
    assert k2.warnings and "outside CUDA graphs" in k2.warnings[0]
    k3 = parse_knobs({"DCP": "1", "TP_SIZE": "4"})
    c3 = launcher.serve_command(k3, python="python")
    assert c3[c3.index("--decode-context-parallel-size") + 1] == "4" and "--speculative-config" in c3
    assert any("without CUDA graphs" in w for w in k3.warnings)
    assert "--decode-context-parallel-size" not in cmd and "--pipeline-parallel-size" not in cmd
    assert "--async-scheduling" in launcher.serve_command(parse_knobs({"ASYNC_SCHED": "1", "SPEC_TOKENS": "0"}), python="python")
    assert "--async-scheduling" not in cmd
    k4 = parse_knobs({"PP_SIZE": "2", "TP_SIZE": "4", "SPEC_TOKENS": "0"})
    c4 = launcher.serve_command(k4, python="python")
    assert "--nproc-per-node=8" in c4 and c4[c4.index("--pipeline-parallel-size") + 1] == "2" and "--pipeline-micro-batches" in c4
    assert c4[c4.index("--tensor-parallel-size") + 1] == "4"
    assert any("only 4 GPU" in p for p in launcher.preflight(parse_knobs({"MODEL_PATH": "/models/x", "PP_SIZE": "2", "TP_SIZE": "4",
                                                                          "SPEC_TOKENS": "0"}), gpu_count=4))
    assert "MODEL_PATH is not set" in launcher.preflight(parse_knobs({}), gpu_count=8)
    assert any("only 2 GPU" in p for p in launcher.preflight(parse_knobs({"MODEL_PATH": "/models/x"}), gpu_count=2))


# ---- manifest ------------------------------------------------------------------------------
def test_manifest_roundtrip_and_invariants(tmp_path):
    entries = M.collect(ROOT)
    paths = [e.path for e in entries]
    assert all(p in paths for p in M.PINNED) and len(set(paths)) == len(paths)
    text = M.dumps(entries)
    back = M.parse(text)
    assert back == entries
    n, problems = M.verify(ROOT, back, require_lib=False)
    assert n == len(entries) and problems == []
    assert M.unlisted(ROOT, back) == []
    good = "\n".join(f"{p}\tpy\t{'a' * 64}" for p in M.PINNED)
    M.parse(good)
    for bad, needle in [
        (good + "\nstkernel_b200/x.py\tpy", "malformed"),
        (good + "\nstkernel_b200/x.py\tpy\t" + "a" * 64 + "\textra", "malformed"),
        (good + "\n../etc/passwd\tpy\t" + "a" * 64, "unsafe path"),
        (good + "\n/abs/x.py\tpy\t" + "a" * 64, "unsafe path"),
        (good + "\nother/x.py\tpy\t" + "a" * 64, "outside"),
        (good + "\nstkernel_b200/x y.py\tpy\t" + "a" * 64, "unsafe path"),
        (good + "\nstkernel_b200/x.py\texe\t" + "a" * 64, "unknown kind"),
        (good + "\nstkernel_b200/x.py\tpy\tABC", "invalid sha256"),
        (good + "\n" + good.splitlines()[0], "duplicate"),
        ("# only a comment\n", "empty"),
        (f"stkernel_b200/x.py\tpy\t{'a' * 64}", "pinned files missing"),
    ]:
        with pytest.raises(M.ManifestError, match=needle):
            M.parse(bad)


def test_attestation_detects_skew(tmp_path):
    root = tmp_path / "tree"
    (root / "stkernel_b200" / "fleet").mkdir(parents=True)
    for p in M.PINNED:
        f = root / p
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_text("x = 1\n")
    entries = M.collect(str(root))
    man = root / "stkernel_b200" / "fleet" / M.MANIFEST_NAME
    man.write_text(M.dumps(entries))
    n, problems = M.verify(str(root), entries, require_lib=False)
    assert problems == []
    with pytest.raises(M.ManifestError, match="no built library"):
        launcher.attest(str(root), str(man))
    (root / "stkernel_b200" / "_lib").mkdir()
    (root / "stkernel_b200" / "_lib" / "libstk_b200.so").write_bytes(b"\x7fELF")
    man.write_text(M.dumps(M.collect(str(root))))
    fp = launcher.attest(str(root), str(man))
    assert len(fp) == 64
    (root / M.PINNED[0]).write_text("x = 2\n")                       # byte skew
    with pytest.raises(M.ManifestError, match="byte skew"):
        launcher.attest(str(root), str(man))
    (root / M.PINNED[0]).write_text("x = 1\n")
    (root / "stkernel_b200" / "sneaky.py").write_text("pass\n")      # list skew
    with pytest.raises(M.ManifestError, match="unlisted file"):
        launcher.attest(str(root), str(man))
    with pytest.raises(M.ManifestError, match="manifest missing"):
        launcher.attest(str(root), str(root / "nope.tsv"))
    # deploy copies and re-verifies
    os.remove(root / "stkernel_b200" / "sneaky.py")
    ents = M.collect(str(root))
    assert deploy.install(str(root), ents, str(tmp_path / "dest")) == M.fingerprint(ents)


# ---- supervisor ----------------------------------------------------------------------------
class FakeIO:
    def __init__(self):
        self.t = 0.0
        self.up = False
        self.chat = True
        self.proc_alive = True
        self.boot_after = 45.0
        self.started_at = None
        self.running, self.waiting, self.gen = 0, 0, 0.0
        self.resets = 0
        self.forensic_calls = 0
        self.starts = 0
        self.hour = 12
        self.logs = []

    def now(self): return self.t
    def sleep(self, s):
        self.t += s
        if self.started_at is not None and self.t - self.started_at >= self.boot_after and self.proc_alive:
            self.up = True
    def localtime(self): return time.struct_time((2026, 8, 12, self.hour, 0, 0, 2, 224, 0))
    def log(self, m): self.logs.append(m)
    def get(self, path, timeout):
        if path == "/v1/models":
            return '{"data":[{"id":"deepseek-v4-flash"}]}' if self.up else None
        if path == "/metrics":
            if not self.up:
                return None
            return (f'vllm:num_requests_running{{model_name="m"}} {self.running}\n'
                    f'vllm:num_requests_waiting{{model_name="m"}} {self.waiting}\n'
                    f'vllm:generation_tokens_total{{model_name="m"}} {self.gen}\n')
        return None
    def post(self, path, body, timeout):
        if path == "/v1/chat/completions":
            return '{"choices":[{}]}' if (self.up and self.chat) else None
        if path == "/reset_prefix_cache":
            self.resets += 1
            return "{}"
        return None
    def start(self):
        self.starts += 1
        self.up = False
        self.started_at = self.t
        return True
    def alive(self): return self.proc_alive
    def stop(self): pass
    def forensics(self, keep):
        self.forensic_calls += 1
        return "/tmp/f"


def test_supervisor_adopts_healthy_stack():
    io = FakeIO(); io.up = True
    s = Supervisor(io, Policy())
    s.start()
    assert io.starts == 0 and "adopting" in " ".join(s.events)


def test_supervisor_boots_and_relaunches_after_three_failures():
    io = FakeIO()
    s = Supervisor(io, Policy())
    s.start()
    assert io.starts == 1 and io.up and any("API up after 45s" in e for e in s.events)
    io.chat = False                              # model list still answers: a corpse
    s.tick(); s.tick()
    assert s.fails == 2 and io.starts == 1
    io.chat = True
    s.tick()
    assert s.fails == 0 and any("recovered" in e for e in s.events)
    io.chat = False
    s.tick(); s.tick()
    io.chat = True                               # the relaunch on the third failure boots a healthy stack
    io.chat = False
    s.tick()
    assert io.starts == 2 and io.forensic_calls >= 2


def test_supervisor_boot_grace_and_dead_process():
    io = FakeIO(); io.boot_after = 10 ** 9
    s = Supervisor(io, Policy(boot_grace=60, boot_poll=15))
    assert s.launch() is False and any("boot grace exceeded" in e for e in s.events)
    io2 = FakeIO(); io2.proc_alive = False
    s2 = Supervisor(io2, Policy())
    assert s2.launch() is False and any("died during boot" in e for e in s2.events)


def test_wedge_watchdog_and_cache_reset():
    io = FakeIO(); io.up = True; io.running = 2; io.gen = 100.0
    s = Supervisor(io, Policy(wedge_cycles=3, cache_reset_hour=4))
    assert s.wedge_check() is False               # first look records the counter
    io.gen = 150.0
    assert s.wedge_check() is False and s.wedge == 0      # progress resets the count
    assert s.wedge_check() is False and s.wedge == 1
    assert s.wedge_check() is False and s.wedge == 2
    assert s.wedge_check() is True and io.starts == 1     # static for 3 cycles with requests running
    io.running = 0
    for _ in range(5):
        assert s.wedge_check() is False           # idle engine with a static counter is not a wedge
    # daily reset: only in the chosen hour, only when idle twice, once per day
    io.hour = 12
    assert s.maybe_cache_reset() is False
    io.hour = 4; io.running = 1
    assert s.maybe_cache_reset() is False and io.resets == 0
    io.running = 0
    assert s.maybe_cache_reset() is True and io.resets == 1
    assert s.maybe_cache_reset() is False and io.resets == 1
    assert metric_sum('a{x="1"} 2\na{x="2"} 3\nb 9\n', "a") == 5


# ---- release watch ---------------------------------------------------------------------------
def test_release_watch_diff_and_state(tmp_path):
    state = str(tmp_path / "s" / "tags.tsv")
    flag = str(tmp_path / "flag.txt")
    tags = {"v1": ("sha256:a", "2026-08-01T00:00:00"), "v2": ("sha256:b", "2026-08-02T00:00:00")}
    assert release_watch.run_once(state, lambda: dict(tags), "org/repo", flag) == 0          # seeds
    assert release_watch.run_once(state, lambda: dict(tags), "org/repo", flag) == 0          # no change
    tags2 = {"v2": ("sha256:c", "2026-08-03T00:00:00"), "v3": ("sha256:d", "2026-08-03T00:00:00")}
    posted = []
    rc = release_watch.run_once(state, lambda: dict(tags2), "org/repo", flag, "http://hook", post=lambda u, b: posted.append((u, b)))
    assert rc == release_watch.EXIT_CHANGED
    rep = open(flag).read()
    assert "NEW TAG   v3" in rep and "REPUSHED  v2  sha256:b -> sha256:c" in rep and "REMOVED   v1" in rep
    assert posted and b"NEW TAG" in posted[0][1]
    assert release_watch.load_state(state) == tags2
    calls = {"n": 0}
    def flaky():
        calls["n"] += 1
        if calls["n"] == 1:
            raise OSError("net down")
        return dict(tags2)
    assert release_watch.fetch_with_retry(flaky, sleep=lambda s: None) == tags2
    with pytest.raises(RuntimeError):
        release_watch.fetch_with_retry(lambda: {}, sleep=lambda s: None)

    class Resp:
        def __init__(self, d): self.d = d
        def __enter__(self): return self
        def __exit__(self, *a): return False
        def read(self): return json.dumps(self.d).encode()
    pages = {"https://hub.docker.com/v2/repositories/o/r/tags/?page_size=100": {"results": [{"name": "a", "digest": "d1", "last_updated": "2026-01-01T00:00:00.123Z"}], "next": "p2"},
             "p2": {"results": [{"name": "b", "digest": "d2"}], "next": None}}
    got = release_watch.fetch_docker_hub("o/r", opener=lambda url, timeout: Resp(pages[url]))
    assert got == {"a": ("d1", "2026-01-01T00:00:00"), "b": ("d2", "")}


# ---- host audit / fabric ------------------------------------------------------------------------
NVLINK_OK = "\n".join([f"GPU {g}: NVIDIA B200 (UUID: x)\n" + "\n".join(f"\t Link {i}: 50 GB/s" for i in range(18)) for g in range(2)])


def test_host_audit_parsers_and_findings():
    files = {"/sys/kernel/mm/transparent_hugepage/enabled": "always [madvise] never",
             "/sys/kernel/mm/transparent_hugepage/defrag": "[always] defer madvise never",
             "/proc/sys/vm/compaction_proactiveness": "20\n",
             "/proc/buddyinfo": "Node 0, zone   Normal   1 2 3 4 5 6 7 8 9 10 11\n"}
    mem = host_audit.memory_policy(files.get)
    assert mem == {"thp_enabled": "madvise", "thp_defrag": "always", "compaction_proactiveness": "20", "buddy_order10_free": "11"}
    smi = ("0, NVIDIA B200, 1965, 1965, 40, 300.1, 1000.0, Enabled, Enabled, 0x0000000000000000, 12\n"
           "1, NVIDIA B200, 1200, 1965, 85, 990.0, 1000.0, Enabled, Enabled, 0x0000000000000004, 90000\n")
    degraded = NVLINK_OK.replace("GPU 1: NVIDIA B200 (UUID: x)\n\t Link 0: 50 GB/s\n", "GPU 1: NVIDIA B200 (UUID: x)\n")
    def run(cmd):
        return smi if "--query-gpu" in " ".join(cmd) else degraded
    gpus = host_audit.gpu_state(run)
    assert len(gpus) == 2 and gpus[1]["clocks.sm"] == "1200"
    links = host_audit.nvlink_state(run)
    assert links[0] == {"links_up": 18, "min_gbs": 50.0} and links[1]["links_up"] == 17
    f = host_audit.findings(mem, gpus, links, [[True, False], [True, True]])
    text = "\n".join(f)
    assert "THP defrag=always" in text and "GPU 1: clock event reasons active" in text
    assert "GPU 1: 17/18 NVLink links up" in text and "GPU 0 cannot access GPU 1" in text and "90000 MiB already in use" in text
    assert fabric.check(2, lambda cmd: NVLINK_OK, [[True, True], [True, True]]) == []
    assert fabric.check(2, lambda cmd: degraded, None) == ["GPU 1: 17/18 links up"]
    assert fabric.check(1, lambda cmd: "", None) == ["GPU 0: no NVLink status reported"]


# ---- guard audit / deploy gates -----------------------------------------------------------------
def test_guard_audit_passes_on_tree_and_self_test():
    assert audit_guards.self_test() == 0
    res = audit_guards.evaluate(audit_guards.read_sources(ROOT))
    assert audit_guards.exit_code(res) == 0, [r for r in res if r.status != "PASS"]
    assert audit_guards.exit_code(audit_guards.evaluate({})) == 2
    src = audit_guards.read_sources(ROOT)
    broken = dict(src)
    broken[audit_guards.KVCACHE] = {"path": "x", "text": src[audit_guards.KVCACHE]["text"].replace("slot >= num_slots", "false")
                                    .replace("slot >= a.num_slots", "false")}
    assert audit_guards.exit_code(audit_guards.evaluate(broken)) == 1
    assert audit_guards.main(["--self-test"]) == 0


def test_deploy_gates():
    assert deploy.gate_compile(ROOT) == []
    assert deploy.gate_audit(ROOT) is None
