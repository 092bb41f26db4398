"""Watch an upstream tag feed for new, re-pushed and removed tags.

    python -m stkernel_b200.fleet.release_watch --state FILE [--slug org/repo] [--flag-file F] [--webhook URL]

The first run seeds the state file; later runs diff {tag: digest} against it, rewrite the state
atomically, append a report to the flag file, POST it to the webhook when one is set, and exit 10 when
something changed (0 when not) so a timer unit can chain an action (reference:
launchers/watch-image-tags.sh:29-142 and its systemd timer).  The fetcher is injectable: the network
call is one function, everything else is pure.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import urllib.request
from typing import Callable, Dict, List, Optional, Tuple

Tags = Dict[str, Tuple[str, str]]          # name -> (digest, last_updated)
EXIT_CHANGED = 10


def fetch_docker_hub(slug: str, opener=urllib.request.urlopen) -> Tags:
    url: Optional[str] = f"https://hub.docker.com/v2/repositories/{slug}/tags/?page_size=100"
    out: Tags = {}
    while url:
        with opener(url, timeout=30) as resp:
            data = json.load(resp)
        for t in data.get("results", []):
            name = t.get("name") or ""
            if name:
                out[name] = (t.get("digest") or "", (t.get("last_updated") or "")[:19])
        url = data.get("next")
    return out


def fetch_with_retry(fetch: Callable[[], Tags], sleep=time.sleep) -> Tags:
    try:
        tags = fetch()
    except Exception as e:                                     # one retry, then a hard failure
        print(f"WARN: fetch failed ({e}); retrying once in 10s", file=sys.stderr)
        sleep(10)
        tags = fetch()
    if not tags:
        raise RuntimeError("empty tag list")
    return tags


def load_state(path: str) -> Tags:
    out: Tags = {}
    with open(path, encoding="utf-8") as f:
        for line in f:
            p = line.rstrip("\n").split("\t")
            if p and p[0]:
                out[p[0]] = (p[1] if len(p) > 1 else "", p[2] if len(p) > 2 else "")
    return out


def dump_state(path: str, tags: Tags) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "w", encoding="utf-8") as f:
        for name in sorted(tags):
            f.write(f"{name}\t{tags[name][0]}\t{tags[name][1]}\n")
    os.replace(tmp, path)


def diff(old: Tags, new: Tags) -> List[str]:
    out = []
    for name in sorted(new):
        digest, updated = new[name]
        if name not in old:
            out.append(f"NEW TAG   {name}  {digest}  {updated}")
        elif old[name][0] != digest:
            out.append(f"REPUSHED  {name}  {old[name][0]} -> {digest}  {updated}")
    out += [f"REMOVED   {name}" for name in sorted(set(old) - set(new))]
    return out


def run_once(state: str, fetch: Callable[[], Tags], slug: str = "", flag_file: str = "", webhook: str = "",
             post: Optional[Callable[[str, bytes], None]] = None) -> int:
    tags = fetch_with_retry(fetch)
    if not os.path.exists(state):
        dump_state(state, tags)
        print(f"initialized state with {len(tags)} tags ({state})")
        return 0
    changes = diff(load_state(state), tags)
    dump_state(state, tags)
    if not changes:
        print(f"no change ({slug})")
        return 0
    report = f"[{time.strftime('%Y-%m-%dT%H:%M:%SZ', time.gmtime())}] {slug} feed changed:\n" + "\n".join(changes)
    print(report)
    if flag_file:
        try:
            os.makedirs(os.path.dirname(os.path.abspath(flag_file)), exist_ok=True)
            with open(flag_file, "a", encoding="utf-8") as f:
                f.write(report + "\n\n")
        except OSError as e:
            print(f"WARN: could not append flag file {flag_file}: {e}", file=sys.stderr)
    if webhook:
        body = json.dumps({"text": "release watch:\n" + "\n".join(changes)}).encode()
        try:
            if post is not None:
                post(webhook, body)
            else:
                urllib.request.urlopen(urllib.request.Request(webhook, data=body, headers={"Content-Type": "application/json"}),
                                       timeout=15).read()
        except Exception as e:
            print(f"WARN: webhook POST failed: {e}", file=sys.stderr)
    return EXIT_CHANGED


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--slug", default=os.environ.get("REPO_SLUG", "deepseek-ai/deepseek-v4-flash"))
    ap.add_argument("--state", required=True)
    ap.add_argument("--flag-file", default=os.environ.get("FLAG_FILE", ""))
    ap.add_argument("--webhook", default=os.environ.get("WEBHOOK_URL", ""))
    a = ap.parse_args(argv)
    try:
        return run_once(a.state, lambda: fetch_docker_hub(a.slug), a.slug, a.flag_file, a.webhook)
    except Exception as e:
        print(f"ERROR: fetch failed for {a.slug}: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    raise SystemExit(main())
