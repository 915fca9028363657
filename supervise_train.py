#!/usr/bin/env python
"""supervise_train — keep a training run alive: relaunch it when it exits abnormally or stalls.

Covers the reference's out-of-process failure handling (``scripts/ensure_supervisor.sh``,
``scripts/v2_stall_watchdog.sh``): the child is declared stalled when its log file has not been modified
for ``--stall-seconds`` (default 1800); it is then terminated (its own process group only) and restarted
with ``-y 1`` so that it resumes from the newest ``model_N.bin`` in its output directory.

    python supervise_train.py --log run/log.txt -- python train_gpt2.py -o run -n 200 ...
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time


def with_resume(cmd):
    cmd = list(cmd)
    if "-y" in cmd:
        cmd[cmd.index("-y") + 1] = "1"
        return cmd
    return cmd + ["-y", "1"]


def run_once(cmd, log_path, stall_seconds, poll_seconds):
    """Returns ("exit", code) or ("stall", None)."""
    os.makedirs(os.path.dirname(os.path.abspath(log_path)), exist_ok=True)
    with open(log_path, "ab") as log:
        proc = subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
        while True:
            try:
                return "exit", proc.wait(timeout=poll_seconds)
            except subprocess.TimeoutExpired:
                pass
            age = time.time() - os.path.getmtime(log_path)
            if age > stall_seconds:
                try:
                    os.killpg(proc.pid, signal.SIGTERM)      # exactly the group this supervisor started
                    proc.wait(timeout=30)
                except Exception:
                    try:
                        os.killpg(proc.pid, signal.SIGKILL)
                    except Exception:
                        pass
                    proc.wait()
                return "stall", None


def supervise(cmd, log_path, stall_seconds=1800.0, max_restarts=100, poll_seconds=5.0) -> int:
    restarts = 0
    while True:
        what, code = run_once(cmd, log_path, stall_seconds, poll_seconds)
        if what == "exit" and code == 0:
            return 0
        restarts += 1
        with open(log_path, "a") as log:
            log.write(f"[supervisor] {'stall detected' if what == 'stall' else f'exit code {code}'}; restart {restarts}\n")
        if restarts > max_restarts:
            return 1
        cmd = with_resume(cmd)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--log", required=True)
    ap.add_argument("--stall-seconds", type=float, default=1800.0)
    ap.add_argument("--max-restarts", type=int, default=100)
    ap.add_argument("--poll-seconds", type=float, default=5.0)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd and a.cmd[0] == "--" else a.cmd
    if not cmd:
        ap.error("no command given")
    return supervise(cmd, a.log, a.stall_seconds, a.max_restarts, a.poll_seconds)


if __name__ == "__main__":
    sys.exit(main())
