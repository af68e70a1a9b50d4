import json
import os
import socket
import subprocess
import sys
import time


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(task: str, world: int, workdir: str, device: str = "cpu", timeout: int = 300):
    """Launch ``world`` worker processes, wait, and return their result dicts."""
    port = free_port()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dist_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, task, str(r), str(world), str(port), workdir, device],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT) for r in range(world)]
    outs = [""] * world
    deadline = time.monotonic() + timeout
    timed_out = False
    try:
        for r, p in enumerate(procs):
            try:
                out, _ = p.communicate(timeout=max(1.0, deadline - time.monotonic()))
            except subprocess.TimeoutExpired:
                timed_out = True
                p.kill()
                out, _ = p.communicate()
            outs[r] = out.decode(errors="replace")
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    failed = [r for r, p in enumerate(procs) if p.returncode != 0]
    if failed or timed_out:
        report = "\n".join(f"--- rank {r} (exit {procs[r].returncode}) ---\n{outs[r][-2500:]}" for r in range(world))
        raise AssertionError(f"ranks {failed} failed{' (timeout)' if timed_out else ''}:\n{report}")
    return [json.load(open(os.path.join(workdir, f"result_{r}.json"))) for r in range(world)]
