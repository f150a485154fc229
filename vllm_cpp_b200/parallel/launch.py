"""Multi-rank serving on one node: one process per GPU, one scheduler.

``launch_engine(args)`` is what the server, the CLI and the C interface call. With a tensor-
parallel size of 1 it just builds the engine. Above that the calling process becomes rank 0 (it
owns the scheduler and every request) and one child process per further rank is started with
``python -m vllm_cpp_b200.parallel.launch <spec>``; the children build the same engine on their
weight shard and run ``LLM.serve_as_worker()``: every step reaches them as the packed step buffer
rank 0 publishes on the host-side channel, so they never see a request.

Failures are noticed on the host: a watcher thread polls the children, and a child that exits
while the engine is live marks the engine dead (the next ``step`` raises ``EngineDeadError``
instead of waiting for a collective that cannot complete).

The reference has no distributed code; its design note has the same shape (one scheduler,
step fan-out to rank workers): ``.agents/specs/tensor-parallelism.md:323-349``,
``include/vllm/v1/executor/executor.h:48-85``.
"""
from __future__ import annotations

import dataclasses
import os
import pickle
import socket
import subprocess
import sys
import tempfile
import threading
import time


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init_process_group(device: str, rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist
    if dist.is_initialized():
        return
    if device.startswith("cuda"):
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)


class WorkerGroup:
    """The child processes of a multi-rank engine and the thread that watches them."""

    def __init__(self, procs: list, spec_path: str):
        self.procs = procs
        self.spec_path = spec_path
        self.failed: str | None = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._watch, daemon=True)
        self._thread.start()

    def _watch(self) -> None:
        while not self._stop.is_set():
            for r, p in enumerate(self.procs, start=1):
                rc = p.poll()
                if rc is not None and not self._stop.is_set():
                    self.failed = f"rank {r} exited with code {rc}"
                    return
            time.sleep(0.2)

    def shutdown(self, timeout: float = 30.0) -> None:
        self._stop.set()
        for p in self.procs:
            try:
                p.wait(timeout=timeout)
            except subprocess.TimeoutExpired:
                p.kill()                      # the exact child we started, by its handle
        try:
            os.unlink(self.spec_path)
        except OSError:
            pass


def launch_engine(args, env: dict | None = None):
    """Returns ``(llm, workers)``; ``workers`` is None for a single-rank engine. ``args`` is an
    ``EngineArgs`` whose ``parallel.tensor_parallel_size`` says how many ranks to run."""
    from ..engine import LLM
    tp = max(1, args.parallel.tensor_parallel_size)
    if tp == 1:
        return LLM(args), None
    port = _free_port()
    spec = tempfile.NamedTemporaryFile("wb", suffix=".b200spec", delete=False)
    pickle.dump(args, spec)
    spec.close()
    base_env = dict(os.environ if env is None else env)
    base_env.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(tp))
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    base_env["PYTHONPATH"] = os.pathsep.join([root, base_env.get("PYTHONPATH", "")])
    procs = []
    for r in range(1, tp):
        e = dict(base_env, RANK=str(r), LOCAL_RANK=str(r))
        procs.append(subprocess.Popen([sys.executable, "-m", "vllm_cpp_b200.parallel.launch", spec.name], env=e))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(tp), RANK="0",
                      LOCAL_RANK="0")
    workers = WorkerGroup(procs, spec.name)
    try:
        _init_process_group(args.device, 0, tp)
        par = dataclasses.replace(args.parallel, rank=0, local_rank=0, driver_worker=True)
        llm = LLM(dataclasses.replace(args, parallel=par))
    except BaseException:
        for p in procs:
            p.kill()
        workers.shutdown(timeout=5.0)
        raise
    llm.workers = workers
    return llm, workers


def worker_main(spec_path: str) -> int:
    """Entry of a child rank: same engine, its own shard, steps from rank 0."""
    import torch.distributed as dist
    from ..engine import LLM
    with open(spec_path, "rb") as f:
        args = pickle.load(f)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    _init_process_group(args.device, rank, world)
    par = dataclasses.replace(args.parallel, rank=rank, local_rank=int(os.environ.get("LOCAL_RANK", rank)),
                              driver_worker=True)
    llm = LLM(dataclasses.replace(args, parallel=par))
    llm.serve_as_worker()
    if dist.is_initialized():
        dist.barrier()
    return 0


if __name__ == "__main__":
    rc = worker_main(sys.argv[1])
    sys.stdout.flush()
    os._exit(rc)
