"""Expert-parallel host logic under gloo, world size 2, on CPU (no GPU involved)."""
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mgpt_b200 import synth
from tests.ep_common import init_pg, run_rank
from tests.ep_cpu_stages import CpuStages


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, shape, q):
    try:
        torch.set_num_threads(1)
        init_pg(rank, world, "gloo", port)
        n, C, H, E, k, skew, chunks = shape
        w = synth.Workload("ep", n, C, H, E, k, "fp32", skew=skew)
        run_rank(w, rank, world, lambda w, el: CpuStages(w.C, w.H, w.E, w.k, el, w.alpha, n_chunks=chunks), "cpu", 2e-4)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()))


@pytest.mark.parametrize("shape", [
    (48, 16, 24, 4, 2, False, 1),
    (33, 16, 16, 8, 3, True, 1),
    (48, 16, 24, 4, 2, False, 2),       # two chunks of one expert per rank: exchange overlapped with the expert work
    (61, 16, 16, 8, 3, True, 2),
    (40, 16, 16, 16, 2, False, 4),
])
def test_expert_parallel_two_ranks_gloo(shape):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, shape, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


@pytest.mark.parametrize("chunks", [1, 2])
def test_single_rank_needs_no_process_group(chunks):
    w = synth.Workload("ep1", 40, 16, 24, 4, 2, "fp32")
    run_rank(w, 0, 1, lambda w, el: CpuStages(w.C, w.H, w.E, w.k, el, w.alpha, n_chunks=chunks), "cpu", 2e-4)


def test_experts_must_divide_evenly():
    from mgpt_b200.ep import ExpertParallelMoE
    ExpertParallelMoE(16, 24, 4, 2, stages=CpuStages(16, 24, 4, 2, 4))     # world 1: fine
