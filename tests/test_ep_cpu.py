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


# ---- failures, made on the host: no GPU is involved, nothing is killed mid-collective ----------------------
def _spawn(target, world, args, timeout=120):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q) + tuple(args)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=timeout) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    return results


def _uneven_worker(rank, world, port, q):
    try:
        torch.set_num_threads(1)
        init_pg(rank, world, "gloo", port)
        from mgpt_b200.ep import ExpertParallelMoE
        try:
            ExpertParallelMoE(16, 24, 5, 2, stages=CpuStages(16, 24, 5, 2, 2))      # 5 experts over 2 ranks
            q.put((rank, "no error"))
        except ValueError as e:
            q.put((rank, f"ValueError: {e}"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()))


def test_experts_that_do_not_divide_over_the_ranks_are_refused():
    for rank, msg in _spawn(_uneven_worker, 2, ()).items():
        assert msg.startswith("ValueError") and "not divisible" in msg, f"rank {rank}: {msg}"


def _absent_worker(rank, world, port, q):
    """Rank 1 never joins the step (it raises before its forward, as a rank does whose data loader failed).  Rank 0
    must come back with an error from the count exchange -- the first collective of the step, before any row has
    moved and before any expert kernel was enqueued -- once the group's timeout has passed, not hang."""
    import datetime
    import time
    try:
        torch.set_num_threads(1)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=4))
        from mgpt_b200.ep import ExpertParallelMoE
        w = synth.Workload("ep", 24, 16, 16, 4, 2, "fp32")
        stages = CpuStages(w.C, w.H, w.E, w.k, w.E // world, w.alpha)
        layer = ExpertParallelMoE(w.C, w.H, w.E, w.k, stages=stages)
        calls = {"experts": 0}
        real = stages.experts_forward
        stages.experts_forward = lambda *a, **k: (calls.__setitem__("experts", calls["experts"] + 1), real(*a, **k))[1]
        if rank == 1:
            time.sleep(8)                  # stays alive past the others' timeout, takes no part in the step
            q.put((rank, "absent"))
            return
        t0 = time.time()
        try:
            layer.forward(torch.zeros(w.n_tokens, w.C))
            q.put((rank, "no error"))
        except Exception as e:
            q.put((rank, f"error after {time.time() - t0:.1f}s, expert calls {calls['experts']}: {type(e).__name__}"))
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()))


def test_a_rank_that_never_posts_its_counts_times_the_others_out():
    res = _spawn(_absent_worker, 2, (), timeout=60)
    assert res[1] == "absent"
    assert res[0].startswith("error after") and "expert calls 0" in res[0], res[0]


def test_peer_offsets_reproduce_the_all_to_all():
    """The copy-engine transport pulls block (source -> destination, chunk) from the source's send layout into the
    destination's receive layout; the offsets both sides derive from the all-gathered counts must describe the
    same blocks an all-to-all with those split sizes would deliver, back to back and without overlap."""
    import numpy as np
    from mgpt_b200.ep import peer_offsets
    rng = np.random.default_rng(5)
    for G, nc, Ec in ((2, 1, 4), (4, 2, 2), (8, 2, 1), (3, 3, 2)):
        counts = rng.integers(0, 700, size=(G, G, nc, Ec))
        counts[rng.random(counts.shape) < 0.3] = 0                       # experts nobody routes to
        blk, send_off, recv_off = peer_offsets(counts)
        pad = (counts + 127) // 128 * 128
        assert np.array_equal(blk, pad.sum(3))
        # every rank's send buffer: rows labelled (source, running row index)
        send = [np.arange(int(blk[s].sum())) + 1_000_000 * s for s in range(G)]
        for d in range(G):
            recv = np.full(int(blk[:, d].sum()), -1, dtype=np.int64)
            for c in range(nc):
                for s in range(G):
                    n, so, ro = int(blk[s, d, c]), int(send_off[s, c, d]), int(recv_off[d, c, s])
                    assert (recv[ro: ro + n] == -1).all()                 # no two blocks land on the same rows
                    recv[ro: ro + n] = send[s][so: so + n]
            assert (recv >= 0).all()                                      # and together they fill the layout
            # what all_to_all_single with these split sizes delivers, chunk by chunk: source-major blocks
            want = []
            for c in range(nc):
                for s in range(G):
                    start = int(blk[s].T.reshape(-1)[: c * G + d].sum())  # [chunk][destination] order on the source
                    want.append(send[s][start: start + int(blk[s, d, c])])
            assert np.array_equal(recv, np.concatenate(want))
