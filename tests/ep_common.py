"""Shared driver of the expert-parallel tests: runs one rank and checks it against the CPU oracle.

Oracle for expert parallelism: the single-process reference run on each rank's token shard with the
FULL expert set; outputs and dx compare per shard, routing per shard (bit-exact), expert gradients
compare with the SUM over shards, router gradients per shard.
"""
import numpy as np
import torch
import torch.distributed as dist

from mgpt_b200 import synth
from mgpt_b200.ep import ExpertParallelMoE
from oracle import oracle
from tests.util import rel_l2


def shard_inputs(w, rank, seed=77):
    x, params, dy = synth.make_inputs(w, seed=seed + rank, bias_std=0.02)
    _, params, _ = synth.make_inputs(w, seed=seed, bias_std=0.02)          # same weights everywhere
    return x, params, dy


def run_rank(w, rank, world, make_stages, device, tol, io=torch.float32, make_layer=None):
    x, params, dy = shard_inputs(w, rank)
    E_local = w.E // world
    if make_layer is not None:
        layer = make_layer(w)                      # e.g. the C-ABI form of the layer
    else:
        layer = ExpertParallelMoE(w.C, w.H, w.E, w.k, stages=make_stages(w, E_local))
    layer.load_parameters(params)
    layer.zero_grad()
    xt = torch.from_numpy(x).to(device).to(io)
    y = layer.forward(xt)
    dx = layer.backward(torch.from_numpy(dy).to(device).to(io))
    if device != "cpu":
        torch.cuda.synchronize()

    d = oracle.Dims(w.n_tokens, w.C, w.H, w.E, w.k, w.alpha)
    refs = [oracle.run(d, *shard_inputs(w, r)[:2], shard_inputs(w, r)[2], threads=2) for r in range(world)]
    mine = refs[rank]
    assert rel_l2(y.float().cpu().numpy(), mine["y"]) <= tol, ("y", rel_l2(y.float().cpu().numpy(), mine["y"]))
    assert rel_l2(dx.float().cpu().numpy(), mine["dx"]) <= tol, ("dx", rel_l2(dx.float().cpu().numpy(), mine["dx"]))
    # rows arrive ordered by (source rank, expert): the receive counts are the senders' counts
    got_counts = layer.last_recv_counts.cpu().numpy()
    mine_global = [layer.global_expert(l) for l in range(E_local)]        # local order: chunk by chunk
    want = np.stack([refs[r]["counts"][mine_global] for r in range(world)])
    assert np.array_equal(got_counts, want)
    ps = layer.get_parameters()
    for i in range(2):      # router gradients: this shard only
        assert rel_l2(ps[i].grad.cpu().numpy(), mine["grads"][i]) <= tol, (f"router grad {i}",)
    for j in range(6 * E_local):      # expert gradients: sum over all shards
        gi = 2 + 6 * mine_global[j // 6] + j % 6
        total = sum(r["grads"][gi] for r in refs)
        assert rel_l2(ps[2 + j].grad.cpu().numpy(), total) <= tol, (f"expert grad {gi}", rel_l2(ps[2 + j].grad.cpu().numpy(), total))
    return layer


def init_pg(rank, world, backend, port):
    dist.init_process_group(backend, init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
