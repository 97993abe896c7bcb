"""Expert-parallel MoE layer: tokens stay on their GPU, experts are sharded.

One process per GPU.  Every rank owns ``E/G`` experts (weights, gradients) and a replica
of the router.  Per step:

    route (local)  ->  counts all-to-all  ->  rows all-to-all  ->  experts (local)
                   ->  rows all-to-all back  ->  combine (local)

and the mirror image for backward.  With ``n_chunks > 1`` the experts are split into that
many groups and the exchange of one group's rows runs while the previous group is being
computed: expert ``e`` belongs to chunk ``c = e // (E/n_chunks)`` and, inside the chunk,
to rank ``(e % (E/n_chunks)) // (E/(G*n_chunks))``, so that in the expert-major row order
every chunk is one contiguous range made of one contiguous block per destination rank
(``n_chunks = 1``: rank ``g`` owns experts ``[g*E/G, (g+1)*E/G)``).  Rows travel tile-aligned: expert-major with every
expert's segment padded by zero rows to a multiple of 128, the layout the single-GPU
layer uses internally.  The block for each destination is then one contiguous range and
what arrives (one block per source rank, inside it one padded segment per local expert)
is fed to the tensor-core kernels where it lands; the expert side moves no rows.
The load-balance term of the router gradient uses
each GPU's own counts, which equals running the reference independently on every
GPU's batch.  The reference itself has no multi-GPU code.

torch.distributed is the transport (NCCL on GPUs; gloo works for the host logic with a
CPU stage backend, which is how the tests exercise this file without GPUs).
"""
from __future__ import annotations

import ctypes as ct

import torch
import torch.distributed as dist


class CudaStages:
    """The six stage-level entry points of libmgpt_moe.so on torch CUDA tensors."""

    def __init__(self, C, H, E, k, E_local, *, mode="bf16", device=0, lb_alpha=0.01, n_chunks=1, sm_budget=0):
        from . import _lib
        self._lib_mod = _lib
        self.lib = _lib.load()
        if E_local % n_chunks:
            raise ValueError(f"{E_local} local experts do not split into {n_chunks} chunks")
        self.C, self.H, self.E, self.k, self.E_local = C, H, E, k, E_local
        self.n_chunks, self.E_chunk = n_chunks, E_local // n_chunks
        self.device = torch.device("cuda", device)
        self.act_dtype = torch.bfloat16 if mode == "bf16" else torch.float32
        m = {"fp32": _lib.FP32, "bf16": _lib.BF16}[mode]
        self.home = ct.c_void_p()
        cfg = _lib.Config(C, H, E, k, lb_alpha, m, device, 0)
        _lib.check(self.lib.mgpt_moe_create(ct.byref(cfg), ct.byref(self.home)))
        self.locals = []                 # one expert-side layer per chunk, each with E_chunk experts
        for _ in range(n_chunks):
            h = ct.c_void_p()
            cfg = _lib.Config(C, H, self.E_chunk, 1, lb_alpha, m, device, 0)
            _lib.check(self.lib.mgpt_moe_create(ct.byref(cfg), ct.byref(h)))
            _lib.check(self.lib.mgpt_moe_set_sm_budget(h, sm_budget))
            self.locals.append(h)
        f32 = dict(dtype=torch.float32, device=self.device)
        self.router_params = [torch.zeros(C, E, **f32), torch.zeros(1, E, **f32)]
        self.expert_params = []
        for _ in range(E_local):
            self.expert_params += [torch.zeros(C, H, **f32), torch.zeros(1, H, **f32), torch.zeros(C, H, **f32),
                                   torch.zeros(1, H, **f32), torch.zeros(H, C, **f32), torch.zeros(1, C, **f32)]
        for p in self.router_params + self.expert_params:
            p.grad = torch.zeros_like(p)
        self._bind()
        self._home_ws = None
        self._local_ws = [None] * n_chunks
        self._rows = [None] * n_chunks
        self._seg_counts = [None] * n_chunks
        self._n = 0

    def close(self):
        for h in [self.home] + self.locals:
            if h and h.value:
                self.lib.mgpt_moe_destroy(h)
        self.home, self.locals = ct.c_void_p(), []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _bind(self):
        c = self._lib_mod.check
        rp = self.router_params
        c(self.lib.mgpt_moe_bind_params(self.home, (ct.c_void_p * 2)(*[p.data_ptr() for p in rp]),
                                        (ct.c_void_p * 2)(*[p.grad.data_ptr() for p in rp]), 2))
        per = 6 * self.E_chunk
        for ci, h in enumerate(self.locals):
            mine = self.expert_params[ci * per: (ci + 1) * per]
            n = 2 + per
            data = (ct.c_void_p * n)(None, None, *[p.data_ptr() for p in mine])
            grad = (ct.c_void_p * n)(None, None, *[p.grad.data_ptr() for p in mine])
            c(self.lib.mgpt_moe_bind_params(h, data, grad, n))
        self.sync_weights()

    def sync_weights(self):
        c = self._lib_mod.check
        for h in [self.home] + self.locals:
            c(self.lib.mgpt_moe_sync_weights(h, self._stream()))

    @staticmethod
    def _stream():
        return ct.c_void_p(torch.cuda.current_stream().cuda_stream)

    def adamw_step(self, t, lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        """One fused AdamW step (BF16 copies refreshed in the same pass) over the router replica and this
        rank's experts; moment buffers ``opt_m`` / ``opt_v`` (router first, then the experts) are created on first use."""
        c = self._lib_mod.check
        if getattr(self, "opt_m", None) is None:
            ps = self.router_params + self.expert_params
            self.opt_m = [torch.zeros_like(p) for p in ps]
            self.opt_v = [torch.zeros_like(p) for p in ps]
            arr = lambda ts: (ct.c_void_p * len(ts))(*[None if a is None else a.data_ptr() for a in ts])
            c(self.lib.mgpt_moe_bind_optimizer_state(self.home, arr(self.opt_m[:2]), arr(self.opt_v[:2]), 2))
            per = 6 * self.E_chunk
            for ci, h in enumerate(self.locals):
                m = [None, None] + self.opt_m[2 + ci * per: 2 + (ci + 1) * per]
                v = [None, None] + self.opt_v[2 + ci * per: 2 + (ci + 1) * per]
                c(self.lib.mgpt_moe_bind_optimizer_state(h, arr(m), arr(v), 2 + per))
        for h in [self.home] + self.locals:
            c(self.lib.mgpt_moe_adamw_step(h, lr, beta1, beta2, eps, weight_decay, int(t), self._stream()))

    def _io(self, t):
        return self._lib_mod.IO_BF16 if t.dtype == torch.bfloat16 else self._lib_mod.IO_F32

    def _ws(self, handle, n, routing, cur):
        need = int(self.lib.mgpt_moe_stage_workspace_bytes(handle, n, 1 if routing else 0))
        if cur is None or cur.numel() < need:
            cur = torch.empty(need, dtype=torch.uint8, device=self.device)
        return cur

    def _view(self, handle, ws, n, name, dtype):
        off, nb = ct.c_size_t(), ct.c_size_t()
        self._lib_mod.check(self.lib.mgpt_moe_workspace_view(handle, n, name.encode(), ct.byref(off), ct.byref(nb)))
        return ws[off.value: off.value + nb.value].view(dtype)

    def check_status(self) -> None:
        """Raises if a kernel of the routing side or of any expert chunk reported an error since the last check."""
        for h in [self.home] + self.locals:
            self._lib_mod.check(self.lib.mgpt_moe_check_status(h, None))

    # ---- per-stage timing of the expert side (CUDA events inside the library)
    def set_profiling(self, enabled: bool) -> None:
        for h in self.locals:
            self._lib_mod.check(self.lib.mgpt_moe_set_profiling(h, 1 if enabled else 0))

    def stage_ms(self) -> dict:
        """Per-stage milliseconds of the expert side, summed over the chunks."""
        out = {}
        for h in self.locals:
            buf = (ct.c_float * self._lib_mod.N_STAGES)()
            self._lib_mod.check(self.lib.mgpt_moe_stage_ms(h, buf))
            for i in range(self._lib_mod.N_STAGES):
                name = self.lib.mgpt_moe_stage_name(i).decode()
                out[name] = out.get(name, 0.0) + float(buf[i])
        return out

    # ---- routing side
    def row_capacity(self, n):
        """Rows of the padded expert-major layout for n tokens (every expert's segment a multiple of 128)."""
        self._home_ws = self._home_ws_for(n)
        return self._view(self.home, self._home_ws, n, "row_src", torch.int32).numel()

    def route(self, x, out=None):
        """Returns (rows [row_cap, C] in the padded expert-major layout, counts[E] real rows per expert).
        ``out``: a buffer of at least row_cap rows to write the rows into (else a new tensor)."""
        n = x.shape[0]
        self._home_ws = self._home_ws_for(n)
        self._n = n
        row_cap = self._view(self.home, self._home_ws, n, "row_src", torch.int32).numel()
        rows = out[:row_cap] if out is not None else torch.empty(row_cap, self.C, dtype=self.act_dtype, device=self.device)
        self._lib_mod.check(self.lib.mgpt_moe_route(self.home, x.data_ptr(), n, self._io(x), self._home_ws.data_ptr(),
                                                    self._home_ws.numel(), rows.data_ptr(), self._stream()))
        counts = self._view(self.home, self._home_ws, n, "counts", torch.int32)
        return rows, counts

    def _home_ws_for(self, n):
        return self._ws(self.home, n, True, self._home_ws)

    def routing_view(self, name, dtype):
        return self._view(self.home, self._home_ws, self._n, name, dtype)

    def combine(self, rows_back, like):
        y = torch.empty_like(like)
        self._lib_mod.check(self.lib.mgpt_moe_combine(self.home, rows_back.data_ptr(), y.data_ptr(), self._io(y),
                                                      self._home_ws.data_ptr(), self._home_ws.numel(), self._stream()))
        return y

    def combine_backward(self, rows_back, dy, out=None):
        d_rows = out[:rows_back.shape[0]] if out is not None else torch.empty_like(rows_back)
        self._lib_mod.check(self.lib.mgpt_moe_combine_backward(
            self.home, rows_back.data_ptr(), dy.data_ptr(), self._io(dy), d_rows.data_ptr(),
            self._home_ws.data_ptr(), self._home_ws.numel(), self._stream()))
        return d_rows

    def route_backward(self, x, d_rows):
        dx = torch.empty_like(x)
        self._lib_mod.check(self.lib.mgpt_moe_route_backward(
            self.home, x.data_ptr(), d_rows.data_ptr(), dx.data_ptr(), self._io(x),
            self._home_ws.data_ptr(), self._home_ws.numel(), self._stream()))
        return dx

    # ---- expert side
    def experts_forward(self, rows, seg_counts, n_src, chunk=0, out=None):
        """rows: n_src blocks of padded per-expert segments of chunk ``chunk``;
        seg_counts: int32 [n_src, E_chunk] real counts."""
        n = rows.shape[0]
        h = self.locals[chunk]
        self._local_ws[chunk] = self._ws(h, n, False, self._local_ws[chunk])
        ws = self._local_ws[chunk]
        out = torch.empty_like(rows) if out is None else out
        self._seg_counts[chunk] = seg_counts.contiguous()
        self._lib_mod.check(self.lib.mgpt_moe_experts_forward(
            h, rows.data_ptr(), self._seg_counts[chunk].data_ptr(), n_src, n, out.data_ptr(),
            ws.data_ptr(), ws.numel(), self._stream()))
        self._rows[chunk] = rows          # read again by the weight gradients
        return out

    def experts_backward(self, d_out, chunk=0):
        d_in = torch.empty_like(d_out)
        ws = self._local_ws[chunk]
        self._lib_mod.check(self.lib.mgpt_moe_experts_backward(
            self.locals[chunk], d_out.data_ptr(), d_in.data_ptr(), ws.data_ptr(), ws.numel(), self._stream()))
        return d_in

    def experts_backward_rows(self, d_out, chunk=0, out=None):
        """First half of experts_backward: the gradient w.r.t. the received rows (what the other ranks wait for)."""
        d_in = torch.empty_like(d_out) if out is None else out
        ws = self._local_ws[chunk]
        self._lib_mod.check(self.lib.mgpt_moe_experts_backward_rows(
            self.locals[chunk], d_out.data_ptr(), d_in.data_ptr(), ws.data_ptr(), ws.numel(), self._stream()))
        self._bwd_bufs = getattr(self, "_bwd_bufs", {})
        self._bwd_bufs[chunk] = (d_out, d_in)
        return d_in

    def experts_backward_params(self, chunk=0):
        """Second half: this chunk's expert parameter gradients, from the buffers of experts_backward_rows."""
        d_out, d_in = self._bwd_bufs.pop(chunk)
        ws = self._local_ws[chunk]
        self._lib_mod.check(self.lib.mgpt_moe_experts_backward_params(
            self.locals[chunk], d_out.data_ptr(), d_in.data_ptr(), ws.data_ptr(), ws.numel(), self._stream()))


class _RawCuda:
    """A device pointer dressed up for torch.as_tensor (bytes; the caller views it in its own dtype)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def peer_offsets(counts):
    """counts[source, destination, chunk, j]: real rows that `source` routes to local expert j of chunk `chunk` on
    `destination`.  Returns (blk[source, destination, chunk] padded rows of the block, send_off[source, chunk,
    destination] its first row in the source's send layout ([chunk][destination] blocks back to back),
    recv_off[destination, chunk, source] its first row in the destination's receive layout ([chunk][source])).
    Every expert's segment is padded to a multiple of 128 rows."""
    import numpy as np
    M = np.asarray(counts).astype(np.int64)
    G, nc = M.shape[0], M.shape[2]
    blk = ((M + 127) // 128 * 128).sum(3)
    send_off = np.zeros((G, nc, G), dtype=np.int64)
    recv_off = np.zeros((G, nc, G), dtype=np.int64)
    for r in range(G):
        a = blk[r].T.reshape(-1)                       # [chunk][destination] of source r
        send_off[r] = (np.cumsum(a) - a).reshape(nc, G)
        b = blk[:, r, :].T.reshape(-1)                 # [chunk][source] into destination r
        recv_off[r] = (np.cumsum(b) - b).reshape(nc, G)
    return blk, send_off, recv_off


class _CopyLanes:
    """A few streams used as one for copy-engine transfers: blocks from different peers go out on different lanes
    (one copy at a time does not fill the NVLink ports when the blocks are small), waits and records apply to all."""

    def __init__(self, device, n):
        self.streams = [torch.cuda.Stream(device=device, priority=-1) for _ in range(n)]

    def wait_event(self, ev):
        for st in self.streams:
            st.wait_event(ev)

    def lane(self, i):
        return self.streams[i % len(self.streams)]

    def record(self):
        evs = []
        for st in self.streams:
            e = torch.cuda.Event()
            e.record(st)
            evs.append(e)
        return evs


def _wait_all(stream, events):
    for e in events:
        stream.wait_event(e)


class PeerRows:
    """One row buffer per rank that the other ranks of the node read directly (``mgpt_moe_peer_*``: cudaMalloc +
    CUDA IPC).  ``tensor`` is this rank's buffer [rows, C]; ``peer[s]`` the device address of rank s's buffer as
    mapped into this process.  Collective over the group (the handles are all-gathered)."""

    def __init__(self, lib_mod, lib, group, rank, world, device, rows, C, dtype):
        self.lib_mod, self.lib, self.device_index = lib_mod, lib, device.index
        self.row_bytes = C * torch.empty((), dtype=dtype).element_size()
        nbytes = max(1, rows) * self.row_bytes
        ptr, handle = ct.c_void_p(), ct.create_string_buffer(lib_mod.PEER_HANDLE_BYTES)
        lib_mod.check(lib.mgpt_moe_peer_alloc(self.device_index, nbytes, ct.byref(ptr), handle))
        self.ptr = ptr.value
        self.tensor = torch.as_tensor(_RawCuda(self.ptr, nbytes), device=device).view(dtype).view(max(1, rows), C)
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.peer, self._opened = [], []
        for s in range(world):
            if s == rank:
                self.peer.append(self.ptr)
                continue
            p = ct.c_void_p()
            lib_mod.check(lib.mgpt_moe_peer_open(self.device_index, handles[s], ct.byref(p)))
            self.peer.append(p.value)
            self._opened.append(p.value)

    def close(self, group=None):
        """Collective: every rank closes its mappings before any rank frees its buffer."""
        for p in self._opened:
            self.lib.mgpt_moe_peer_close(self.device_index, ct.c_void_p(p))
        self._opened = []
        if dist.is_initialized():
            dist.barrier(group=group)
        if self.ptr:
            self.tensor = None
            self.lib.mgpt_moe_peer_free(self.device_index, ct.c_void_p(self.ptr))
            self.ptr = None


class ExpertParallelMoE:
    """Same role as the reference's MoELayer, with the experts sharded over a process group."""

    def __init__(self, embed_dim, hidden_dim, num_experts, top_k, *, group=None, stages=None, mode="bf16",
                 device=0, lb_alpha=0.01, n_chunks=1, sm_budget=0, transport="collective"):
        """``transport``: "collective" moves the rows with ``all_to_all_single`` (NCCL's copy kernels; gloo on CPU);
        "peer" lets the rank that needs a block pull it from the producer's buffer with a copy engine
        (one node, GPUs with peer access; see ``PeerRows``), so that the exchange needs no SM."""
        if transport not in ("collective", "peer"):
            raise ValueError(f"unknown transport {transport!r}")
        self.transport = transport
        self.copy_lanes = 1      # streams the pulls are spread over; more than one lets a later chunk's copies compete with the chunk the compute stream is waiting for (8 GPUs: 5.44 ms with three against 5.07 with one)
        self._peer = None
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world:
            raise ValueError(f"num_experts={num_experts} is not divisible by the group size {self.world}")
        self.C = embed_dim
        self.H = 4 * embed_dim if hidden_dim == -1 else hidden_dim
        self.E, self.k = num_experts, top_k
        self.E_local = num_experts // self.world
        self.stages = stages if stages is not None else CudaStages(
            self.C, self.H, self.E, self.k, self.E_local, mode=mode, device=device, lb_alpha=lb_alpha,
            n_chunks=n_chunks, sm_budget=sm_budget)
        self.n_chunks = getattr(self.stages, "n_chunks", 1)
        if self.E_local % self.n_chunks:
            raise ValueError(f"{self.E_local} local experts do not split into {self.n_chunks} chunks")
        self.E_chunk = self.E_local // self.n_chunks
        self._saved = None
        self.phase_events = None        # set to {} to record CUDA events around every phase of a step

    def _mark(self, name):
        if self.phase_events is not None and torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_events.setdefault("order", []).append((name, ev))

    def phase_ms(self):
        """Milliseconds between consecutive marks of the last recorded step (after a synchronize)."""
        marks = (self.phase_events or {}).get("order", [])
        out = {}
        for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out

    # parameters: the router replica and this rank's experts, in the reference's order
    def get_parameters(self):
        return list(self.stages.router_params) + list(self.stages.expert_params)

    def global_expert(self, local_index: int, rank=None) -> int:
        """Global id of local expert ``local_index`` (local order: chunk by chunk) of ``rank``."""
        rank = self.rank if rank is None else rank
        c, j = divmod(local_index, self.E_chunk)
        return c * (self.E // self.n_chunks) + rank * self.E_chunk + j

    def load_parameters(self, full_params):
        """Takes the full 2+6E list (as numpy arrays or tensors) and keeps the router and this rank's experts."""
        import numpy as np
        mine = list(full_params[:2])
        for l in range(self.E_local):
            e = self.global_expert(l)
            mine += list(full_params[2 + 6 * e: 2 + 6 * (e + 1)])
        for p, a in zip(self.get_parameters(), mine):
            t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)) if not torch.is_tensor(a) else a
            p.copy_(t.reshape(p.shape))
        self.stages.sync_weights()

    def zero_grad(self):
        for p in self.get_parameters():
            p.grad.zero_()

    def adamw_step(self, t, **hyper):
        """Optimiser step over the router replica and this rank's experts (sum the router gradients over the
        group first with ``allreduce_router_grads()`` if the replicas are to stay identical)."""
        self.stages.adamw_step(t, **hyper)

    def allreduce_router_grads(self):
        """Sum the router gradients over the group so that the replicas stay identical."""
        if self.world > 1:
            for p in self.stages.router_params:
                dist.all_reduce(p.grad, group=self.group)

    # ---- exchange helpers
    def _exchange(self, recv, send, recv_splits, send_splits):
        """Starts recv <- all-to-all(send) (rows split per rank); returns a handle to wait on, or None."""
        if self.world == 1:
            recv.copy_(send)
            return None
        return dist.all_to_all_single(recv, send, list(recv_splits), list(send_splits), group=self.group, async_op=True)

    @staticmethod
    def _pad128(t):
        return (t + 127) // 128 * 128

    # ---- "peer" transport: persistent buffers, pulled by copy engines
    def _peer_setup(self, n):
        """Buffers for up to n tokens per rank (collective on first use or growth).  Four are readable by the peers:
        the rows this rank routes (A), its experts' outputs (B), and the two gradient mirrors (Cg, D)."""
        pb = self._peer
        if pb is not None and n <= pb["n"]:
            return pb
        st = self.stages
        t = torch.tensor([n], device=st.device, dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        n_max = int(t.item())
        if pb is not None:
            self.close_peer()
        cap_send = st.row_capacity(n_max)
        cap_recv = self.world * cap_send              # worst case: every rank routes all of its rows to this one
        mk = lambda rows: PeerRows(st._lib_mod, st.lib, self.group, self.rank, self.world, st.device, rows, self.C,
                                   st.act_dtype)
        loc = lambda rows: torch.empty(rows, self.C, dtype=st.act_dtype, device=st.device)
        pb = {"n": n_max, "A": mk(cap_send), "B": mk(cap_recv), "Cg": mk(cap_send), "D": mk(cap_recv),
              "recv": loc(cap_recv), "rows_back": loc(cap_send), "d_recv": loc(cap_recv), "d_back": loc(cap_send),
              "stream": _CopyLanes(st.device, self.copy_lanes),
              "flag": torch.zeros(1, device=st.device)}
        self._peer = pb
        return pb

    def close_peer(self):
        """Collective: releases the peer-readable buffers."""
        if self._peer is not None:
            torch.cuda.synchronize()
            for k in ("A", "B", "Cg", "D"):
                self._peer[k].close(self.group)
            self._peer = None

    def _barrier_then(self, X):
        """Every rank's kernels queued on the current stream so far are complete on every rank before anything
        queued on X from here on starts.  The barrier (a one-element all-reduce) is queued in the order of the
        compute stream, not beside it: its kernel needs an SM, the persistent kernels hold them all, and queued
        beside them it would start only when the NEXT compute kernel ends, which is when the copies it releases
        should already be done."""
        cur = torch.cuda.current_stream()
        dist.all_reduce(self._peer["flag"], group=self.group)
        e = torch.cuda.Event()
        e.record(cur)
        X.wait_event(e)

    def _pull(self, dst, dst_row, src_ptr, src_row, rows, row_bytes, stream):
        if rows > 0:
            st = self.stages
            st._lib_mod.check(st.lib.mgpt_moe_peer_copy(
                ct.c_void_p(dst.data_ptr() + dst_row * row_bytes), ct.c_void_p(src_ptr + src_row * row_bytes),
                rows * row_bytes, ct.c_void_p(stream.cuda_stream)))

    def _peer_layout(self, counts):
        """All-gathers the per-destination counts and derives, for every (source, destination, chunk), the rows of
        the block and where it sits in the source's send layout ([chunk][destination]) and in the destination's
        receive layout ([chunk][source]).  One host synchronisation."""
        import numpy as np
        G, nc, Ec = self.world, self.n_chunks, self.E_chunk
        send_counts = counts.view(nc, G, Ec).permute(1, 0, 2).contiguous()             # [destination, chunk, j]
        every = torch.empty((G,) + tuple(send_counts.shape), dtype=send_counts.dtype, device=send_counts.device)
        dist.all_gather_into_tensor(every, send_counts, group=self.group)               # [source, destination, chunk, j]
        blk, send_off, recv_off = peer_offsets(every.cpu().numpy())
        return every, blk, send_off, recv_off

    def _forward_peer(self, x):
        G, nc, me = self.world, self.n_chunks, self.rank
        pb = self._peer_setup(x.shape[0])
        X, cur = pb["stream"], torch.cuda.current_stream()
        rb = pb["A"].row_bytes
        rows, counts = self.stages.route(x, out=pb["A"].tensor)
        ev_rows = torch.cuda.Event()
        ev_rows.record(cur)
        self._mark("route")
        every, blk, send_off, recv_off = self._peer_layout(counts)
        self._mark("counts_exchange_and_host_sync")
        order = [(me + i) % G for i in range(G)]          # every rank starts at a different peer
        n_send = int(blk[me].sum())
        recv_rows_c = [int(blk[:, me, c].sum()) for c in range(nc)]
        recv_base = [int(recv_off[me][c][0]) for c in range(nc)]
        # the all-gather of the counts was queued behind the routing kernels on every rank and has completed (the host
        # has read its result): every rank's rows are written
        X.wait_event(ev_rows)
        ev_recv = []
        for c in range(nc):
            for i, s in enumerate(order):
                self._pull(pb["recv"], int(recv_off[me][c][s]), pb["A"].peer[s], int(send_off[s][c][me]),
                           int(blk[s][me][c]), rb, X.lane(i))
            ev_recv.append(X.record())
        rows_back = pb["rows_back"][:n_send]
        for c in range(nc):
            _wait_all(cur, ev_recv[c])
            self._mark("rows_all_to_all")
            lo, hi = recv_base[c], recv_base[c] + recv_rows_c[c]
            self.stages.experts_forward(pb["recv"][lo:hi], every[:, me, c, :], G, *([c] if nc > 1 else []),
                                        out=pb["B"].tensor[lo:hi])
            self._mark("experts_forward")
            self._barrier_then(X)                         # chunk c's outputs are written on every rank
            for i, o in enumerate(order):
                self._pull(rows_back, int(send_off[me][c][o]), pb["B"].peer[o], int(recv_off[o][c][me]),
                           int(blk[me][o][c]), rb, X.lane(i))
        _wait_all(cur, X.record())
        self._mark("rows_back_all_to_all")
        y = self.stages.combine(rows_back, x)
        self._mark("combine")
        self._saved = (x, rows_back, (blk, send_off, recv_off, recv_base, recv_rows_c, order), None, None)
        self.last_recv_counts = every[:, me].reshape(G, nc * self.E_chunk)      # [source rank, local expert]
        return y

    def _backward_peer(self, dy):
        G, nc, me = self.world, self.n_chunks, self.rank
        pb = self._peer
        X, cur = pb["stream"], torch.cuda.current_stream()
        rb = pb["A"].row_bytes
        x, rows_back, (blk, send_off, recv_off, recv_base, recv_rows_c, order), _, _ = self._saved
        n_send = rows_back.shape[0]
        self.stages.combine_backward(rows_back, dy, out=pb["Cg"].tensor)
        self._mark("combine_backward")
        self._barrier_then(X)                             # every rank's row gradients are written
        ev_recv = []
        for c in range(nc):
            for i, s in enumerate(order):
                self._pull(pb["d_recv"], int(recv_off[me][c][s]), pb["Cg"].peer[s], int(send_off[s][c][me]),
                           int(blk[s][me][c]), rb, X.lane(i))
            ev_recv.append(X.record())
        d_back = pb["d_back"][:n_send]
        for c in range(nc):
            _wait_all(cur, ev_recv[c])
            self._mark("grad_rows_all_to_all")
            lo, hi = recv_base[c], recv_base[c] + recv_rows_c[c]
            self.stages.experts_backward_rows(pb["d_recv"][lo:hi], *([c] if nc > 1 else []), out=pb["D"].tensor[lo:hi])
            self._mark("experts_backward_rows")
            self._barrier_then(X)                         # chunk c's input gradients are written on every rank
            for i, o in enumerate(order):
                self._pull(d_back, int(send_off[me][c][o]), pb["D"].peer[o], int(recv_off[o][c][me]),
                           int(blk[me][o][c]), rb, X.lane(i))
            self.stages.experts_backward_params(*([c] if nc > 1 else []))
            self._mark("experts_backward_params")
        _wait_all(cur, X.record())
        self._mark("grad_rows_back_all_to_all")
        dx = self.stages.route_backward(x, d_back)
        self._mark("route_backward")
        return dx

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        G, nc, Ec = self.world, self.n_chunks, self.E_chunk
        if self.phase_events is not None:
            self.phase_events["order"] = []
        self._mark("start")
        if self.transport == "peer" and G > 1:
            return self._forward_peer(x)
        rows, counts = self.stages.route(x)              # padded expert-major rows, counts[E] in (chunk, rank, j) order
        self._mark("route")
        send_counts = counts.view(nc, G, Ec).permute(1, 0, 2).contiguous()      # [destination, chunk, j]
        recv_counts = torch.empty_like(send_counts)                            # [source, chunk, j]
        if G == 1:
            recv_counts.copy_(send_counts)
        else:
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        both = torch.stack([send_counts, recv_counts]).cpu().numpy()           # the one host sync; the rest is host arithmetic
        padded = (both + 127) // 128 * 128                                     # [2][rank][chunk][j]
        send_splits, recv_splits = padded[0].sum(2).T.tolist(), padded[1].sum(2).T.tolist()      # [chunk][rank] padded rows
        starts, n_send = [], 0
        for c in range(nc):
            starts.append(n_send)
            n_send += int(sum(send_splits[c]))
        self._mark("counts_exchange_and_host_sync")
        # every chunk's exchange is started at once (they run in this order on the communication stream);
        # chunk c is computed while chunk c+1 is still arriving and its results travel back during chunk c+1's work
        recv_rows, pending = [], []
        for c in range(nc):
            r = rows.new_empty((int(sum(recv_splits[c])), self.C))
            pending.append(self._exchange(r, rows[starts[c]: starts[c] + int(sum(send_splits[c]))],
                                          recv_splits[c], send_splits[c]))
            recv_rows.append(r)
        rows_back = torch.empty_like(rows[:n_send])
        back = []
        for c in range(nc):
            if pending[c] is not None:
                pending[c].wait()
            self._mark("rows_all_to_all")
            out_rows = self.stages.experts_forward(recv_rows[c], recv_counts[:, c, :], G, *([c] if nc > 1 else []))
            self._mark("experts_forward")
            back.append(self._exchange(rows_back[starts[c]: starts[c] + int(sum(send_splits[c]))], out_rows,
                                       send_splits[c], recv_splits[c]))
        for wk in back:
            if wk is not None:
                wk.wait()
        self._mark("rows_back_all_to_all")
        y = self.stages.combine(rows_back, x)
        self._mark("combine")
        self._saved = (x, rows_back, send_splits, recv_splits, starts)
        self.last_recv_counts = recv_counts.reshape(G, nc * Ec)      # [source rank, local expert]
        return y

    def backward(self, dy: torch.Tensor) -> torch.Tensor:
        if self._saved is None:
            raise RuntimeError("backward before forward")
        nc = self.n_chunks
        if self.transport == "peer" and self.world > 1:
            return self._backward_peer(dy)
        x, rows_back, send_splits, recv_splits, starts = self._saved
        d_rows = self.stages.combine_backward(rows_back, dy)
        self._mark("combine_backward")
        d_recv, pending = [], []
        for c in range(nc):
            r = d_rows.new_empty((int(sum(recv_splits[c])), self.C))
            pending.append(self._exchange(r, d_rows[starts[c]: starts[c] + int(sum(send_splits[c]))],
                                          recv_splits[c], send_splits[c]))
            d_recv.append(r)
        d_back = torch.empty_like(rows_back)
        back = []
        for c in range(nc):
            if pending[c] is not None:
                pending[c].wait()
            self._mark("grad_rows_all_to_all")
            # the rows' gradients first: they start travelling back while this chunk's parameter gradients
            # (the larger half of the work) are still being formed
            d_in = self.stages.experts_backward_rows(d_recv[c], *([c] if nc > 1 else []))
            self._mark("experts_backward_rows")
            back.append(self._exchange(d_back[starts[c]: starts[c] + int(sum(send_splits[c]))], d_in,
                                       send_splits[c], recv_splits[c]))
            self.stages.experts_backward_params(*([c] if nc > 1 else []))
            self._mark("experts_backward_params")
        for wk in back:
            if wk is not None:
                wk.wait()
        self._mark("grad_rows_back_all_to_all")
        dx = self.stages.route_backward(x, d_back)
        self._mark("route_backward")
        return dx


class NativeExpertParallelMoE:
    """The same layer through the C ABI alone (``mgpt_moe_ep_*``): routing, exchange (NCCL point-to-point on the
    library's own stream) and overlap all happen inside ``libmgpt_moe.so``, which is what an engine written in C++
    binds.  torch is used here for device memory and, in ``create_id``, to hand rank 0's NCCL id to the other ranks."""

    def __init__(self, embed_dim, hidden_dim, num_experts, top_k, *, rank=0, world=1, nccl_id=None, mode="bf16",
                 device=0, lb_alpha=0.01, n_chunks=1, max_tokens=0):
        """``max_tokens`` > 0 (one node, peer access): rows are pulled by copy engines from peer-readable buffers
        sized for that many tokens per call (``mgpt_moe_ep_config::max_tokens``); 0: NCCL point-to-point."""
        from . import _lib
        self._lib_mod = _lib
        self.lib = _lib.load()
        self.C = embed_dim
        self.H = 4 * embed_dim if hidden_dim == -1 else hidden_dim
        self.E, self.k, self.rank, self.world, self.n_chunks = num_experts, top_k, rank, world, n_chunks
        self.E_local = num_experts // world
        self.device = torch.device("cuda", device)
        m = {"fp32": _lib.FP32, "bf16": _lib.BF16}[mode]
        cfg = _lib.EpConfig(embed_dim, hidden_dim, num_experts, top_k, lb_alpha, m, device, rank, world, n_chunks,
                            int(max_tokens))
        self._h = ct.c_void_p()
        idbuf = (ct.c_char * _lib.EP_ID_BYTES).from_buffer_copy(nccl_id) if nccl_id is not None else None
        _lib.check(self.lib.mgpt_moe_ep_create(ct.byref(cfg), idbuf, ct.byref(self._h)))
        f32 = dict(dtype=torch.float32, device=self.device)
        self.params = [torch.zeros(self.C, self.E, **f32), torch.zeros(1, self.E, **f32)]
        for _ in range(self.E_local):
            self.params += [torch.zeros(self.C, self.H, **f32), torch.zeros(1, self.H, **f32), torch.zeros(self.C, self.H, **f32),
                            torch.zeros(1, self.H, **f32), torch.zeros(self.H, self.C, **f32), torch.zeros(1, self.C, **f32)]
        for p in self.params:
            p.grad = torch.zeros_like(p)
        n = len(self.params)
        assert n == self.lib.mgpt_moe_ep_num_params(self._h)
        data = (ct.c_void_p * n)(*[p.data_ptr() for p in self.params])
        grad = (ct.c_void_p * n)(*[p.grad.data_ptr() for p in self.params])
        _lib.check(self.lib.mgpt_moe_ep_bind_params(self._h, data, grad, n))
        self._x = None

    @staticmethod
    def create_id(group=None) -> bytes:
        """Rank 0 asks NCCL for an id; every rank of the torch.distributed group gets it."""
        from . import _lib
        lib = _lib.load()
        buf = torch.zeros(_lib.EP_ID_BYTES, dtype=torch.uint8)
        if not dist.is_initialized() or dist.get_rank(group) == 0:
            raw = (ct.c_char * _lib.EP_ID_BYTES)()
            _lib.check(lib.mgpt_moe_ep_unique_id(raw))
            buf = torch.frombuffer(bytearray(raw.raw), dtype=torch.uint8).clone()
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dev = buf.cuda() if dist.get_backend(group) == "nccl" else buf
            dist.broadcast(dev, src=0, group=group)
            buf = dev.cpu()
        return bytes(buf.numpy().tobytes())

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            self.lib.mgpt_moe_ep_destroy(self._h)
            self._h = ct.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _stream():
        return ct.c_void_p(torch.cuda.current_stream().cuda_stream)

    def get_parameters(self):
        return self.params

    def global_expert(self, local_index: int) -> int:
        return int(self.lib.mgpt_moe_ep_global_expert(self._h, local_index))

    def load_parameters(self, full_params):
        import numpy as np
        mine = list(full_params[:2])
        for l in range(self.E_local):
            e = self.global_expert(l)
            mine += list(full_params[2 + 6 * e: 2 + 6 * (e + 1)])
        for p, a in zip(self.params, mine):
            t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)) if not torch.is_tensor(a) else a
            p.copy_(t.reshape(p.shape))
        self._lib_mod.check(self.lib.mgpt_moe_ep_sync_weights(self._h, self._stream()))

    def zero_grad(self):
        for p in self.params:
            p.grad.zero_()

    def _io(self, t):
        return self._lib_mod.IO_BF16 if t.dtype == torch.bfloat16 else self._lib_mod.IO_F32

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = torch.empty_like(x)
        self._lib_mod.check(self.lib.mgpt_moe_ep_forward(self._h, x.data_ptr(), y.data_ptr(), x.shape[0], self._io(x),
                                                         self._stream()))
        self._x = x
        buf = (ct.c_int32 * (self.world * self.E_local))()
        self._lib_mod.check(self.lib.mgpt_moe_ep_received_counts(self._h, buf))
        self.last_recv_counts = torch.tensor(list(buf), dtype=torch.int32).view(self.world, self.E_local)
        return y

    def backward(self, dy: torch.Tensor) -> torch.Tensor:
        dx = torch.empty_like(dy)
        self._lib_mod.check(self.lib.mgpt_moe_ep_backward(self._h, self._x.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                                          self._io(dy), self._stream()))
        return dx

    def check_status(self):
        self._lib_mod.check(self.lib.mgpt_moe_ep_check_status(self._h))
