"""A CPU stand-in for the six stage-level entry points (numpy + the CPU oracle's routing).

Test infrastructure: lets the host logic of mgpt_b200/ep.py (count exchange, split sizes,
row order, regrouping) run under gloo without a GPU.
"""
import numpy as np
import torch

from oracle import oracle


def _silu(g):
    return g / (1.0 + np.exp(-g))


class CpuStages:
    def __init__(self, C, H, E, k, E_local, alpha=0.01, n_chunks=1):
        self.C, self.H, self.E, self.k, self.E_local, self.alpha = C, H, E, k, E_local, alpha
        self.n_chunks, self.E_chunk = n_chunks, E_local // n_chunks
        self.saved = [None] * n_chunks
        z = lambda *s: torch.zeros(*s, dtype=torch.float32)
        self.router_params = [z(C, E), z(1, E)]
        self.expert_params = []
        for _ in range(E_local):
            self.expert_params += [z(C, H), z(1, H), z(C, H), z(1, H), z(H, C), z(1, C)]
        for p in self.router_params + self.expert_params:
            p.grad = torch.zeros_like(p)

    def sync_weights(self):
        pass

    # ---- routing side (rows in the padded expert-major layout of the CUDA stages)
    def _layout(self):
        r, k = self.r, self.k
        cnt, off = r["counts"].astype(np.int64), r["offsets"].astype(np.int64)
        poff = np.concatenate([[0], np.cumsum((cnt + 127) // 128 * 128)])
        flat_e = r["top_idx"].reshape(-1).astype(np.int64)
        slot_of = np.empty(self.n * k, np.int64)
        slot_of[r["map"]] = np.arange(self.n * k)
        self.pos = poff[flat_e] + slot_of - off[flat_e]          # flat index -> padded row
        self.n_rows = int(poff[-1])

    def route(self, x):
        xn = x.numpy()
        n = xn.shape[0]
        dummy = [np.zeros(s, np.float32) for s in oracle.param_shapes(self.C, self.H, self.E)[2:]]
        params = [p.numpy() for p in self.router_params] + dummy
        r = oracle.run(oracle.Dims(n, self.C, self.H, self.E, self.k, self.alpha), xn, params, route_only=True)
        self.r, self.n = r, n
        self._layout()
        rows = np.zeros((self.n_rows + 128, self.C), np.float32)      # a little spare capacity, like row_cap
        rows[self.pos] = xn[np.arange(n * self.k) // self.k]
        return torch.from_numpy(rows), torch.from_numpy(r["counts"].copy())

    def combine(self, rows_back, like):
        k = self.k
        y = np.zeros((self.n, self.C), np.float32)
        rb, tp = rows_back.numpy(), self.r["top_p"].reshape(-1)
        for flat in np.argsort(self.pos):                 # ascending row order, like the reference's slot order
            y[flat // k] += rb[self.pos[flat]] * tp[flat]
        return torch.from_numpy(y)

    def combine_backward(self, rows_back, dy):
        k = self.k
        rb, g, tp = rows_back.numpy(), dy.numpy(), self.r["top_p"].reshape(-1)
        d_rows = np.zeros_like(rb)
        self.dtp = np.zeros(self.n * k, np.float32)
        for flat in range(self.n * k):
            p = self.pos[flat]
            d_rows[p] = g[flat // k] * tp[flat]
            self.dtp[flat] = float(rb[p] @ g[flat // k])
        return torch.from_numpy(d_rows)

    def route_backward(self, x, d_rows):
        r, k, E, n = self.r, self.k, self.E, self.n
        xn, dr = x.numpy(), d_rows.numpy()
        dx = np.zeros_like(xn)
        for flat in range(n * k):
            dx[flat // k] += dr[self.pos[flat]]
        dP = np.zeros((n, E), np.float32)
        flat_e = r["top_idx"].reshape(-1)
        dP[np.arange(n * k) // k, flat_e] = self.dtp
        dP += (self.alpha * E * (r["counts"].astype(np.float32) / n)) / n
        P = r["probs"]
        dL = P * (dP - (dP * P).sum(1, keepdims=True))
        Wr = self.router_params[0].numpy()
        self.router_params[0].grad += torch.from_numpy(xn.T @ dL)
        self.router_params[1].grad += torch.from_numpy(dL.sum(0, keepdims=True))
        return torch.from_numpy(dx + dL @ Wr.T)

    # ---- expert side: n_src blocks, each one padded segment per local expert
    def experts_forward(self, rows, seg_counts, n_src, chunk=0):
        Ec = self.E_chunk
        X, sc = rows.numpy(), seg_counts.numpy().reshape(n_src, Ec)
        index = [[] for _ in range(Ec)]
        r0 = 0
        for s in range(n_src):
            for e in range(Ec):
                c = int(sc[s, e])
                index[e] += list(range(r0, r0 + c))
                assert not X[r0 + c: r0 + (c + 127) // 128 * 128].any(), "padding rows must arrive as zeros"
                r0 += (c + 127) // 128 * 128
        assert r0 == X.shape[0]
        out = np.zeros_like(X)
        saved = self.saved[chunk] = []
        for e in range(Ec):
            idx = np.array(index[e], dtype=np.int64)
            le = chunk * Ec + e                     # local expert
            Wg, bg, Wu, bu, Wd, bd = [p.numpy() for p in self.expert_params[6 * le: 6 * le + 6]]
            xe = X[idx]
            G, U = xe @ Wg + bg, xe @ Wu + bu
            Hh = _silu(G) * U
            out[idx] = Hh @ Wd + bd
            saved.append((idx, xe, G, U, Hh))
        return torch.from_numpy(out)

    def experts_backward(self, d_out, chunk=0):
        D = d_out.numpy()
        d_in = np.zeros_like(D)
        for e, (idx, xe, G, U, Hh) in enumerate(self.saved[chunk]):
            le = chunk * self.E_chunk + e
            p = self.expert_params[6 * le: 6 * le + 6]
            Wg, Wu, Wd = p[0].numpy(), p[2].numpy(), p[4].numpy()
            dy = D[idx]
            p[5].grad += torch.from_numpy(dy.sum(0, keepdims=True))
            p[4].grad += torch.from_numpy(Hh.T @ dy)
            dH = dy @ Wd.T
            sig = 1.0 / (1.0 + np.exp(-G))
            dU = dH * (G * sig)
            dG = (dH * U) * (sig * (1.0 + G * (1.0 - sig)))
            p[1].grad += torch.from_numpy(dG.sum(0, keepdims=True))
            p[0].grad += torch.from_numpy(xe.T @ dG)
            p[3].grad += torch.from_numpy(dU.sum(0, keepdims=True))
            p[2].grad += torch.from_numpy(xe.T @ dU)
            d_in[idx] = dG @ Wg.T + dU @ Wu.T
        return torch.from_numpy(d_in.astype(np.float32))

    # the two-call form (rows first, so that they can travel back while the parameter gradients are formed)
    def experts_backward_rows(self, d_out, chunk=0):
        return self.experts_backward(d_out, chunk)

    def experts_backward_params(self, chunk=0):
        pass
