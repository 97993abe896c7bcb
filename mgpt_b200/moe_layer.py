"""Host-side mirror of the reference's ``MoELayer`` over the C ABI.

Same constructor arguments and method names as the reference class
(src/main/neuralnetwork/layers/MoELayer.h:37-50): ``forward`` / ``forward_into``,
``backward`` / ``backward_into``, ``get_parameters``, ``get_footprint``,
``get_expert_counts``.  torch is used for device memory and streams only; all
arithmetic happens in ``libmgpt_moe.so``.  The parameters are FP32 device
tensors owned by this object, standing where the engine's ``Tensor`` masters
stand; gradients accumulate into ``param.grad`` like ``Tensor::add_grad``.
"""
from __future__ import annotations

import ctypes as ct

import numpy as np
import torch

from . import _lib
from ._lib import BF16, FP32, IO_BF16, IO_F32, MoeError  # noqa: F401


class MoELayer:
    def __init__(self, embed_dim: int, hidden_dim: int, num_experts: int, top_k: int, *,
                 mode: str = "bf16", device: int = 0, lb_alpha: float = 0.01, gemm_impl: int = 0):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise MoeError("mgpt_b200.MoELayer needs a CUDA device; there is no CPU path")
        self.C = embed_dim
        self.H = 4 * embed_dim if hidden_dim == -1 else hidden_dim
        self.E, self.k = num_experts, top_k
        self.mode = {"fp32": FP32, "bf16": BF16}[mode]
        self.device = torch.device("cuda", device)
        cfg = _lib.Config(embed_dim, hidden_dim, num_experts, top_k, lb_alpha, self.mode, device, gemm_impl)
        self._h = ct.c_void_p()
        _lib.check(self.lib.mgpt_moe_create(ct.byref(cfg), ct.byref(self._h)))
        self.params = []
        r, c = ct.c_int(), ct.c_int()
        for i in range(self.lib.mgpt_moe_num_params(self._h)):
            _lib.check(self.lib.mgpt_moe_param_shape(self._h, i, ct.byref(r), ct.byref(c)))
            p = torch.zeros((r.value, c.value), dtype=torch.float32, device=self.device)
            p.grad = torch.zeros_like(p)
            self.params.append(p)
        self._bind()
        self._ws = None
        self._x = None
        self._n = 0
        self.cached_out = None
        self.cached_dX = None

    # -- lifetime ----------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            self.lib.mgpt_moe_destroy(self._h)
            self._h = ct.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _bind(self):
        n = len(self.params)
        data = (ct.c_void_p * n)(*[p.data_ptr() for p in self.params])
        grad = (ct.c_void_p * n)(*[p.grad.data_ptr() for p in self.params])
        _lib.check(self.lib.mgpt_moe_bind_params(self._h, data, grad, n))

    @staticmethod
    def _stream():
        return ct.c_void_p(torch.cuda.current_stream().cuda_stream)

    # -- parameters --------------------------------------------------------
    def get_parameters(self):
        """2+6E FP32 tensors in the reference's order (MoELayer.cpp:225-236)."""
        return self.params

    def load_parameters(self, arrays):
        assert len(arrays) == len(self.params)
        for p, a in zip(self.params, arrays):
            p.copy_(torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).reshape(p.shape))
        self.sync_weights()

    def sync_weights(self):
        """Refresh the BF16 shadows after the FP32 masters changed."""
        _lib.check(self.lib.mgpt_moe_sync_weights(self._h, self._stream()))

    def zero_grad(self):
        for p in self.params:
            p.grad.zero_()

    # -- optimiser -----------------------------------------------------------
    def adamw_step(self, t: int, lr: float = 3e-4, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                   weight_decay: float = 0.01, grad_clip: float = 0.0, skip_nonfinite: bool = False):
        """One AdamW step over this layer's parameters (defaults and arithmetic of the reference's
        AdamWOptimizer, optimisers/AdamWOptimiser.h:21-36), fused with the refresh of the BF16 copies:
        no ``sync_weights`` is needed afterwards.  ``t`` counts steps from 1; the moment buffers
        ``self.opt_m`` / ``self.opt_v`` are created (zero) on first use.  ``grad_clip`` / ``skip_nonfinite``
        apply the guards of the reference's GPU kernel (utils/cuda_ops.cu:727-728) to the gradient first."""
        if getattr(self, "opt_m", None) is None:
            self.opt_m = [torch.zeros_like(p) for p in self.params]
            self.opt_v = [torch.zeros_like(p) for p in self.params]
            n = len(self.params)
            m = (ct.c_void_p * n)(*[a.data_ptr() for a in self.opt_m])
            v = (ct.c_void_p * n)(*[a.data_ptr() for a in self.opt_v])
            _lib.check(self.lib.mgpt_moe_bind_optimizer_state(self._h, m, v, n))
        if grad_clip or skip_nonfinite:
            _lib.check(self.lib.mgpt_moe_adamw_step_guarded(self._h, lr, beta1, beta2, eps, weight_decay, int(t),
                                                            float(grad_clip), int(bool(skip_nonfinite)), self._stream()))
        else:
            _lib.check(self.lib.mgpt_moe_adamw_step(self._h, lr, beta1, beta2, eps, weight_decay, int(t), self._stream()))

    # -- memory ------------------------------------------------------------
    def get_footprint(self, B: int, T: int) -> int:
        """Arena bytes for B*T tokens (the reference reports floats, MoELayer.cpp:238-251)."""
        return int(self.lib.mgpt_moe_workspace_bytes(self._h, B * T))

    def _workspace(self, n: int):
        need = int(self.lib.mgpt_moe_workspace_bytes(self._h, n))
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._ws

    def workspace_view(self, name: str, dtype, shape=None):
        """A tensor view of a named workspace buffer of the last forward."""
        off, nbytes = ct.c_size_t(), ct.c_size_t()
        _lib.check(self.lib.mgpt_moe_workspace_view(self._h, self._n, name.encode(), ct.byref(off), ct.byref(nbytes)))
        t = self._ws[off.value: off.value + nbytes.value].view(dtype)
        return t.view(shape) if shape is not None else t

    # -- compute -----------------------------------------------------------
    def _io(self, t: torch.Tensor) -> int:
        if t.dtype == torch.float32:
            return IO_F32
        if t.dtype == torch.bfloat16:
            return IO_BF16
        raise MoeError(f"unsupported token dtype {t.dtype}")

    def forward_into(self, x: torch.Tensor, out: torch.Tensor, residual: torch.Tensor = None) -> None:
        """``out = moe(x)``, or ``out = residual + moe(x)`` (the block's skip connection, TransformerBlock.cpp:44)."""
        assert x.is_cuda and x.is_contiguous() and x.shape[-1] == self.C
        assert out.shape == x.shape and out.dtype == x.dtype and out.is_contiguous()
        n = x.numel() // self.C
        ws = self._workspace(n)
        if residual is None:
            _lib.check(self.lib.mgpt_moe_forward(self._h, x.data_ptr(), out.data_ptr(), n, self._io(x),
                                                 ws.data_ptr(), ws.numel(), self._stream()))
        else:
            assert residual.shape == x.shape and residual.dtype == x.dtype and residual.is_contiguous()
            _lib.check(self.lib.mgpt_moe_forward_residual(self._h, x.data_ptr(), residual.data_ptr(), out.data_ptr(), n,
                                                          self._io(x), ws.data_ptr(), ws.numel(), self._stream()))
        self._x, self._n = x, n
        self.cached_out = out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        self.forward_into(x, out)
        return out

    def forward_inference_into(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """Forward for generation (pipeline/Generator.cpp:10-31 runs forward only and drops the activations):
        same routing and output as ``forward_into``, nothing kept for backward, a smaller workspace."""
        assert x.is_cuda and x.is_contiguous() and x.shape[-1] == self.C
        assert out.shape == x.shape and out.dtype == x.dtype and out.is_contiguous()
        n = x.numel() // self.C
        need = int(self.lib.mgpt_moe_inference_workspace_bytes(self._h, n))
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        ws = self._ws
        _lib.check(self.lib.mgpt_moe_forward_inference(self._h, x.data_ptr(), out.data_ptr(), n, self._io(x),
                                                       ws.data_ptr(), ws.numel(), self._stream()))
        self._x, self._n = None, n
        self.cached_out = out

    def forward_inference(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        self.forward_inference_into(x, out)
        return out

    # -- the block's glue: x2 = x1 + moe(rmsnorm(x1)*scale) and its backward (TransformerBlock.cpp:42-46, 80-84)
    def block_forward(self, x1: torch.Tensor, rms_scale: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
        assert x1.is_cuda and x1.is_contiguous() and x1.shape[-1] == self.C
        assert rms_scale.dtype == torch.float32 and rms_scale.numel() == self.C
        n = x1.numel() // self.C
        io = self._io(x1)
        need = int(self.lib.mgpt_moe_block_workspace_bytes(self._h, n, io))
        if getattr(self, "_bws", None) is None or self._bws.numel() < need:
            self._bws = torch.empty(need, dtype=torch.uint8, device=self.device)
        x2 = torch.empty_like(x1)
        _lib.check(self.lib.mgpt_moe_block_forward(self._h, x1.data_ptr(), rms_scale.data_ptr(), float(eps), x2.data_ptr(),
                                                   n, io, self._bws.data_ptr(), self._bws.numel(), self._stream()))
        moe_ws = int(self.lib.mgpt_moe_workspace_bytes(self._h, n))
        self._ws = self._bws[need - moe_ws: need]          # the layer's own workspace, for workspace_view()
        self._x, self._n, self._x1 = None, n, x1
        return x2

    def block_backward(self, rms_scale: torch.Tensor, dout: torch.Tensor, d_rms_scale: torch.Tensor = None) -> torch.Tensor:
        d_x1 = torch.empty_like(dout)
        _lib.check(self.lib.mgpt_moe_block_backward(
            self._h, self._x1.data_ptr(), rms_scale.data_ptr(), d_rms_scale.data_ptr() if d_rms_scale is not None else None,
            dout.data_ptr(), d_x1.data_ptr(), self._io(dout), self._bws.data_ptr(), self._bws.numel(), self._stream()))
        return d_x1

    def block_input(self) -> torch.Tensor:
        """The normalised rows the layer saw in the last block_forward (its own input), for checks."""
        n, C = self._n, self.C
        dt = self._x1.dtype
        return self._bws[: n * C * self._x1.element_size()].view(dt).view(n, C)

    # -- activation checkpointing: keep the routing of a forward, recompute without router and plan
    def save_routing(self) -> torch.Tensor:
        """Routing results and plan of the last forward, in memory of their own (the reference rewinds its
        arena between the first forward and the recompute, GPT.cpp:79-96)."""
        n = int(self.lib.mgpt_moe_routing_bytes(self._h, self._n))
        state = torch.empty(n, dtype=torch.uint8, device=self.device)
        _lib.check(self.lib.mgpt_moe_save_routing(self._h, state.data_ptr(), self._stream()))
        return state

    def recompute_into(self, x: torch.Tensor, out: torch.Tensor, routing: torch.Tensor) -> None:
        """Forward again on the same tokens with the saved routing; backward may follow."""
        assert x.is_cuda and x.is_contiguous() and x.shape[-1] == self.C
        assert out.shape == x.shape and out.dtype == x.dtype and out.is_contiguous()
        n = x.numel() // self.C
        assert routing.numel() == int(self.lib.mgpt_moe_routing_bytes(self._h, n)), "routing state of another size"
        ws = self._workspace(n)
        _lib.check(self.lib.mgpt_moe_forward_with_routing(self._h, x.data_ptr(), out.data_ptr(), n, self._io(x),
                                                          ws.data_ptr(), ws.numel(), routing.data_ptr(), self._stream()))
        self._x, self._n = x, n
        self.cached_out = out

    def backward_into(self, dout: torch.Tensor, din: torch.Tensor) -> None:
        if self._x is None:
            raise MoeError("backward before forward")
        assert dout.shape == self._x.shape and dout.dtype == self._x.dtype and dout.is_contiguous()
        assert din.shape == dout.shape and din.dtype == dout.dtype and din.is_contiguous()
        ws = self._ws
        _lib.check(self.lib.mgpt_moe_backward(self._h, self._x.data_ptr(), dout.data_ptr(), din.data_ptr(),
                                              self._io(dout), ws.data_ptr(), ws.numel(), self._stream()))
        self.cached_dX = din

    def backward(self, dout: torch.Tensor) -> torch.Tensor:
        din = torch.empty_like(dout)
        self.backward_into(dout, din)
        return din

    def get_expert_counts(self):
        """Per-expert routed rows of the last forward (MoELayer.h:39), as a list of ints."""
        buf = (ct.c_int32 * self.E)()
        _lib.check(self.lib.mgpt_moe_expert_counts(self._h, buf))
        return list(buf)

    def set_weight_grad_overwrite(self, enabled: bool) -> None:
        """Backward stores the expert weight gradients instead of adding to them (see include/mgpt_moe.h): for a
        caller that would have zeroed them first, e.g. the first micro-batch after ``zero_grad``."""
        _lib.check(self.lib.mgpt_moe_set_weight_grad_overwrite(self._h, 1 if enabled else 0))

    def check_status(self) -> None:
        """Raises MoeError if a kernel of this layer reported an error since the last check (a bounded wait
        that ran out, an expert id out of range); synchronises the stream of the last call."""
        _lib.check(self.lib.mgpt_moe_check_status(self._h, None))

    def status_bits(self) -> int:
        """The error word itself (0 = ok); reading clears it."""
        bits = ct.c_int32(0)
        self.lib.mgpt_moe_check_status(self._h, ct.byref(bits))
        return int(bits.value)

    def set_profiling(self, enabled: bool) -> None:
        _lib.check(self.lib.mgpt_moe_set_profiling(self._h, 1 if enabled else 0))

    def stage_ms(self) -> dict:
        """Milliseconds per stage of the last forward/backward pair (profiling must be on)."""
        buf = (ct.c_float * _lib.N_STAGES)()
        _lib.check(self.lib.mgpt_moe_stage_ms(self._h, buf))
        return {self.lib.mgpt_moe_stage_name(i).decode(): float(buf[i]) for i in range(_lib.N_STAGES)}

    def step_host(self, x_host: torch.Tensor, dy_host, y_host: torch.Tensor, dx_host) -> None:
        """Forward (+ backward) with host buffers; copies in and out inside the call."""
        n = x_host.numel() // self.C
        _lib.check(self.lib.mgpt_moe_step_host(
            self._h, x_host.data_ptr(), dy_host.data_ptr() if dy_host is not None else None,
            y_host.data_ptr(), dx_host.data_ptr() if dx_host is not None else None,
            n, self._io(x_host), self._stream()))


    def step_host_async(self, x_host: torch.Tensor, dy_host, y_host: torch.Tensor, dx_host) -> None:
        """The same step, enqueued without waiting: consecutive calls overlap one step's copies with another's
        kernels (two steps in flight at most).  ``y_host`` / ``dx_host`` are valid after the call after next, or
        after :meth:`step_host_wait`; all four buffers must stay alive (pinned) until then."""
        n = x_host.numel() // self.C
        _lib.check(self.lib.mgpt_moe_step_host_async(
            self._h, x_host.data_ptr(), dy_host.data_ptr() if dy_host is not None else None,
            y_host.data_ptr(), dx_host.data_ptr() if dx_host is not None else None,
            n, self._io(x_host), self._stream()))

    def step_host_wait(self) -> None:
        """Waits for every step enqueued by :meth:`step_host_async`; raises if a kernel recorded an error."""
        _lib.check(self.lib.mgpt_moe_step_host_wait(self._h))


def launch_count(reset: bool = False) -> int:
    return int(_lib.load().mgpt_moe_launch_count(1 if reset else 0))
