"""Symmetric (peer-mapped) buffers and the host side of the fused tensor-parallel kernels.

One process per GPU; every rank allocates the same set of buffers with ``cudaMalloc`` inside
the kernel library, publishes their CUDA-IPC handles through ``torch.distributed`` and maps
its peers' buffers, so each rank holds a table of ``world`` base pointers per buffer. The
fused kernels (``csrc/kernels/gemm_bf16.cu`` scatter epilogue / gather prologue and
``csrc/kernels/tp_fused.cu``) read and write those pointers directly over NVLink with plain
loads, stores and system-scope reductions.

The flow per transformer block (rows = tokens, split into contiguous shards per rank):

    o_proj/down GEMM  --scatter epilogue-->  owner's receive slots      (GEMM + reduce-scatter)
    reduce + residual + RMSNorm on the shard --stores--> every rank     (+ all-gather)
    qkv/gate_up GEMM  waits for the gathered rows of each tile          (all-gather + GEMM)
"""
from __future__ import annotations

import ctypes
import os

import torch

from ..ops import _lib
from ..ops._lib import check, lib, ptr, stream_ptr

MAX_WORLD = 8


class B200TpGemm(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("rows_per_rank", ctypes.c_int),
                ("scatter", ctypes.c_int), ("gather", ctypes.c_int),
                ("peer_recv", ctypes.c_void_p * 8), ("peer_rs_flags", ctypes.c_void_p * 8),
                ("recv_parity_stride", ctypes.c_longlong), ("rs_flag_parity_stride", ctypes.c_int),
                ("a_alt", ctypes.c_void_p),
                ("ag_flags", ctypes.c_void_p), ("ag_flag_parity_stride", ctypes.c_int),
                ("op_counter", ctypes.c_void_p), ("out_f32", ctypes.c_int),
                ("scatter_splits", ctypes.c_int), ("act_fuse", ctypes.c_int)]


class B200TpReduce(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("rows_per_rank", ctypes.c_int),
                ("M", ctypes.c_int), ("H", ctypes.c_int), ("recv", ctypes.c_void_p),
                ("recv_parity_stride", ctypes.c_longlong), ("rs_flags", ctypes.c_void_p),
                ("rs_flag_parity_stride", ctypes.c_int), ("expected_rs", ctypes.c_int),
                ("nsrc", ctypes.c_int),
                ("residual", ctypes.c_void_p), ("norm_w", ctypes.c_void_p),
                ("eps", ctypes.c_float), ("gemma", ctypes.c_int),
                ("peer_x", ctypes.c_void_p * 8), ("x_parity_stride", ctypes.c_longlong),
                ("peer_ag_flags", ctypes.c_void_p * 8), ("ag_flag_parity_stride", ctypes.c_int),
                ("ag_groups", ctypes.c_int), ("op_counter", ctypes.c_void_p),
                ("done_counter", ctypes.c_void_p)]


class B200TpOneShot(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("M", ctypes.c_int), ("H", ctypes.c_int),
                ("peer_partial", ctypes.c_void_p * 8), ("peer_flags", ctypes.c_void_p * 8),
                ("mc_partial", ctypes.c_void_p), ("seq", ctypes.c_void_p), ("done_counter", ctypes.c_void_p),
                ("residual", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("eps", ctypes.c_float), ("gemma", ctypes.c_int)]


def _declare():
    P, I, L, F, Z = _lib.P, _lib.I, _lib.L, _lib.F, _lib.Z
    _lib.declare("b200_tp_oneshot_allreduce_norm", [ctypes.POINTER(B200TpOneShot), P], I)
    _lib.declare("b200_symm_alloc", [Z], P)
    _lib.declare("b200_symm_free", [P], I)
    _lib.declare("b200_ipc_get_handle", [P, P], I)
    _lib.declare("b200_ipc_open", [P], P)
    _lib.declare("b200_ipc_close", [P], I)
    _lib.declare("b200_memset_async", [P, I, Z, P], I)
    _lib.declare("b200_gemm_bf16_tp", [P, I, P, I, P, I, I, I, I, ctypes.POINTER(B200TpGemm),
                                       ctypes.POINTER(ctypes.c_int), P], I)
    _lib.declare("b200_tp_reduce_norm_gather", [ctypes.POINTER(B200TpReduce), P], I)
    _lib.declare("b200_tp_gather_rows", [P, L, I, P, I, P, I, P, I, P, P], I)
    _lib.declare("b200_tp_first_norm", [P, P, P, P, L, P, I, I, P, I, I, I, I, I, F, I, P, P, P], I)


class _DevPtrView:
    """Wraps a raw device pointer so torch can view it (``torch.as_tensor(view, device=...)``)."""

    def __init__(self, p: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (p, False),
                                         "version": 3, "strides": None}


class SymmetricBuffer:
    """``nbytes`` of device memory allocated on every rank; ``ptrs[r]`` is rank r's copy as
    seen from this process (``ptrs[rank]`` is the local one)."""

    def __init__(self, comm, nbytes: int, device: torch.device):
        _declare()
        l = lib()
        self.nbytes = nbytes
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.local = l.b200_symm_alloc(nbytes)
        if not self.local:
            raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed")
        h = (ctypes.c_char * 64)()
        check(l.b200_ipc_get_handle(self.local, h), "ipc_get_handle")
        handles = comm.all_gather_object(bytes(h)) if hasattr(comm, "all_gather_object") else [bytes(h)]
        self.ptrs = []
        self._opened = []
        for r, hb in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local)
            else:
                p = l.b200_ipc_open(ctypes.c_char_p(hb))
                if not p:
                    raise RuntimeError(f"cannot map rank {r}'s buffer (no peer access?)")
                self._opened.append(p)
                self.ptrs.append(p)
        self.tensor = torch.as_tensor(_DevPtrView(self.local, nbytes), device=device)

    def close(self):
        l = lib()
        for p in self._opened:
            l.b200_ipc_close(p)
        self._opened = []
        if self.local:
            l.b200_symm_free(self.local)
            self.local = None


def _round_up(a, b):
    return (a + b - 1) // b * b


class OneShotAllReduce:
    """Decode-sized batches: the GEMM writes this rank's partial rows into one of two peer-readable
    buffers and one kernel per all-reduce site reads every rank's partial, sums in rank order, adds
    the residual and applies RMSNorm (``tp_oneshot_allreduce_norm_kernel``). The two buffers
    alternate with the parity of the op within the forward pass (host-known, so the pointers a CUDA
    graph captures stay right); the arrival counters are monotonic and live on the device."""

    def __init__(self, comm, device, hidden: int, max_tokens: int):
        self.comm, self.device, self.H = comm, device, hidden
        self.world, self.rank = comm.world, comm.rank
        self.max_tokens = max_tokens
        self.mc_base = 0
        self.partial = None
        if os.environ.get("B200_TP_NVLS", "0") == "1" and self.world > 1:
            self._init_nvls(device, 2 * max_tokens * hidden)
        if self.partial is None:
            self.partial = SymmetricBuffer(comm, 2 * max_tokens * hidden * 2, device)
            self.partial_ptrs = self.partial.ptrs
            self._views = self.partial.tensor.view(torch.bfloat16).view(2, max_tokens, hidden)
        # [world arrival counters | pad | seq | done]
        self.flags = SymmetricBuffer(comm, 256, device)
        self.op = 0                       # ops issued in the current forward pass
        comm.barrier()

    def _init_nvls(self, device, numel: int) -> None:
        """NVLS variant (B200_TP_NVLS=1, chosen here, at set-up): the partial buffers live in
        symmetric memory that is also bound to an NVSwitch multicast object, and the kernel sums all
        ranks' rows with one ``multimem.ld_reduce`` per 16 bytes. The allocation, the handle
        exchange and the multicast binding are torch's (``torch.distributed._symmetric_memory``).
        Falls back to peer loads when the system offers no multicast. A rank must not exit while
        the buffer is bound (peers' GPUs would see NVLink faults): ``close()`` is collective."""
        try:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            t = symm_mem.empty(numel, dtype=torch.bfloat16, device=device)
            hdl = symm_mem.rendezvous(t, dist.group.WORLD)
            mc = int(hdl.multicast_ptr or 0)      # 0 when the system offers no multicast
        except Exception as e:          # no multicast on this system / this torch build
            print(f"[tp_fused] NVLS unavailable, using peer loads: {e}", flush=True)
            return
        if not mc:
            return
        self._symm_tensor, self._symm_handle = t, hdl
        self.mc_base = mc
        self.partial = t                 # keeps the allocation alive; no IPC buffer to close
        self.partial_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._views = t.view(2, self.max_tokens, self.H)

    def begin_forward(self) -> None:
        self.op = 0

    def partial_out(self, T: int) -> torch.Tensor:
        """Where the next partial-product GEMM must write its ``[T, H]`` output."""
        return self._views[self.op & 1][:T]

    def allreduce_norm(self, T: int, weight, eps: float, gemma: bool, residual, out: torch.Tensor):
        """Sum of all ranks' partials (+ ``residual``, updated in place) -> RMSNorm -> ``out``;
        ``weight`` None leaves the plain sum in ``out``."""
        a = B200TpOneShot()
        a.world, a.rank, a.M, a.H = self.world, self.rank, T, self.H
        off = (self.op & 1) * self.max_tokens * self.H * 2
        for r in range(self.world):
            a.peer_partial[r] = self.partial_ptrs[r] + off
            a.peer_flags[r] = self.flags.ptrs[r]
        a.mc_partial = self.mc_base + off if self.mc_base else None
        a.seq = self.flags.local + 128
        a.done_counter = self.flags.local + 192
        a.residual = ptr(residual)
        a.norm_w = ptr(weight)
        a.out = ptr(out)
        a.eps, a.gemma = eps, int(gemma)
        check(lib().b200_tp_oneshot_allreduce_norm(ctypes.byref(a), stream_ptr()), "tp_oneshot")
        self.op += 1
        return out

    def close(self):
        if self.mc_base:
            torch.cuda.synchronize()
            self.comm.barrier()          # nobody unbinds while a peer may still read through the switch
            self._symm_handle = self._symm_tensor = self.partial = None
        else:
            self.partial.close()
        self.flags.close()


class TpFusedContext:
    """Buffers + launch helpers of the fused path for one model (hidden size ``H``)."""

    def __init__(self, comm, device, hidden: int, max_tokens: int):
        self.comm, self.device, self.H = comm, device, hidden
        self.world, self.rank = comm.world, comm.rank
        self.max_tokens = _round_up(max_tokens, 32)
        self.rpr_max = _round_up(-(-self.max_tokens // self.world), 32)
        H, W = hidden, self.world
        self.recv_parity = W * self.rpr_max * H                     # elements
        self.x_parity = self.max_tokens * H
        self.rs_groups = self.rpr_max // 32
        self.ag_groups = self.max_tokens // 32
        self.recv = SymmetricBuffer(comm, 2 * self.recv_parity * 2, device)
        self.x_full = SymmetricBuffer(comm, 2 * self.x_parity * 2, device)
        # counters: [rs 2 x groups | ag 2 x groups | op counter | done counter]
        self.n_rs, self.n_ag = 2 * self.rs_groups, 2 * self.ag_groups
        self.flags = SymmetricBuffer(comm, (self.n_rs + self.n_ag + 64) * 4, device)
        self.residual = torch.zeros((self.rpr_max, H), dtype=torch.bfloat16, device=device)
        self._x_view = self.x_full.tensor.view(torch.bfloat16).view(2, self.max_tokens, H)
        comm.barrier()

    # pointer arithmetic helpers
    def _rs_flags(self, r):
        return self.flags.ptrs[r]

    def _ag_flags(self, r):
        return self.flags.ptrs[r] + self.n_rs * 4

    def _op_counter(self):
        return self.flags.local + (self.n_rs + self.n_ag) * 4

    def _done_counter(self):
        return self.flags.local + (self.n_rs + self.n_ag + 16) * 4

    def rows_per_rank(self, T: int) -> int:
        return _round_up(-(-T // self.world), 32)

    def x_gathered_device_parity(self, T: int) -> torch.Tensor:
        """The gathered activations the last fused op wrote. Reads the device op counter, so it
        synchronises: for tests and the final-norm row gather outside CUDA graphs only."""
        k = int(self.flags.tensor.view(torch.int32)[self.n_rs + self.n_ag].item())
        return self._x_view[(k - 1) & 1][:T]

    # ---- launches -------------------------------------------------------------------------
    def first_norm(self, hidden: torch.Tensor, weight: torch.Tensor, eps: float, gemma: bool):
        T = hidden.shape[0]
        rpr = self.rows_per_rank(T)
        check(lib().b200_tp_first_norm(
            ptr(hidden), ptr(self.residual), ptr(weight), self.x_full.local, self.x_parity,
            self._ag_flags(self.rank), self.ag_groups, self.ag_groups, self._rs_flags(self.rank),
            self.rs_groups, self.rank, rpr, T, self.H, eps, int(gemma), self._op_counter(),
            self._done_counter(), stream_ptr()), "tp_first_norm")

    def gemm_scatter(self, a: torch.Tensor, w: torch.Tensor) -> int:
        """Partial ``a @ w^T`` (K sharded) scattered row-wise to the owners. Returns the arrival
        count the following reduce must wait for."""
        T, K = a.shape
        N = w.shape[0]
        assert N == self.H
        d = B200TpGemm()
        d.world, d.rank, d.rows_per_rank = self.world, self.rank, self.rows_per_rank(T)
        d.scatter, d.gather = 1, 0
        for r in range(self.world):
            d.peer_recv[r] = self.recv.ptrs[r]
            d.peer_rs_flags[r] = self._rs_flags(r)
        d.recv_parity_stride = self.recv_parity
        d.rs_flag_parity_stride = self.rs_groups
        d.op_counter = self._op_counter()
        # small batches: split K so that more than N/128 CTAs stream the weight shard; every
        # (rank, split) pair owns a source slot in the receive buffer
        splits = 1
        if T <= 256:
            tiles_n = -(-N // 128)
            kblocks = -(-K // 64)
            splits = max(1, min(_lib.lib().b200_num_sms() // tiles_n, kblocks // 4,
                                self.rpr_max // d.rows_per_rank, 8))
            kb_per = -(-kblocks // splits)
            splits = -(-kblocks // kb_per)
        d.scatter_splits = splits
        self._last_nsrc = self.world * splits
        exp = ctypes.c_int(0)
        check(lib().b200_gemm_bf16_tp(ptr(a), a.stride(0), ptr(w), w.stride(0), None, N, T, N, K,
                                      ctypes.byref(d), ctypes.byref(exp), stream_ptr()),
              "gemm_scatter")
        return exp.value

    def reduce_norm_gather(self, T: int, expected_rs: int, weight: torch.Tensor, eps: float,
                           gemma: bool, use_residual: bool = True, nsrc: int = 0):
        a = B200TpReduce()
        a.world, a.rank, a.rows_per_rank, a.M, a.H = (self.world, self.rank, self.rows_per_rank(T),
                                                      T, self.H)
        a.recv = self.recv.local
        a.recv_parity_stride = self.recv_parity
        a.rs_flags = self._rs_flags(self.rank)
        a.rs_flag_parity_stride = self.rs_groups
        a.expected_rs = expected_rs
        a.nsrc = nsrc if nsrc else getattr(self, "_last_nsrc", self.world)
        a.residual = ptr(self.residual) if use_residual else None
        a.norm_w = ptr(weight)
        a.eps, a.gemma = eps, int(gemma)
        for r in range(self.world):
            a.peer_x[r] = self.x_full.ptrs[r]
            a.peer_ag_flags[r] = self._ag_flags(r)
        a.x_parity_stride = self.x_parity
        a.ag_flag_parity_stride = self.ag_groups
        a.ag_groups = self.ag_groups
        a.op_counter = self._op_counter()
        a.done_counter = self._done_counter()
        check(lib().b200_tp_reduce_norm_gather(ctypes.byref(a), stream_ptr()), "tp_reduce")

    def gemm_gather(self, T: int, w: torch.Tensor, out: torch.Tensor, wait: bool = True,
                    act_fuse: int = 0):
        """``out = x_gathered @ w^T`` where the producer waits for the gathered rows tile by tile.
        ``act_fuse`` (activation kind + 1, T > 256 only): ``w`` holds [128 gate | 128 up] row blocks
        and ``out[T, N / 2] = act(gate) * up`` comes out of the epilogue."""
        x = self._x_view[0][:T]      # parity-0 copy; the kernel switches to a_alt by device parity
        d = B200TpGemm()
        d.world, d.rank, d.rows_per_rank = self.world, self.rank, self.rows_per_rank(T)
        d.scatter, d.gather = 0, 1 if wait else 0
        d.a_alt = self._x_view[1].data_ptr()
        d.ag_flags = self._ag_flags(self.rank)
        d.ag_flag_parity_stride = self.ag_groups
        d.op_counter = self._op_counter()
        d.out_f32 = 1 if out.dtype == torch.float32 else 0
        d.act_fuse = act_fuse
        check(lib().b200_gemm_bf16_tp(ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(out),
                                      out.stride(0), T, w.shape[0], x.shape[1], ctypes.byref(d),
                                      None, stream_ptr()), "gemm_gather")
        return out

    def gather_rows(self, T: int, idx: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``out[i] = x_gathered[idx[i]]`` (rows that go through the lm_head)."""
        check(lib().b200_tp_gather_rows(self.x_full.local, self.x_parity, self.H, ptr(idx),
                                        idx.numel(), self._ag_flags(self.rank), self.ag_groups,
                                        self._op_counter(), T, ptr(out), stream_ptr()),
              "tp_gather_rows")
        return out

    def gather_all(self, T: int, out: torch.Tensor) -> torch.Tensor:
        """Local copy of all ``T`` gathered rows (waits for every group to arrive)."""
        if not hasattr(self, "_arange") or self._arange.numel() < T:
            self._arange = torch.arange(self.max_tokens, dtype=torch.int32, device=self.device)
        return self.gather_rows(T, self._arange[:T], out)

    def native_ctx(self, final_norm: torch.Tensor):
        """The buffer table as the native layer-stack entry takes it (built once)."""
        c = getattr(self, "_native", None)
        if c is None or c.final_norm != final_norm.data_ptr():
            from ..ops.layer import TpLayers
            c = TpLayers()
            c.world, c.rank, c.rpr_max, c.max_tokens = self.world, self.rank, self.rpr_max, self.max_tokens
            for r in range(self.world):
                c.recv[r] = self.recv.ptrs[r]
                c.rs_flags[r] = self._rs_flags(r)
                c.x_full[r] = self.x_full.ptrs[r]
                c.ag_flags[r] = self._ag_flags(r)
            c.op_counter, c.done_counter = self._op_counter(), self._done_counter()
            c.residual = self.residual.data_ptr()
            c.final_norm = final_norm.data_ptr()
            self._native = c
        return c

    def close(self):
        for b in (self.recv, self.x_full, self.flags):
            b.close()
        if getattr(self, "oneshot", None) is not None:
            self.oneshot.close()
