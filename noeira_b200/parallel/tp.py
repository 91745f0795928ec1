"""Tensor parallelism with sequence-parallel activations (Megatron layout) over the fused kernels of
csrc/tp_gemm_tcgen05.cu.

``TPLinearContext`` owns the symmetric-heap buffers one linear shape needs:
  * column-parallel (all-gather → GEMM): the rank's input shard ``x_shard [Ms, K]`` lives in symmetric memory so
    peers can pull it; ``stage [P·Ms, K]`` is local and receives the remote shards;
  * row-parallel (GEMM → reduce-scatter): ``slots [P, Ms, N]`` in symmetric memory receive every rank's partial
    tiles for this rank's rows.
A control block of epoch flags per context makes the kernels replayable from CUDA graphs.
``NcclTP`` is the library baseline (all_gather_into_tensor / reduce_scatter_tensor around the unfused GEMM) and
the oracle in tests.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import ops
from .._native import check, cuda_lib, ptr, stream_ptr
from ..ops.gemm import ACT
from ..ops.status import device_status
from .symm import SymmetricHeap


class TPLinearContext:
    def __init__(self, world: int, rank: int, ms: int, k: int, n: int, kind: str, group=None, n_fetch: int = 24,
                 spin_limit: int = 1 << 24, alloc_stage: bool = True):
        """kind = "ag" (column parallel: K = full input width, N = local output width)
                  "rs" (row parallel:    K = local input width, N = full output width).
        ``spin_limit`` bounds every device-side wait on a peer, in units of 256 ns (default about 4.3 s)."""
        if not (1 <= world <= 8 and 0 <= rank < world):
            raise ValueError(f"tensor-parallel world {world} / rank {rank}: the kernels take up to 8 ranks of one node")
        if k % 8 or n % 8:
            raise ValueError(f"K = {k} and N = {n} must be multiples of 8 (16-byte rows)")
        if 16 + world * (ms // 128) > 4096:
            raise ValueError(f"{world} x {ms // 128} row blocks exceed the control block (4080 flags)")
        assert ms % 128 == 0, "row shards are whole 128-row blocks"
        self.world, self.rank, self.ms, self.k, self.n, self.kind = world, rank, ms, k, n, kind
        self.n_fetch, self.spin_limit = n_fetch, spin_limit
        self.lib = cuda_lib()
        words = self.lib.nb_tp_ctl_words()
        nbytes = words * 4 + 4096
        if kind == "ag":
            nbytes += ms * k * 2 + 4096
        else:
            nbytes += world * ms * n * 2 + 4096
        self.heap = SymmetricHeap(nbytes, group, solo=(world == 1))
        self.ctl = self.heap.tensor(words, torch.int32)
        dev = self.ctl.local.device
        if kind == "ag":
            self.x = self.heap.tensor(ms * k, torch.bfloat16)
            self.x_shard = self.x.local.view(ms, k)
            self.stage = torch.zeros(world * ms, k, device=dev, dtype=torch.bfloat16) if alloc_stage else None
        else:
            self.slots = self.heap.tensor(world * ms * n, torch.bfloat16)
        if self.heap.world != world or self.heap.rank != rank:
            raise ValueError(f"context is rank {rank} of {world} but its process group is rank {self.heap.rank} of {self.heap.world}")
        torch.cuda.synchronize()
        if dist.is_initialized() and world > 1:
            dist.barrier(group=group)

    def gathered_input(self):
        """[P·Ms, K] view of the gathered activations after ``ag_gemm`` (own rows copied in lazily)."""
        st = getattr(self, "last_stage", self.stage)
        st[self.rank * self.ms:(self.rank + 1) * self.ms].copy_(self.x_shard)
        return st

    def ag_gemm(self, w, b_mn: bool, out=None, bias=None, act=None, stage=None):
        """Y[P·Ms, N] = act(all_gather(x_shard) · W + bias).  ``w`` is [K, N] (b_mn) or [N, K].
        ``stage`` (optional [P·Ms, K]) receives the remote shards instead of the context's own buffer, so a
        layer can keep its gathered input for the backward pass."""
        assert self.kind == "ag"
        if out is None:
            out = torch.empty(self.world * self.ms, self.n, device=w.device, dtype=torch.bfloat16)
        stage = self.stage if stage is None else stage
        self.last_stage = stage
        check(self.lib.nb_tp_ag_gemm(
            ctypes.c_int(self.world), ctypes.c_int(self.rank), self.x.ptr_table(), ptr(stage), self.ctl.ptr_table(),
            ptr(w), ptr(out), ctypes.c_int(self.ms), ctypes.c_int(self.n), ctypes.c_int(self.k), ctypes.c_int(self.k),
            ctypes.c_int(w.stride(0)), ctypes.c_int(out.stride(0)), ctypes.c_int(int(b_mn)), ptr(bias),
            ctypes.c_int(ACT[act]), ctypes.c_int(self.n_fetch), ctypes.c_uint(self.spin_limit),
            ptr(device_status(w.device)), stream_ptr()), "tp_ag_gemm")
        return out

    def gemm_rs(self, a, w, b_mn: bool, out=None, residual=None):
        """out[Ms, N] = residual + reduce_scatter(a · W).  ``a`` is the local [P·Ms, K_local] activation."""
        assert self.kind == "rs"
        if out is None:
            out = torch.empty(self.ms, self.n, device=a.device, dtype=torch.bfloat16)
        check(self.lib.nb_tp_gemm_rs(
            ctypes.c_int(self.world), ctypes.c_int(self.rank), ptr(a), ptr(w), self.slots.ptr_table(), self.ctl.ptr_table(),
            ptr(out), ptr(residual), ctypes.c_int(self.ms), ctypes.c_int(self.n), ctypes.c_int(self.k),
            ctypes.c_int(a.stride(0)), ctypes.c_int(w.stride(0)), ctypes.c_int(self.n), ctypes.c_int(out.stride(0)),
            ctypes.c_int(residual.stride(0) if residual is not None else 0), ctypes.c_int(int(b_mn)),
            ctypes.c_uint(self.spin_limit), ptr(device_status(a.device)), stream_ptr()), "tp_gemm_rs")
        return out


class NcclTP:
    """Baseline / oracle: NCCL collectives around the unfused tcgen05 GEMM."""

    def __init__(self, world, rank, group=None):
        self.world, self.rank, self.group = world, rank, group

    def ag_gemm(self, x_shard, w, b_mn, bias=None, act=None):
        full = torch.empty(self.world * x_shard.shape[0], x_shard.shape[1], device=x_shard.device, dtype=x_shard.dtype)
        if self.world > 1:
            dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        else:
            full.copy_(x_shard)
        return ops.gemm(full, w, b_mn=b_mn, bias=bias, act=act), full

    def gemm_rs(self, a, w, b_mn, residual=None):
        part = ops.gemm(a, w, b_mn=b_mn, out_dtype=torch.float32)
        ms = a.shape[0] // self.world
        out = torch.empty(ms, part.shape[1], device=a.device, dtype=torch.float32)
        if self.world > 1:
            dist.reduce_scatter_tensor(out, part, group=self.group)
        else:
            out.copy_(part)
        if residual is not None:
            out = out + residual.float()
        return out.to(torch.bfloat16)
