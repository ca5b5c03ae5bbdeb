"""Tensor-parallel all-reduce of a decode step over NVLink peer memory.

`TPCommunicator.all_reduce` stands where RowParallelLinear.forward calls `dist.all_reduce(y)`
(third_party/nanovllm/layers/linear.py:149-153); `all_reduce_add_rms_norm` also does the
`RMSNorm(x, residual)` that consumes the reduced tensor in the decoder block
(third_party/nanovllm/models/qwen3.py:146-152, layernorm.py:28-40) in the same launch.
`torch.distributed` is used once, at construction, to exchange the CUDA IPC handles of the ranks'
segments; the calls themselves involve no library collective.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist
from torch import nn

from .. import _lib as L
from ..kernel import _count

ALGO = {"auto": 0, "one_shot": 1, "two_shot": 2, "flagged_lines": 3}


class TPCommunicator:
    def __init__(self, group=None, max_bytes=8 << 20, timeout_ms=10000, device=None, large_messages=None):
        """One per (process group, stream of use).  `max_bytes`: the largest message of the
        peer-memory kernels.  Every rank of `group` must sit on its own GPU of one node.
        `large_messages="library"`: messages above `max_bytes` (prefill batches) take the
        `torch.distributed` route instead of failing."""
        self.group = group
        self.large = LibraryCommunicator(group) if large_messages == "library" else None
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_bytes = max_bytes
        lib = L.load()
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            L.check(lib.zp_comm_create(self.rank, self.world, max_bytes, timeout_ms, C.byref(self._h)),
                    "zp_comm_create")
            mine = C.create_string_buffer(64)
            L.check(lib.zp_comm_ipc_handle(self._h, mine), "zp_comm_ipc_handle")
            handles = [None] * self.world
            dist.all_gather_object(handles, mine.raw, group=group)
            for peer, h in enumerate(handles):
                if peer != self.rank:
                    L.check(lib.zp_comm_open_peer(self._h, peer, C.create_string_buffer(h, 64)),
                            "zp_comm_open_peer")
        dist.barrier(group=group)   # every segment is mapped everywhere before the first launch

    def all_reduce(self, x, out=None, algo="auto"):
        """Sum of `x` over the ranks (fp32 accumulation in rank order, one rounding); in place when
        `out` is None, as dist.all_reduce."""
        L.require_cuda(x, out)
        assert x.is_contiguous() and (out is None or (out.is_contiguous() and out.shape == x.shape))
        if self.large is not None and x.numel() * x.element_size() > self.max_bytes:
            return self.large.all_reduce(x, out)
        out = x if out is None else out
        L.check(L.load().zp_all_reduce(self._h, L.ptr(x), L.ptr(out), x.numel(), L.dtype_code(x), ALGO[algo],
                                       L.stream_ptr()), "all_reduce")
        _count(1)
        return out

    def all_reduce_add_rms_norm(self, x, residual, weight, eps, algo="auto"):
        """(RMSNorm(all_reduce(x) + residual) * weight, all_reduce(x) + residual)."""
        L.require_cuda(x, residual, weight)
        if self.large is not None and x.numel() * x.element_size() > self.max_bytes:
            return self.large.all_reduce_add_rms_norm(x, residual, weight, eps)
        H = x.shape[-1]
        x2, r2 = x.reshape(-1, H), residual.reshape(-1, H)
        assert x2.is_contiguous() and r2.is_contiguous() and weight.is_contiguous()
        assert r2.dtype == x.dtype and weight.dtype == x.dtype
        out, res_out = torch.empty_like(x2), torch.empty_like(r2)
        L.check(L.load().zp_all_reduce_add_rms_norm(self._h, L.ptr(x2), L.ptr(r2), L.ptr(weight), L.ptr(out),
                                                    L.ptr(res_out), x2.shape[0], H, float(eps),
                                                    L.dtype_code(x), ALGO[algo], L.stream_ptr()),
                "all_reduce_add_rms_norm")
        _count(1)
        return out.view(x.shape), res_out.view(x.shape)

    def sample(self, logits_shard, temperatures, noise_shard=None, seed=0):
        """tokens [B] int64, the same on every rank, from this rank's vocabulary shard
        logits_shard [B, V / world] (rank r holds columns r*V/world ..., as ParallelLMHead
        computes them) — stands where embed_head.py:27-34 gathers the shards to rank 0 and
        sampler.py:17-31 samples there."""
        L.require_cuda(logits_shard, temperatures, noise_shard)
        B, Vs = logits_shard.shape
        assert logits_shard.is_contiguous() and temperatures.dtype == torch.float32
        if noise_shard is not None:
            assert noise_shard.dtype == torch.float32 and noise_shard.is_contiguous() and noise_shard.shape == logits_shard.shape
        out = torch.empty(B, dtype=torch.int64, device=logits_shard.device)
        L.check(L.load().zp_sample_sharded(self._h, L.ptr(logits_shard), L.ptr(temperatures), L.ptr(noise_shard),
                                           L.ptr(out), B, Vs, int(seed), L.dtype_code(logits_shard),
                                           L.stream_ptr()), "sample_sharded")
        _count(1)
        return out

    def status(self) -> int:
        """0, or 1 when a device-side wait of an earlier call ran out (synchronises)."""
        code = C.c_int(0)
        L.check(L.load().zp_comm_status(self._h, C.byref(code)), "zp_comm_status")
        return code.value

    def close(self):
        if self._h:
            dist.barrier(group=self.group)   # no peer is still reading this rank's segment
            L.load().zp_comm_destroy(self._h)
            self._h = C.c_void_p()


class LibraryCommunicator:
    """The same interface on `torch.distributed` collectives (NCCL) and the stand-alone RMSNorm
    kernel — the reference's route, kept for comparisons and for groups that span nodes."""

    def __init__(self, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def all_reduce(self, x, out=None, algo="auto"):
        if out is not None:
            out.copy_(x)
            x = out
        dist.all_reduce(x, group=self.group)
        return x

    def all_reduce_add_rms_norm(self, x, residual, weight, eps, algo="auto"):
        from .step_ops import rms_norm
        dist.all_reduce(x, group=self.group)
        return rms_norm(x, weight, eps, residual)


class RowParallelLinear(nn.Module):
    """third_party/nanovllm/layers/linear.py:131-153 with the all-reduce on a TPCommunicator.
    `weight` holds this rank's [output_size, input_size / tp_size] shard."""

    def __init__(self, input_size, output_size, comm: TPCommunicator, bias=False):
        super().__init__()
        self.comm = comm
        self.tp_rank, self.tp_size = comm.rank, comm.world
        assert input_size % self.tp_size == 0
        self.weight = nn.Parameter(torch.empty(output_size, input_size // self.tp_size))
        self.bias = nn.Parameter(torch.empty(output_size)) if bias else None

    def forward(self, x):
        y = nn.functional.linear(x, self.weight, self.bias if self.tp_rank == 0 else None)
        return self.comm.all_reduce(y)
