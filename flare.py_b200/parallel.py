"""Context-parallel FLARE mixer: the token axis N is sharded over the ranks of a process group.

The reference has no such mode (its only parallelism is DDP replicas,
mlutils/trainer.py:195-202).  FLARE's cross-token state is only the per-latent
record (max, sum, M x D accumulator), so one small collective per direction is
enough:

  forward : local gather records -> all_gather -> log-sum-exp combine (rank
            order, deterministic) -> every rank holds the same z and L -> the
            scatter is local.
  backward: local dZ partial -> all_reduce(SUM) -> local dK, dV, dQ partial ->
            all_reduce(SUM) of dQ (the latents are replicated).

``RecordExchange`` does this with plain ``torch.distributed`` calls (NCCL on GPUs,
gloo in the CPU tests), so that the plumbing can be exercised without a GPU.
``PeerExchange`` (GPUs of one node) fuses each collective into the kernel that
consumes it: every rank writes its record (or partial sum) into a symmetric-memory
buffer, a barrier on the stream orders the writes, and the combine / reduce kernel
reads all ranks' buffers through peer pointers with plain loads over NVLink
(``flare_combine_peers``, ``flare_reduce_sum_peers``).  Ordinary loads only, no waiting
inside the library's kernels.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from . import _cabi
from ._cabi import check, lib, ptr, stream_of
from .mixer import _need_cuda, _q3, _tok, make_problem

__all__ = ["RecordExchange", "PeerExchange", "flare_mixer_context_parallel", "shard_bounds"]


def shard_bounds(n_tokens: int, world: int, rank: int, multiple: int = 1):
    """Token range [n0, n1) of `rank`: contiguous, sizes differ by at most `multiple`."""
    per = -(-n_tokens // world)
    per = -(-per // multiple) * multiple
    n0 = min(n_tokens, rank * per)
    return n0, min(n_tokens, n0 + per)


class RecordExchange:
    """The two collectives of the context-parallel mixer over one process group."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def gather_records(self, rec: torch.Tensor) -> torch.Tensor:
        """rec [B,H,M,D+2] on every rank -> [world,B,H,M,D+2], rank-major, identical on all ranks."""
        rec = rec.contiguous()
        out = torch.empty((self.world,) + tuple(rec.shape), dtype=rec.dtype, device=rec.device)
        # concatenation along dim 0 is the layout every backend accepts
        dist.all_gather_into_tensor(out.view((self.world * rec.shape[0],) + tuple(rec.shape[1:])), rec,
                                    group=self.group)
        return out

    def sum_(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t


class PeerExchange(RecordExchange):
    """The same exchanges through symmetric memory and peer loads (one node, NVLink).

    Buffers are allocated once per (name, size) and used alternately (two halves), so one barrier
    per exchange is enough: a half is rewritten two exchanges later, after every rank has passed
    the barrier of the exchange in between, which it reaches only after its reads.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        super().__init__(group)
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self._slots = {}

    def _slot(self, name: str, numel: int, device):
        key = (name, numel)
        if key not in self._slots:
            buf = self._symm.empty(2 * numel, dtype=torch.float32, device=device)
            hdl = self._symm.rendezvous(buf, group=self.group if self.group is not None else dist.group.WORLD)
            ptrs = [torch.tensor([int(p) + half * numel * 4 for p in hdl.buffer_ptrs], dtype=torch.int64, device=device)
                    for half in (0, 1)]
            self._slots[key] = dict(buf=buf, hdl=hdl, ptrs=ptrs, turn=0)
        s = self._slots[key]
        half = s["turn"] & 1
        s["turn"] += 1
        return s["buf"][half * numel:(half + 1) * numel], s["ptrs"][half], s["hdl"]

    def exchange_buffer(self, name: str, shape, device):
        """(this rank's buffer for the next exchange, device array of all ranks' pointers, barrier handle)."""
        numel = 1
        for d in shape:
            numel *= int(d)
        local, ptrs, hdl = self._slot(name, numel, device)
        return local.view(*shape), ptrs, hdl


class _CPMixerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, ex: RecordExchange, reduce_dq: bool):
        _need_cuda(q, k, v)
        q, batched = _q3(q)
        k, v = _tok(k), _tok(v)
        B, H, N, D = k.shape
        M = q.shape[-2]
        dev = k.device
        with torch.cuda.device(dev):
            st = stream_of(k)
            y = torch.empty_like(k)
            if y.stride(-1) != 1:
                y = torch.empty(k.shape, dtype=k.dtype, device=dev)
            p = make_problem(q, k, scale, v=v, y=y)
            p.n_splits = lib.flare_pick_splits(C.byref(p))
            rec = torch.empty(p.n_splits, B, H, M, D + 2, dtype=torch.float32, device=dev)
            peer = isinstance(ex, PeerExchange)
            if peer:
                merged, rec_ptrs, hdl = ex.exchange_buffer("rec", (B, H, M, D + 2), dev)
            else:
                merged = torch.empty(B, H, M, D + 2, dtype=torch.float32, device=dev)
            check(lib.flare_gather_partial(C.byref(p), ptr(q), ptr(k), ptr(v), None, ptr(rec), st), "flare_gather_partial")
            check(lib.flare_combine(C.byref(p), ptr(rec), p.n_splits, None, None, None, ptr(merged), st), "flare_combine")
            z32 = torch.empty(B, H, M, D, dtype=torch.float32, device=dev)
            lse_m = torch.empty(B, H, M, dtype=torch.float32, device=dev)
            lse_n = torch.empty(B, H, N, dtype=torch.float32, device=dev)
            if peer:
                hdl.barrier()
                check(lib.flare_combine_peers(C.byref(p), ptr(rec_ptrs), ex.world, ptr(z32), None, ptr(lse_m), None, st),
                      "flare_combine_peers")
            else:
                allrec = ex.gather_records(merged)
                check(lib.flare_combine(C.byref(p), ptr(allrec), ex.world, ptr(z32), None, ptr(lse_m), None, st), "flare_combine")
            check(lib.flare_scatter(C.byref(p), ptr(q), ptr(k), ptr(z32), None, ptr(y), ptr(lse_n), st), "flare_scatter")
        ctx.save_for_backward(q, k, v, y, z32, lse_m, lse_n)
        ctx.scale, ctx.ex, ctx.reduce_dq, ctx.batched = scale, ex, reduce_dq, batched
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, v, y, z32, lse_m, lse_n = ctx.saved_tensors
        ex = ctx.ex
        B, H, N, D = k.shape
        M = q.shape[-2]
        dev = k.device
        with torch.cuda.device(dev):
            st = stream_of(k)
            dy = _tok(dy)
            dk = torch.empty_like(k)
            dv = torch.empty_like(v)
            if dk.stride(-1) != 1:
                dk = torch.empty(k.shape, dtype=k.dtype, device=dev)
            if dv.stride(-1) != 1:
                dv = torch.empty(v.shape, dtype=v.dtype, device=dev)
            p = make_problem(q, k, ctx.scale, v=v, y=y, dy=dy, dk=dk, dv=dv)
            p.n_splits = lib.flare_pick_splits(C.byref(p))
            part = torch.empty(p.n_splits, B, H, M, D, dtype=torch.float32, device=dev)
            dz32 = torch.empty(B, H, M, D, dtype=torch.float32, device=dev)
            delta = torch.empty(B, H, N, dtype=torch.float32, device=dev)
            T = _cabi.TERM_BOTH
            check(lib.flare_bwd_dz_partial(C.byref(p), ptr(q), ptr(k), ptr(dy), None, ptr(lse_n), ptr(part), st), "flare_bwd_dz_partial")
            peer = isinstance(ex, PeerExchange)
            if peer:
                mine, ptrs, hdl = ex.exchange_buffer("dz", (B, H, M, D), dev)
                check(lib.flare_reduce_sum(ptr(part), p.n_splits, B * H * M, D, ptr(mine), st), "flare_reduce_sum")
                hdl.barrier()
                check(lib.flare_reduce_sum_peers(ptr(ptrs), ex.world, B * H * M, D, ptr(dz32), st), "flare_reduce_sum_peers")
            else:
                check(lib.flare_reduce_sum(ptr(part), p.n_splits, B * H * M, D, ptr(dz32), st), "flare_reduce_sum")
                ex.sum_(dz32)
            check(lib.flare_bwd_main(C.byref(p), T, ptr(q), ptr(k), ptr(v), ptr(dy), ptr(y), None, ptr(z32), ptr(dz32),
                                     ptr(lse_m), ptr(lse_n), ptr(dk), ptr(dv), ptr(delta), ptr(part), st),
                  "flare_bwd_main")
            dq_shape = (B, H, M, D) if ctx.batched else (H, M, D)
            n_parts, rows = (p.n_splits, B * H * M) if ctx.batched else (p.n_splits * B, H * M)
            dq = torch.empty(dq_shape, dtype=torch.float32, device=dev)
            if peer and ctx.reduce_dq:
                mine, ptrs, hdl = ex.exchange_buffer("dq", dq_shape, dev)
                check(lib.flare_reduce_sum(ptr(part), n_parts, rows, D, ptr(mine), st), "flare_reduce_sum")
                hdl.barrier()
                check(lib.flare_reduce_sum_peers(ptr(ptrs), ex.world, rows, D, ptr(dq), st), "flare_reduce_sum_peers")
            else:
                check(lib.flare_reduce_sum(ptr(part), n_parts, rows, D, ptr(dq), st), "flare_reduce_sum")
                if ctx.reduce_dq:
                    ex.sum_(dq)
        return dq.to(q.dtype), dk, dv, None, None, None


def flare_mixer_context_parallel(q, k_local, v_local, scale: float = 1.0,
                                 group: Optional[dist.ProcessGroup] = None, reduce_dq: bool = True,
                                 exchange: Optional[RecordExchange] = None):
    """Mixer over a token axis sharded across `group`: k_local, v_local are this rank's [B,H,N/R,D] shard.

    Returns this rank's y shard.  Equals ``flare_multihead_mixer`` on the concatenated
    tokens.  With ``reduce_dq`` the latent gradient is summed over the group inside the
    backward; pass False when a DDP-style reducer over the same group already does it.
    """
    ex = exchange or RecordExchange(group)
    if q.dim() == 4 and q.stride(0) == 0:
        q = q[0]
    return _CPMixerFn.apply(q, k_local, v_local, float(scale), ex, reduce_dq)
