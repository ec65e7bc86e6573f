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
buffer, the library's bounded flag barrier orders the writes, and the combine / reduce
kernel reads all ranks' buffers through peer pointers with plain loads over NVLink
(``flare_cp_mixer_fwd`` / ``flare_cp_mixer_bwd``: one call per pass).  Ordinary loads
and stores only: no multicast, no ``multimem``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from . import _cabi
from ._cabi import check, lib, ptr, stream_of
from .mixer import _need_cuda, _q3, _tok, make_problem

__all__ = ["RecordExchange", "PeerExchange", "GraphedStep", "flare_mixer_context_parallel", "shard_bounds"]


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

    Per exchange kind ("rec", "dz", "dq") and size: one symmetric allocation holding two buffers used
    alternately and an int32[world] array of arrival flags.  The ordering barrier is the library's own
    (``flare_peer_barrier``: release/acquire flags in peer memory, a bounded wait that records a status
    bit instead of hanging when a peer has left); torch supplies the allocation and the rendezvous only.
    The barrier numbers the exchanges itself on the device, so a step can be recorded in a CUDA graph and
    replayed (``GraphedStep``); every rank has to make the same sequence of calls.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        super().__init__(group)
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self._slots = {}

    def prepare(self, name: str, numel: int, device) -> None:
        """Allocate and rendezvous the buffers of one exchange kind now (a collective call: every rank makes
        it; not possible while a CUDA graph is being recorded)."""
        self._slot(name, numel, device)

    def prepare_mixer(self, B: int, H: int, M: int, D: int, device, batched_q: bool = False) -> None:
        """The three exchanges of one context-parallel mixer step."""
        self.prepare("rec", _numel(B, H, M, D + 2), device)
        self.prepare("dz", _numel(B, H, M, D), device)
        self.prepare("dq", _numel(B, H, M, D) if batched_q else _numel(H, M, D), device)

    def _slot(self, name: str, numel: int, device):
        key = (name, numel)
        s = self._slots.get(key)
        if s is None:
            pad = -(-numel // 64) * 64                                   # 256-byte aligned halves
            total = 2 * pad + 64                                          # + the flags (int32 viewed through the float buffer)
            buf = self._symm.empty(total, dtype=torch.float32, device=device)
            buf.zero_()
            grp = self.group if self.group is not None else dist.group.WORLD
            hdl = self._symm.rendezvous(buf, group=grp)
            torch.cuda.synchronize(device)
            dist.barrier(group=self.group)                                # every rank's flags are zero before anyone signals
            base = [int(x) for x in hdl.buffer_ptrs]
            i64 = dict(dtype=torch.int64, device=device)
            s = dict(buf=buf, hdl=hdl, pad=pad, turn=0,
                     bufs=[torch.tensor([b + half * pad * 4 for b in base], **i64) for half in (0, 1)],
                     flags=torch.tensor([b + 2 * pad * 4 for b in base], **i64))
            self._slots[key] = s
        return s

    def peers(self, name: str, numel: int, device) -> _cabi.FlarePeers:
        """The FlarePeers description of the next exchange of this kind (advances its number)."""
        s = self._slot(name, numel, device)
        half = s["turn"] & 1
        s["turn"] += 1
        g = _cabi.FlarePeers()
        g.rank, g.world = self.rank, self.world
        g.bufs = s["bufs"][half].data_ptr()
        g.mine = s["buf"].data_ptr() + half * s["pad"] * 4
        g.flags = s["flags"].data_ptr()
        g.epoch = 0                                                   # numbered on the device
        return g


def _numel(*dims):
    n = 1
    for d in dims:
        n *= int(d)
    return n


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
            z32 = torch.empty(B, H, M, D, dtype=torch.float32, device=dev)
            lse_m = torch.empty(B, H, M, dtype=torch.float32, device=dev)
            lse_n = torch.empty(B, H, N, dtype=torch.float32, device=dev)
            p = make_problem(q, k, scale, v=v, y=y)
            if isinstance(ex, PeerExchange):
                # one call: records -> merged record in peer-visible memory -> barrier -> combine over all
                # ranks' records (peer loads) -> scatter
                nbytes = lib.flare_fwd_workspace_bytes(C.byref(p))
                ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
                g = ex.peers("rec", _numel(B, H, M, D + 2), dev)
                check(lib.flare_cp_mixer_fwd(C.byref(p), ptr(q), ptr(k), ptr(v), None, ptr(y), ptr(z32), ptr(lse_m),
                                             ptr(lse_n), ptr(ws), nbytes, C.byref(g), st), "flare_cp_mixer_fwd")
            else:
                p.n_splits = lib.flare_pick_splits(C.byref(p))
                rec = torch.empty(p.n_splits, B, H, M, D + 2, dtype=torch.float32, device=dev)
                merged = torch.empty(B, H, M, D + 2, dtype=torch.float32, device=dev)
                check(lib.flare_gather_partial(C.byref(p), ptr(q), ptr(k), ptr(v), None, ptr(rec), st), "flare_gather_partial")
                check(lib.flare_combine(C.byref(p), ptr(rec), p.n_splits, None, None, None, ptr(merged), st), "flare_combine")
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
            dq_shape = (B, H, M, D) if ctx.batched else (H, M, D)
            dq = torch.empty(dq_shape, dtype=torch.float32, device=dev)
            if isinstance(ex, PeerExchange):
                nbytes = lib.flare_bwd_workspace_bytes(C.byref(p))
                ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
                gz = ex.peers("dz", _numel(B, H, M, D), dev)
                gq = ex.peers("dq", _numel(*dq_shape), dev) if ctx.reduce_dq else None
                check(lib.flare_cp_mixer_bwd(C.byref(p), ptr(q), ptr(k), ptr(v), ptr(dy), ptr(y), None, ptr(z32), ptr(lse_m),
                                             ptr(lse_n), ptr(dq), ptr(dk), ptr(dv), ptr(ws), nbytes, C.byref(gz),
                                             C.byref(gq) if gq is not None else None, st), "flare_cp_mixer_bwd")
            else:
                p.n_splits = lib.flare_pick_splits(C.byref(p))
                part = torch.empty(p.n_splits, B, H, M, D, dtype=torch.float32, device=dev)
                dz32 = torch.empty(B, H, M, D, dtype=torch.float32, device=dev)
                delta = torch.empty(B, H, N, dtype=torch.float32, device=dev)
                check(lib.flare_bwd_dz_partial(C.byref(p), ptr(q), ptr(k), ptr(dy), None, ptr(lse_n), ptr(part), st), "flare_bwd_dz_partial")
                check(lib.flare_reduce_sum(ptr(part), p.n_splits, B * H * M, D, ptr(dz32), st), "flare_reduce_sum")
                ex.sum_(dz32)
                check(lib.flare_bwd_main(C.byref(p), _cabi.TERM_BOTH, ptr(q), ptr(k), ptr(v), ptr(dy), ptr(y), None, ptr(z32),
                                         ptr(dz32), ptr(lse_m), ptr(lse_n), ptr(dk), ptr(dv), ptr(delta), ptr(part), st),
                      "flare_bwd_main")
                n_parts, rows = (p.n_splits, B * H * M) if ctx.batched else (p.n_splits * B, H * M)
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
    from .mixer import _autocast, _same_dtype
    ex = exchange or RecordExchange(group)
    if q.dim() == 4 and q.stride(0) == 0:
        q = q[0]
    q, k_local, v_local = _autocast(q, k_local, v_local)
    _same_dtype(q, k_local, v_local)
    return _CPMixerFn.apply(q, k_local, v_local, float(scale), ex, reduce_dq)


class GraphedStep:
    """Two consecutive calls of ``step_fn`` recorded in one CUDA graph.

    At eight ranks a million-token mixer step is a fraction of a millisecond of device work per rank,
    less than the host needs to enqueue its dozen launches through Python; replaying a recorded launch
    sequence removes that.  Two steps are recorded because a ``PeerExchange`` alternates between the two
    halves of its buffers from one exchange of a kind to the next: the pair restores the parity, so
    replays can follow each other.  ``step_fn`` must use tensors that stay alive and a ``PeerExchange`` of
    its own (prepared beforehand with ``prepare_mixer``) that nothing outside the graph uses.  No autograd
    graph of an earlier eager step over the same leaf tensors may be alive when recording starts (drop or
    detach its outputs): its gradient accumulators are tied to the stream they were created on.
    """

    def __init__(self, step_fn, warmup: int = 2):
        dev = torch.cuda.current_device()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2 * ((warmup + 1) // 2)):                 # an even number: the halves stay in step
                step_fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: another thread of the process (a communicator's watchdog polling its events)
        # may make CUDA calls while this thread records
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            step_fn()
            self.result = step_fn()
        self.steps_per_replay = 2

    def replay(self):
        self.graph.replay()
        return self.result
