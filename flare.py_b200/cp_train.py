"""Context-parallel training glue: a FLARE model whose token axis is sharded over the ranks of one group.

The reference trains data-parallel replicas only (mlutils/trainer.py:195-202: DDP); its train step is
mlutils/trainer.py:693-765 (autocast, loss, scaled backward, unscale, clip, step).  For point clouds too large
for one GPU (millions of points) this module keeps that step but shards every sample's N points:

* all pointwise layers (projections, norms, feed-forward) act on the local shard with replicated weights;
* the mixer exchanges its per-latent records (``flare_mixer_context_parallel``), nothing else crosses ranks
  in the forward pass;
* the loss is the global mean: every rank divides its local sum by the global element count;
* after backward the gradients of the replicated weights (the latent queries included) are summed over the
  group, in flat buckets;
* blocks may be activation-checkpointed: one [N/R, C] activation of the 16.7M-point configuration is about
  a gigabyte per rank at R = 8, and a block holds some twenty of them.
"""
from __future__ import annotations

from typing import Iterator, Optional, Tuple

import torch
import torch.distributed as dist

from .parallel import PeerExchange, RecordExchange, shard_bounds

__all__ = ["ContextParallel", "enable_context_parallel", "ShardedPointCloud", "cp_train_step"]


class ContextParallel:
    """The group a model's token axis is sharded over, and how its records are exchanged
    ("peer": symmetric memory + peer loads on one node; "collective": all_gather / all_reduce)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, exchange: str = "collective",
                 bucket_bytes: int = 64 << 20):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.exchange = PeerExchange(group) if exchange == "peer" else RecordExchange(group)
        self.bucket_bytes = bucket_bytes

    def global_count(self, local_count: int, device) -> int:
        t = torch.tensor([local_count], dtype=torch.int64, device=device)
        dist.all_reduce(t, group=self.group)
        return int(t.item())

    def reduce_gradients(self, model: torch.nn.Module) -> None:
        """Sum every parameter gradient over the group (the weights are replicated, each rank saw its tokens)."""
        params = [p for p in model.parameters() if p.grad is not None]
        bucket, size = [], 0
        for p in params + [None]:
            if p is not None:
                bucket.append(p)
                size += p.grad.numel() * p.grad.element_size()
            if bucket and (p is None or size >= self.bucket_bytes):
                by_dtype = {}
                for b in bucket:
                    by_dtype.setdefault(b.grad.dtype, []).append(b)
                for group_params in by_dtype.values():
                    flat = torch.cat([b.grad.reshape(-1) for b in group_params])
                    dist.all_reduce(flat, group=self.group)
                    off = 0
                    for b in group_params:
                        n = b.grad.numel()
                        b.grad.copy_(flat[off:off + n].view_as(b.grad))
                        off += n
                bucket, size = [], 0


def enable_context_parallel(model: torch.nn.Module, cp: Optional[ContextParallel], checkpoint_blocks: bool = False):
    """Route every FLARE mixer of `model` through the context-parallel exchange of `cp` (None switches it
    off again) and, optionally, recompute each block in the backward pass instead of keeping its activations."""
    from .modules import FLAREModel, _FlareCore
    for m in model.modules():
        if isinstance(m, _FlareCore):
            m.cp = cp
        if isinstance(m, FLAREModel):
            m.checkpoint_blocks = bool(checkpoint_blocks)
    return model


class ShardedPointCloud:
    """Synthetic point clouds, generated shard by shard: rank r makes only its N/R points of every sample, from
    a seed that depends on (seed, sample, rank) -- the whole cloud never exists anywhere.  Coordinates ~ U[0,1)^3
    plus `fields` input channels ~ N(0,1); targets ~ N(0,1)."""

    def __init__(self, n_points: int, fields: int, out_dim: int, rank: int, world: int, seed: int = 0,
                 device="cuda", dtype=torch.float32, multiple: int = 128):
        self.n0, self.n1 = shard_bounds(n_points, world, rank, multiple)
        self.n_points, self.fields, self.out_dim = n_points, fields, out_dim
        self.rank, self.seed, self.device, self.dtype = rank, seed, torch.device(device), dtype

    def sample(self, index: int, batch: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
        g = torch.Generator(device=self.device).manual_seed(self.seed * 1_000_003 + index * 1009 + self.rank)
        n = self.n1 - self.n0
        coords = torch.rand(batch, n, 3, generator=g, device=self.device, dtype=self.dtype)
        fields = torch.randn(batch, n, self.fields, generator=g, device=self.device, dtype=self.dtype)
        target = torch.randn(batch, n, self.out_dim, generator=g, device=self.device, dtype=self.dtype)
        return torch.cat([coords, fields], dim=-1), target

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        i = 0
        while True:
            yield self.sample(i)
            i += 1


def cp_train_step(model, opt, x_local, target_local, cp: ContextParallel, scaler=None, autocast_dtype=None,
                  clip_grad_norm: Optional[float] = None):
    """One step of mlutils/trainer.py:693-765 on a token-sharded sample: returns the global mean-squared error."""
    model.train()
    dev = x_local.device
    n_global = cp.global_count(target_local.numel(), dev)
    if autocast_dtype is not None:
        with torch.autocast(dev.type, dtype=autocast_dtype):
            y = model(x_local)
    else:
        y = model(x_local)
    loss_local = (y.float() - target_local.float()).square().sum() / n_global      # this rank's share of the global mean
    if scaler is not None:
        scaler.scale(loss_local).backward()
    else:
        loss_local.backward()
    cp.reduce_gradients(model)
    if scaler is not None:
        scaler.unscale_(opt)
    if clip_grad_norm is not None:
        torch.nn.utils.clip_grad_norm_(model.parameters(), clip_grad_norm)
    if scaler is not None:
        scaler.step(opt)
        scaler.update()
    else:
        opt.step()
    opt.zero_grad(set_to_none=True)
    loss = loss_local.detach().clone()
    dist.all_reduce(loss, group=cp.group)
    return loss
