"""Host side of the FLARE gather-scatter mixer: the reference's Python surface over the C ABI.

``flare_multihead_mixer(q, k, v)`` has the signature and meaning of the function
of the same name in the reference's README.md:37-53 (the two SDPA calls inside
``FLARE.forward``, pdebench/models/flare.py:136-138 and
lra/models/backends.py:603-606) and is differentiable.  ``flare_gather`` and
``flare_scatter`` expose the two calls separately for callers that touch the
latents in between (pdebench/models/flare_ablations.py:93-132).

PyTorch supplies device memory, streams and autograd bookkeeping; all
arithmetic happens in libflare_b200.so.  CPU tensors are rejected: there is no
fallback path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _cabi
from ._cabi import FlareProblem, check, lib, ptr, stream_of

__all__ = [
    "flare_multihead_mixer", "flare_gather", "flare_scatter",
    "mixer_forward", "mixer_backward", "gather_forward", "gather_backward", "scatter_forward", "scatter_backward",
    "make_problem", "set_kernel_path", "device_status", "pass_counts",
]


def set_kernel_path(path: str) -> str:
    """'auto' (tensor-core kernels where the shape allows) or 'simt'; returns the previous one."""
    code = {"auto": 0, "simt": 1, "tc_exact": 2}[path]
    prev = lib.flare_set_path(code)
    return {0: "auto", 1: "simt", 2: "tc_exact"}[prev]


def device_status(clear: bool = True) -> int:
    """Status word of the current device (synchronises): non-zero if a tensor-core kernel gave up on a
    bounded wait since the word was last cleared, in which case that kernel's output is not valid."""
    out = C.c_int(0)
    check(lib.flare_device_status(C.byref(out), 1 if clear else 0), "flare_device_status")
    return out.value


def pass_counts():
    """(tensor-core passes, fp32-kernel passes) enqueued by this process so far."""
    tc, simt = C.c_longlong(0), C.c_longlong(0)
    check(lib.flare_pass_counts(C.byref(tc), C.byref(simt)), "flare_pass_counts")
    return tc.value, simt.value


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flare_b200 runs on CUDA tensors only (sm_100a); got a CPU tensor")


def _tok(t: torch.Tensor) -> torch.Tensor:
    """A [B,H,N,D] tensor the kernels can address: unit stride on D, 16-byte aligned rows, no broadcast
    (stride 0) dimension -- a TMA tensor map cannot describe one."""
    e = t.element_size()
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and \
        all((s * e) % 16 == 0 and (s != 0 or n == 1) for s, n in zip(t.stride()[:-1], t.shape[:-1]))
    return t if ok else t.contiguous()


def _q3(q: torch.Tensor) -> Tuple[torch.Tensor, bool]:
    """q as [H,M,D] (shared latents) or [B,H,M,D]; an expand()-ed batch is folded back."""
    if q.dim() == 4 and q.stride(0) == 0:
        q = q[0]
    if q.dim() not in (3, 4):
        raise ValueError(f"q must be [H,M,D] or [B,H,M,D], got {tuple(q.shape)}")
    return _tok(q), q.dim() == 4


def make_problem(q, k, scale: float, n_splits: int = 0, v=None, y=None, dy=None, dk=None, dv=None,
                 dropout_p: float = 0.0, dropout_seed: int = 0) -> FlareProblem:
    B, H, N, D = k.shape
    if q.dim() == 3:
        Hq, M, Dq = q.shape
        qs = (0, q.stride(0), q.stride(1))
    else:
        Bq, Hq, M, Dq = q.shape
        if Bq != B:
            raise ValueError("q batch does not match k")
        qs = (q.stride(0), q.stride(1), q.stride(2))
    if (Hq, Dq) != (H, D):
        raise ValueError(f"q {tuple(q.shape)} does not match k {tuple(k.shape)}")
    if k.dtype not in _cabi.DTYPE_CODE:
        raise TypeError(f"unsupported dtype {k.dtype}")
    p = FlareProblem()
    p.B, p.H, p.N, p.M, p.D = B, H, N, M, D
    p.dtype = _cabi.DTYPE_CODE[k.dtype]
    p.scale = float(scale)
    p.n_splits = int(n_splits)
    p.dropout_p = float(dropout_p)
    p.dropout_seed = int(dropout_seed) & 0xFFFFFFFFFFFFFFFF
    p.q_stride[:] = qs
    p.k_stride[:] = k.stride()[:3]
    for name, t in (("v_stride", v), ("y_stride", y), ("dy_stride", dy), ("dk_stride", dk), ("dv_stride", dv)):
        if t is not None:
            getattr(p, name)[:] = t.stride()[:3]
    return p


def _mask_u8(key_mask, B, N, device):
    if key_mask is None:
        return None
    if tuple(key_mask.shape) != (B, N):
        raise ValueError(f"key_mask must be [B,N]={B, N}, got {tuple(key_mask.shape)}")
    return key_mask.to(device=device, dtype=torch.uint8).contiguous()


def mixer_forward(q, k, v, scale=1.0, key_mask=None, dropout_p=0.0, dropout_seed=0):
    """y, z32[B,H,M,D], lse_m[B,H,M], lse_n[B,H,N] via flare_mixer_fwd."""
    _need_cuda(q, k, v)
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k, v must share a dtype")
    q, _ = _q3(q)
    k, v = _tok(k), _tok(v)
    B, H, N, D = k.shape
    M = q.shape[-2]
    mask = _mask_u8(key_mask, B, N, k.device)
    with torch.cuda.device(k.device):
        y = torch.empty_like(k)
        if y.stride(-1) != 1:
            y = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        z32 = torch.empty(B, H, M, D, dtype=torch.float32, device=k.device)
        lse_m = torch.empty(B, H, M, dtype=torch.float32, device=k.device)
        lse_n = torch.empty(B, H, N, dtype=torch.float32, device=k.device)
        p = make_problem(q, k, scale, v=v, y=y, dropout_p=dropout_p, dropout_seed=dropout_seed)
        nbytes = lib.flare_fwd_workspace_bytes(C.byref(p))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=k.device)
        check(lib.flare_mixer_fwd(C.byref(p), ptr(q), ptr(k), ptr(v), ptr(mask), ptr(y), ptr(z32),
                                  ptr(lse_m), ptr(lse_n), ptr(ws), nbytes, stream_of(k)), "flare_mixer_fwd")
    return y, z32, lse_m, lse_n


def mixer_backward(q, k, v, dy, y, z32, lse_m, lse_n, scale=1.0, key_mask=None, dropout_p=0.0, dropout_seed=0):
    """dq (fp32, [H,M,D] or [B,H,M,D]), dk, dv via flare_mixer_bwd."""
    _need_cuda(q, k, v, dy, y)
    q, batched = _q3(q)
    k, v, dy, y = _tok(k), _tok(v), _tok(dy), _tok(y)
    B, H, N, D = k.shape
    M = q.shape[-2]
    mask = _mask_u8(key_mask, B, N, k.device)
    with torch.cuda.device(k.device):
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        if dk.stride(-1) != 1:
            dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        if dv.stride(-1) != 1:
            dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        dq = torch.empty((B, H, M, D) if batched else (H, M, D), dtype=torch.float32, device=k.device)
        p = make_problem(q, k, scale, v=v, y=y, dy=dy, dk=dk, dv=dv, dropout_p=dropout_p, dropout_seed=dropout_seed)
        nbytes = lib.flare_bwd_workspace_bytes(C.byref(p))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=k.device)
        check(lib.flare_mixer_bwd(C.byref(p), ptr(q), ptr(k), ptr(v), ptr(dy), ptr(y), ptr(mask), ptr(z32),
                                  ptr(lse_m), ptr(lse_n), ptr(dq), ptr(dk), ptr(dv), ptr(ws), nbytes,
                                  stream_of(k)), "flare_mixer_bwd")
    return dq, dk, dv


# ------------------------------------------------------------------------------------
# the two SDPA calls as separate passes (host side of flare_gather / flare_scatter)
# ------------------------------------------------------------------------------------
def _dq_from_parts(p, part, B, H, M, D, batched, st):
    dq = torch.empty((B, H, M, D) if batched else (H, M, D), dtype=torch.float32, device=part.device)
    if batched:
        check(lib.flare_reduce_sum(ptr(part), p.n_splits, B * H * M, D, ptr(dq), st), "flare_reduce_sum")
    else:
        check(lib.flare_reduce_sum(ptr(part), p.n_splits * B, H * M, D, ptr(dq), st), "flare_reduce_sum")
    return dq


def gather_forward(q, k, v, scale=1.0, key_mask=None):
    """z (input dtype), z32, lse_m[B,H,M] via flare_gather_partial + flare_combine."""
    _need_cuda(q, k, v)
    q, _ = _q3(q)
    k, v = _tok(k), _tok(v)
    B, H, N, D = k.shape
    M = q.shape[-2]
    dev = k.device
    mask = _mask_u8(key_mask, B, N, dev)
    with torch.cuda.device(dev):
        z32 = torch.empty(B, H, M, D, dtype=torch.float32, device=dev)
        z = torch.empty(B, H, M, D, dtype=k.dtype, device=dev)
        lse_m = torch.empty(B, H, M, dtype=torch.float32, device=dev)
        p = make_problem(q, k, scale, v=v)
        p.n_splits = lib.flare_pick_splits(C.byref(p))
        rec = torch.empty(p.n_splits, B, H, M, D + 2, dtype=torch.float32, device=dev)
        st = stream_of(k)
        check(lib.flare_gather_partial(C.byref(p), ptr(q), ptr(k), ptr(v), ptr(mask), ptr(rec), st), "flare_gather_partial")
        check(lib.flare_combine(C.byref(p), ptr(rec), p.n_splits, ptr(z32), ptr(z), ptr(lse_m), None, st), "flare_combine")
    return z, z32, lse_m


def gather_backward(q, k, v, dz, z32, lse_m, scale=1.0, key_mask=None):
    """dq (fp32), dk, dv of the gather alone (term 1 of the backward)."""
    q, batched = _q3(q)
    k, v = _tok(k), _tok(v)
    B, H, N, D = k.shape
    M = q.shape[-2]
    mask = _mask_u8(key_mask, B, N, k.device)
    with torch.cuda.device(k.device):
        dz32 = dz.to(torch.float32).contiguous()
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        p = make_problem(q, k, scale, v=v, dk=dk, dv=dv)
        p.n_splits = lib.flare_pick_splits(C.byref(p))
        st = stream_of(k)
        part = torch.empty(p.n_splits, B, H, M, D, dtype=torch.float32, device=k.device)
        check(lib.flare_bwd_main(C.byref(p), _cabi.TERM_GATHER, ptr(q), ptr(k), ptr(v), None, None, ptr(mask), ptr(z32),
                                 ptr(dz32), ptr(lse_m), None, ptr(dk), ptr(dv), None, ptr(part), st), "flare_bwd_main")
        dq = _dq_from_parts(p, part, B, H, M, D, batched, st)
    return dq, dk, dv


def scatter_forward(q, k, z, scale=1.0, key_mask=None):
    """y, lse_n[B,H,N] via flare_scatter."""
    _need_cuda(q, k, z)
    q, _ = _q3(q)
    k = _tok(k)
    B, H, N, D = k.shape
    mask = _mask_u8(key_mask, B, N, k.device)
    with torch.cuda.device(k.device):
        z32 = z.to(torch.float32).contiguous()
        y = torch.empty_like(k)
        if y.stride(-1) != 1:
            y = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        lse_n = torch.empty(B, H, N, dtype=torch.float32, device=k.device)
        p = make_problem(q, k, scale, y=y)
        check(lib.flare_scatter(C.byref(p), ptr(q), ptr(k), ptr(z32), ptr(mask), ptr(y), ptr(lse_n), stream_of(k)),
              "flare_scatter")
    return y, lse_n


def scatter_backward(q, k, z, dy, y, lse_n, scale=1.0, key_mask=None):
    """dq (fp32), dk, dz (fp32) of the scatter alone (term 2 of the backward)."""
    q, batched = _q3(q)
    k, dy, y = _tok(k), _tok(dy), _tok(y)
    B, H, N, D = k.shape
    M = q.shape[-2]
    mask = _mask_u8(key_mask, B, N, k.device)
    with torch.cuda.device(k.device):
        z32 = z.to(torch.float32).contiguous()
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        p = make_problem(q, k, scale, y=y, dy=dy, dk=dk)
        p.n_splits = lib.flare_pick_splits(C.byref(p))
        st = stream_of(k)
        part = torch.empty(p.n_splits, B, H, M, D, dtype=torch.float32, device=k.device)
        dz32 = torch.empty(B, H, M, D, dtype=torch.float32, device=k.device)
        delta = torch.empty(B, H, N, dtype=torch.float32, device=k.device)
        check(lib.flare_bwd_dz_partial(C.byref(p), ptr(q), ptr(k), ptr(dy), ptr(mask), ptr(lse_n), ptr(part), st),
              "flare_bwd_dz_partial")
        check(lib.flare_reduce_sum(ptr(part), p.n_splits, B * H * M, D, ptr(dz32), st), "flare_reduce_sum")
        check(lib.flare_bwd_main(C.byref(p), _cabi.TERM_SCATTER, ptr(q), ptr(k), None, ptr(dy), ptr(y), ptr(mask), ptr(z32),
                                 None, None, ptr(lse_n), ptr(dk), None, ptr(delta), ptr(part), st), "flare_bwd_main")
        dq = _dq_from_parts(p, part, B, H, M, D, batched, st)
    return dq, dk, dz32


# ------------------------------------------------------------------------------------
# torch operators: opaque to torch.compile (fake kernels give the shapes), differentiable,
# autocast-aware.  The reference runs this path under torch.compile and torch.autocast
# (mlutils/trainer.py:135-137, 185; ablation/time_memory_bwd.py:460-470).
# ------------------------------------------------------------------------------------
Tensor = torch.Tensor


def _like_tokens(k: Tensor) -> Tensor:
    """What the kernels return for a [B,H,N,D] result: k's strides when those are addressable, else dense."""
    e = k.element_size()
    if k.stride(-1) == 1 and all((s * e) % 16 == 0 for s in k.stride()[:-1]):
        out = torch.empty_like(k)
        if out.stride(-1) == 1:
            return out
    return torch.empty(k.shape, dtype=k.dtype, device=k.device)


def _dq_like(q: Tensor) -> Tensor:
    return torch.empty(q.shape, dtype=torch.float32, device=q.device)


@torch.library.custom_op("flare_b200::mixer_fwd", mutates_args=())
def _op_mixer_fwd(q: Tensor, k: Tensor, v: Tensor, scale: float, key_mask: Optional[Tensor], dropout_p: float,
                  dropout_seed: int) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    return mixer_forward(q, k, v, scale, key_mask, dropout_p, dropout_seed)


@_op_mixer_fwd.register_fake
def _(q, k, v, scale, key_mask, dropout_p, dropout_seed):
    B, H, N, D = k.shape
    M = q.shape[-2]
    f32 = dict(dtype=torch.float32, device=k.device)
    return _like_tokens(k), torch.empty(B, H, M, D, **f32), torch.empty(B, H, M, **f32), torch.empty(B, H, N, **f32)


@torch.library.custom_op("flare_b200::mixer_bwd", mutates_args=())
def _op_mixer_bwd(q: Tensor, k: Tensor, v: Tensor, dy: Tensor, y: Tensor, z32: Tensor, lse_m: Tensor, lse_n: Tensor,
                  scale: float, key_mask: Optional[Tensor], dropout_p: float, dropout_seed: int) -> Tuple[Tensor, Tensor, Tensor]:
    return mixer_backward(q, k, v, dy, y, z32, lse_m, lse_n, scale, key_mask, dropout_p, dropout_seed)


@_op_mixer_bwd.register_fake
def _(q, k, v, dy, y, z32, lse_m, lse_n, scale, key_mask, dropout_p, dropout_seed):
    return _dq_like(q), _like_tokens(k), _like_tokens(v)


def _mixer_setup(ctx, inputs, output):
    q, k, v, scale, key_mask, dropout_p, dropout_seed = inputs
    y, z32, lse_m, lse_n = output
    ctx.save_for_backward(q, k, v, y, z32, lse_m, lse_n, key_mask)
    ctx.scale, ctx.dropout = scale, (dropout_p, dropout_seed)
    # z32, lse_m, lse_n are the backward's operands, not results anyone differentiates: without this the engine
    # fills a zero tensor for each of them on every backward (one of them B*H*N floats)
    ctx.set_materialize_grads(False)


def _mixer_backward(ctx, dy, _dz32, _dlm, _dln):
    if dy is None:
        return None, None, None, None, None, None, None
    q, k, v, y, z32, lse_m, lse_n, key_mask = ctx.saved_tensors
    dq, dk, dv = _op_mixer_bwd(q, k, v, dy, y, z32, lse_m, lse_n, ctx.scale, key_mask, *ctx.dropout)
    return dq.to(q.dtype), dk, dv, None, None, None, None


_op_mixer_fwd.register_autograd(_mixer_backward, setup_context=_mixer_setup)


@torch.library.custom_op("flare_b200::gather_fwd", mutates_args=())
def _op_gather_fwd(q: Tensor, k: Tensor, v: Tensor, scale: float, key_mask: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    return gather_forward(q, k, v, scale, key_mask)


@_op_gather_fwd.register_fake
def _(q, k, v, scale, key_mask):
    B, H, N, D = k.shape
    M = q.shape[-2]
    return (torch.empty(B, H, M, D, dtype=k.dtype, device=k.device), torch.empty(B, H, M, D, dtype=torch.float32, device=k.device),
            torch.empty(B, H, M, dtype=torch.float32, device=k.device))


@torch.library.custom_op("flare_b200::gather_bwd", mutates_args=())
def _op_gather_bwd(q: Tensor, k: Tensor, v: Tensor, dz: Tensor, z32: Tensor, lse_m: Tensor, scale: float,
                   key_mask: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    return gather_backward(q, k, v, dz, z32, lse_m, scale, key_mask)


@_op_gather_bwd.register_fake
def _(q, k, v, dz, z32, lse_m, scale, key_mask):
    return _dq_like(q), torch.empty(k.shape, dtype=k.dtype, device=k.device), torch.empty(v.shape, dtype=v.dtype, device=v.device)


def _gather_setup(ctx, inputs, output):
    q, k, v, scale, key_mask = inputs
    _z, z32, lse_m = output
    ctx.save_for_backward(q, k, v, z32, lse_m, key_mask)
    ctx.scale = scale
    ctx.set_materialize_grads(False)


def _gather_backward(ctx, dz, _dz32, _dlse):
    if dz is None:
        return None, None, None, None, None
    q, k, v, z32, lse_m, key_mask = ctx.saved_tensors
    dq, dk, dv = _op_gather_bwd(q, k, v, dz.contiguous(), z32, lse_m, ctx.scale, key_mask)
    return dq.to(q.dtype), dk, dv, None, None


_op_gather_fwd.register_autograd(_gather_backward, setup_context=_gather_setup)


@torch.library.custom_op("flare_b200::scatter_fwd", mutates_args=())
def _op_scatter_fwd(q: Tensor, k: Tensor, z: Tensor, scale: float, key_mask: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return scatter_forward(q, k, z, scale, key_mask)


@_op_scatter_fwd.register_fake
def _(q, k, z, scale, key_mask):
    B, H, N, D = k.shape
    return _like_tokens(k), torch.empty(B, H, N, dtype=torch.float32, device=k.device)


@torch.library.custom_op("flare_b200::scatter_bwd", mutates_args=())
def _op_scatter_bwd(q: Tensor, k: Tensor, z: Tensor, dy: Tensor, y: Tensor, lse_n: Tensor, scale: float,
                    key_mask: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    return scatter_backward(q, k, z, dy, y, lse_n, scale, key_mask)


@_op_scatter_bwd.register_fake
def _(q, k, z, dy, y, lse_n, scale, key_mask):
    return _dq_like(q), torch.empty(k.shape, dtype=k.dtype, device=k.device), torch.empty(z.shape, dtype=torch.float32, device=z.device)


def _scatter_setup(ctx, inputs, output):
    q, k, z, scale, key_mask = inputs
    y, lse_n = output
    ctx.save_for_backward(q, k, z, y, lse_n, key_mask)
    ctx.scale = scale
    ctx.set_materialize_grads(False)


def _scatter_backward(ctx, dy, _dlse):
    if dy is None:
        return None, None, None, None, None
    q, k, z, y, lse_n, key_mask = ctx.saved_tensors
    dq, dk, dz32 = _op_scatter_bwd(q, k, z, dy, y, lse_n, ctx.scale, key_mask)
    return dq.to(q.dtype), dk, dz32.to(z.dtype), None, None


_op_scatter_fwd.register_autograd(_scatter_backward, setup_context=_scatter_setup)


# ------------------------------------------------------------------------------------
# the public functions
# ------------------------------------------------------------------------------------
def _fold_q(q):
    # an expand()-ed q (stride 0 over the batch, pdebench/models/flare.py:136) is the shared-latent case
    if q.dim() == 4 and q.stride(0) == 0:
        return q[0]
    return q


def _autocast(*ts):
    """What SDPA does under torch.autocast: floating-point CUDA inputs are cast to the autocast dtype, so that
    fp32 latent parameters meet half-precision projections (mlutils/trainer.py:135-137 runs every step so)."""
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        return tuple(t.to(dt) if t is not None and t.is_cuda and t.is_floating_point() else t for t in ts)
    return ts


def _same_dtype(q, k, v):
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError(f"q, k, v must share a dtype outside torch.autocast; got {q.dtype}, {k.dtype}, {v.dtype}")


_dropout_calls = 0


def next_dropout_seed() -> int:
    """A new 64-bit seed per call, reproducible from torch.manual_seed and the order of the calls."""
    global _dropout_calls
    _dropout_calls += 1
    x = (torch.initial_seed() * 0x9E3779B97F4A7C15 + _dropout_calls * 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 31
    x = (x * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 29
    return x & 0x7FFFFFFFFFFFFFFF


def flare_multihead_mixer(q, k, v, scale: float = 1.0, key_mask: Optional[torch.Tensor] = None,
                          dropout_p: float = 0.0, dropout_seed: Optional[int] = None):
    """y[B,H,N,D] = SDPA(k, q, SDPA(q, k, v, scale), scale)   (README.md:37-53 of the reference).

    q: [H,M,D] (or [B,H,M,D]); k, v: [B,H,N,D], any strides with unit stride on D.
    key_mask: optional bool [B,N], True = token takes part (lra/models/backends.py:615-622);
    masked tokens are ignored by the gather and their output rows are zero.
    dropout_p: attention dropout of both SDPA calls (lra/models/backends.py:604-606): each softmax weight is
    dropped with this probability after normalisation and the rest scaled by 1/(1-p), independently in the
    gather and in the scatter; the masks come from a counter hash of torch's seed (``torch.manual_seed``) and
    the number of dropout calls made so far, not from torch's Philox stream (equal in distribution, not bit
    for bit).  ``dropout_seed`` fixes the masks explicitly.  16-bit dtypes with D in {16, 32} only.
    Works under torch.autocast (inputs are cast to the autocast dtype, as SDPA does) and inside
    torch.compile (registered operators ``flare_b200::mixer_fwd`` / ``mixer_bwd``).
    """
    _need_cuda(q, k, v)
    q, k, v = _autocast(_fold_q(q), k, v)
    _same_dtype(q, k, v)
    if not 0.0 <= dropout_p < 1.0:
        raise ValueError(f"dropout_p must be in [0, 1), got {dropout_p}")
    seed = 0
    if dropout_p > 0.0:
        if k.dtype == torch.float32:
            raise NotImplementedError("attention dropout runs on the tensor-core kernels: bf16 or fp16 inputs (or autocast)")
        seed = next_dropout_seed() if dropout_seed is None else int(dropout_seed)
    return _op_mixer_fwd(q, k, v, float(scale), key_mask, float(dropout_p), seed)[0]


def flare_gather(q, k, v, scale: float = 1.0, key_mask=None):
    """(z[B,H,M,D], lse[B,H,M]): the first SDPA call, z = softmax_N(scale q k^T) v."""
    _need_cuda(q, k, v)
    q, k, v = _autocast(_fold_q(q), k, v)
    _same_dtype(q, k, v)
    z, _z32, lse_m = _op_gather_fwd(q, k, v, float(scale), key_mask)
    return z, lse_m.detach()


def flare_scatter(q, k, z, scale: float = 1.0, key_mask=None):
    """y[B,H,N,D]: the second SDPA call, y = softmax_M(scale k q^T) z."""
    _need_cuda(q, k, z)
    q, k, z = _autocast(_fold_q(q), k, z)
    return _op_scatter_fwd(q, k, z, float(scale), key_mask)[0]
