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
    "mixer_forward", "mixer_backward", "make_problem", "set_kernel_path", "device_status",
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


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flare_b200 runs on CUDA tensors only (sm_100a); got a CPU tensor")


def _tok(t: torch.Tensor) -> torch.Tensor:
    """A [B,H,N,D] tensor the kernels can address: unit stride on D, 16-byte aligned rows."""
    e = t.element_size()
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all((s * e) % 16 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def _q3(q: torch.Tensor) -> Tuple[torch.Tensor, bool]:
    """q as [H,M,D] (shared latents) or [B,H,M,D]; an expand()-ed batch is folded back."""
    if q.dim() == 4 and q.stride(0) == 0:
        q = q[0]
    if q.dim() not in (3, 4):
        raise ValueError(f"q must be [H,M,D] or [B,H,M,D], got {tuple(q.shape)}")
    return _tok(q), q.dim() == 4


def make_problem(q, k, scale: float, n_splits: int = 0, v=None, y=None, dy=None, dk=None, dv=None) -> FlareProblem:
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


def mixer_forward(q, k, v, scale=1.0, key_mask=None):
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
        p = make_problem(q, k, scale, v=v, y=y)
        nbytes = lib.flare_fwd_workspace_bytes(C.byref(p))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=k.device)
        check(lib.flare_mixer_fwd(C.byref(p), ptr(q), ptr(k), ptr(v), ptr(mask), ptr(y), ptr(z32),
                                  ptr(lse_m), ptr(lse_n), ptr(ws), nbytes, stream_of(k)), "flare_mixer_fwd")
    return y, z32, lse_m, lse_n


def mixer_backward(q, k, v, dy, y, z32, lse_m, lse_n, scale=1.0, key_mask=None):
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
        p = make_problem(q, k, scale, v=v, y=y, dy=dy, dk=dk, dv=dv)
        nbytes = lib.flare_bwd_workspace_bytes(C.byref(p))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=k.device)
        check(lib.flare_mixer_bwd(C.byref(p), ptr(q), ptr(k), ptr(v), ptr(dy), ptr(y), ptr(mask), ptr(z32),
                                  ptr(lse_m), ptr(lse_n), ptr(dq), ptr(dk), ptr(dv), ptr(ws), nbytes,
                                  stream_of(k)), "flare_mixer_bwd")
    return dq, dk, dv


class _MixerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, key_mask):
        y, z32, lse_m, lse_n = mixer_forward(q, k, v, scale, key_mask)
        ctx.save_for_backward(q, k, v, y, z32, lse_m, lse_n, key_mask)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, v, y, z32, lse_m, lse_n, key_mask = ctx.saved_tensors
        dq, dk, dv = mixer_backward(q, k, v, dy, y, z32, lse_m, lse_n, ctx.scale, key_mask)
        return dq.to(q.dtype).reshape(q.shape), dk, dv, None, None


def _fold_q(q):
    # an expand()-ed q (stride 0 over the batch, pdebench/models/flare.py:136) is the shared-latent case
    if q.dim() == 4 and q.stride(0) == 0:
        return q[0]
    return q


def flare_multihead_mixer(q, k, v, scale: float = 1.0, key_mask: Optional[torch.Tensor] = None,
                          dropout_p: float = 0.0):
    """y[B,H,N,D] = SDPA(k, q, SDPA(q, k, v, scale), scale)   (README.md:37-53 of the reference).

    q: [H,M,D] (or [B,H,M,D]); k, v: [B,H,N,D], any strides with unit stride on D.
    key_mask: optional bool [B,N], True = token takes part (lra/models/backends.py:615-622);
    masked tokens are ignored by the gather and their output rows are zero.
    """
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not supported by the fused mixer (dropout_p must be 0)")
    return _MixerFn.apply(_fold_q(q), k, v, float(scale), key_mask)


# ------------------------------------------------------------------------------------
# gather and scatter as separate differentiable operators
# ------------------------------------------------------------------------------------
def _gather_fwd(q, k, v, scale, mask):
    B, H, N, D = k.shape
    M = q.shape[-2]
    dev = k.device
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


def _dq_from_parts(p, part, B, H, M, D, batched, st):
    dq = torch.empty((B, H, M, D) if batched else (H, M, D), dtype=torch.float32, device=part.device)
    if batched:
        check(lib.flare_reduce_sum(ptr(part), p.n_splits, B * H * M, D, ptr(dq), st), "flare_reduce_sum")
    else:
        check(lib.flare_reduce_sum(ptr(part), p.n_splits * B, H * M, D, ptr(dq), st), "flare_reduce_sum")
    return dq


class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, key_mask):
        _need_cuda(q, k, v)
        q, _ = _q3(q)
        k, v = _tok(k), _tok(v)
        mask = _mask_u8(key_mask, k.shape[0], k.shape[2], k.device)
        with torch.cuda.device(k.device):
            z, z32, lse_m = _gather_fwd(q, k, v, scale, mask)
        ctx.save_for_backward(q, k, v, z32, lse_m, mask)
        ctx.scale = scale
        ctx.mark_non_differentiable(lse_m)
        return z, lse_m

    @staticmethod
    def backward(ctx, dz, _dlse):
        q, k, v, z32, lse_m, mask = ctx.saved_tensors
        B, H, N, D = k.shape
        M = q.shape[-2]
        batched = q.dim() == 4
        with torch.cuda.device(k.device):
            dz32 = dz.to(torch.float32).contiguous()
            dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
            dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
            p = make_problem(q, k, ctx.scale, v=v, dk=dk, dv=dv)
            p.n_splits = lib.flare_pick_splits(C.byref(p))
            st = stream_of(k)
            T = _cabi.TERM_GATHER
            check(lib.flare_bwd_tokens(C.byref(p), T, ptr(q), ptr(k), ptr(v), None, None, ptr(mask), ptr(z32),
                                       ptr(dz32), ptr(lse_m), None, ptr(dk), ptr(dv), None, st), "flare_bwd_tokens")
            part = torch.empty(p.n_splits, B, H, M, D, dtype=torch.float32, device=k.device)
            check(lib.flare_bwd_dq_partial(C.byref(p), T, ptr(q), ptr(k), ptr(v), None, ptr(mask), ptr(z32),
                                           ptr(dz32), ptr(lse_m), None, None, ptr(part), st), "flare_bwd_dq_partial")
            dq = _dq_from_parts(p, part, B, H, M, D, batched, st)
        return dq.to(q.dtype), dk, dv, None, None


class _ScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, z, scale, key_mask):
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
            check(lib.flare_scatter(C.byref(p), ptr(q), ptr(k), ptr(z32), ptr(mask), ptr(y), ptr(lse_n),
                                    stream_of(k)), "flare_scatter")
        ctx.save_for_backward(q, k, z32, y, lse_n, mask)
        ctx.scale = scale
        ctx.z_dtype = z.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, z32, y, lse_n, mask = ctx.saved_tensors
        B, H, N, D = k.shape
        M = q.shape[-2]
        batched = q.dim() == 4
        with torch.cuda.device(k.device):
            dy = _tok(dy)
            dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
            p = make_problem(q, k, ctx.scale, y=y, dy=dy, dk=dk)
            p.n_splits = lib.flare_pick_splits(C.byref(p))
            st = stream_of(k)
            T = _cabi.TERM_SCATTER
            part = torch.empty(p.n_splits, B, H, M, D, dtype=torch.float32, device=k.device)
            dz32 = torch.empty(B, H, M, D, dtype=torch.float32, device=k.device)
            delta = torch.empty(B, H, N, dtype=torch.float32, device=k.device)
            check(lib.flare_bwd_dz_partial(C.byref(p), ptr(q), ptr(k), ptr(dy), ptr(mask), ptr(lse_n), ptr(part), st),
                  "flare_bwd_dz_partial")
            check(lib.flare_reduce_sum(ptr(part), p.n_splits, B * H * M, D, ptr(dz32), st), "flare_reduce_sum")
            check(lib.flare_bwd_tokens(C.byref(p), T, ptr(q), ptr(k), None, ptr(dy), ptr(y), ptr(mask), ptr(z32),
                                       None, None, ptr(lse_n), ptr(dk), None, ptr(delta), st), "flare_bwd_tokens")
            check(lib.flare_bwd_dq_partial(C.byref(p), T, ptr(q), ptr(k), None, ptr(dy), ptr(mask), ptr(z32),
                                           None, None, ptr(lse_n), ptr(delta), ptr(part), st), "flare_bwd_dq_partial")
            dq = _dq_from_parts(p, part, B, H, M, D, batched, st)
        return dq.to(q.dtype), dk, dz32.to(ctx.z_dtype), None, None


def flare_gather(q, k, v, scale: float = 1.0, key_mask=None):
    """(z[B,H,M,D], lse[B,H,M]): the first SDPA call, z = softmax_N(scale q k^T) v."""
    return _GatherFn.apply(_fold_q(q), k, v, float(scale), key_mask)


def flare_scatter(q, k, z, scale: float = 1.0, key_mask=None):
    """y[B,H,N,D]: the second SDPA call, y = softmax_M(scale k q^T) z."""
    return _ScatterFn.apply(_fold_q(q), k, z, float(scale), key_mask)
