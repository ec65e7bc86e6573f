"""Causal FLARE: prefill over a whole sequence and recurrent decode on a per-(b, h) state.

The reference links this path (README.md:60) without shipping code, a formula or a test vector (its
figs/flare_decoder.py only animates a decoder diagram), so the definition is this library's own choice:
``y_t = softmax_M(S[:, t]) . z_t`` with ``z_t = softmax_{n <= t}(S) v`` and ``S = scale * q k^T`` -- token t
sees the latent summary of tokens 0..t inclusive, the natural reading of "causal" for the gather and the one
under which decoding token by token reproduces the prefill.  The state is one record per latent,
``[B, H, M, D + 2] = (acc[D], m, l)`` in fp32, the same record the non-causal gather writes per token
range; ``causal_state_init`` gives the empty one.  ``flare_causal_mixer`` is the differentiable form for
training (a whole sequence from an empty prefix); prefill with a carried state and decode are forward only.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._cabi import check, lib, ptr, stream_of
from .mixer import _need_cuda, _q3, _tok, make_problem

__all__ = ["causal_state_init", "flare_causal_prefill", "flare_causal_decode", "flare_causal_mixer"]


def causal_state_init(B: int, H: int, M: int, D: int, device) -> torch.Tensor:
    """The record of an empty prefix: acc = 0, m = -inf, l = 0."""
    st = torch.zeros(B, H, M, D + 2, dtype=torch.float32, device=device)
    st[..., D] = float("-inf")
    return st


def flare_causal_prefill(q, k, v, scale: float = 1.0, state=None):
    """All tokens of k, v [B,H,N,D] at once.  Returns (y [B,H,N,D], state after the last token)."""
    _need_cuda(q, k, v)
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k, v must share a dtype")
    q, _ = _q3(q)
    k, v = _tok(k), _tok(v)
    B, H, N, D = k.shape
    M = q.shape[-2]
    with torch.cuda.device(k.device):
        y = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        out = torch.empty(B, H, M, D + 2, dtype=torch.float32, device=k.device)
        p = make_problem(q, k, scale, v=v, y=y)
        ws = torch.empty(lib.flare_causal_workspace_bytes(C.byref(p)), dtype=torch.uint8, device=k.device)
        if state is not None:
            state = state.contiguous()
        check(lib.flare_causal_prefill(C.byref(p), ptr(q), ptr(k), ptr(v), ptr(y), ptr(state), ptr(out), ptr(ws),
                                       stream_of(k)), "flare_causal_prefill")
    return y, out


def flare_causal_decode(q, k, v, state, scale: float = 1.0):
    """The tokens of k, v [B,H,T,D] (T is usually 1) one after the other; `state` is updated in place."""
    _need_cuda(q, k, v, state)
    q, _ = _q3(q)
    k, v = _tok(k), _tok(v)
    B, H, T, D = k.shape
    M = q.shape[-2]
    if tuple(state.shape) != (B, H, M, D + 2) or state.dtype != torch.float32 or not state.is_contiguous():
        raise ValueError(f"state must be a contiguous fp32 [B,H,M,D+2] = {(B, H, M, D + 2)} tensor")
    with torch.cuda.device(k.device):
        y = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        p = make_problem(q, k, scale, v=v, y=y)
        check(lib.flare_causal_decode(C.byref(p), ptr(q), ptr(k), ptr(v), ptr(y), ptr(state), stream_of(k)),
              "flare_causal_decode")
    return y


class _CausalMixerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        y, _ = flare_causal_prefill(q, k, v, scale)
        ctx.save_for_backward(q, k, v)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, v = ctx.saved_tensors
        q3, _ = _q3(q)
        kk, vv, dy = _tok(k), _tok(v), _tok(dy)
        B, H, N, D = kk.shape
        M = q3.shape[-2]
        dev = kk.device
        with torch.cuda.device(dev):
            dk = torch.empty(kk.shape, dtype=kk.dtype, device=dev)
            dv = torch.empty(vv.shape, dtype=vv.dtype, device=dev)
            dq32 = torch.empty(B, H, M, D, dtype=torch.float32, device=dev)
            p = make_problem(q3, kk, ctx.scale, v=vv, dy=dy, dk=dk, dv=dv)
            ws = torch.empty(lib.flare_causal_bwd_workspace_bytes(C.byref(p)), dtype=torch.uint8, device=dev)
            check(lib.flare_causal_bwd(C.byref(p), ptr(q3), ptr(kk), ptr(vv), ptr(dy), ptr(dq32), ptr(dk), ptr(dv),
                                       ptr(ws), stream_of(kk)), "flare_causal_bwd")
        # one latent gradient per (b, h): shared latents sum over the batch; a batch made by expand() gets the
        # per-batch gradients, which autograd folds back itself
        dq = dq32.sum(0) if q.dim() == 3 else dq32
        return dq.to(q.dtype), dk, dv, None


def flare_causal_mixer(q, k, v, scale: float = 1.0):
    """Causal FLARE over a whole sequence, differentiable in q, k, v: token t sees the latent summary of
    tokens 0..t only.  q [H,M,D] (or [B,H,M,D]), k, v [B,H,N,D]; returns y [B,H,N,D]."""
    _need_cuda(q, k, v)
    return _CausalMixerFn.apply(q, k, v, float(scale))
