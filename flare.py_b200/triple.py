"""Triple attention and causal linear attention over the C ABI.

``triple_attention(q1, q2, k1, k2, v)`` has the meaning of ``TripleAttentionFunction`` in the reference
(lra/models/triton/triple.py:27-290; einsum form :846-860): it returns ``(STATE, O)`` with
``STATE[b,h,i,j,k] = (1/N) sum_n K1[n,i] V[n,j] K2[n,k]`` (fp32) and
``O[n,j] = sum_{i,k} Q1[n,i] STATE[i,j,k] Q2[n,k]``, and is differentiable (backward formulas :887-931).
``causal_linear(q, k, v)`` is ``CausalLinear`` (lra/models/triton/causal_linear.py:23-145, reference
:317-336): ``Y_t = Q_t sum_{n<=t} K_n^T V_n / N``, forward only as there.
"""
from __future__ import annotations

import torch

from . import _cabi
from ._cabi import check, lib, ptr, stream_of
from .mixer import _need_cuda, _tok

__all__ = ["triple_attention", "causal_linear"]


def _flat(t):
    """[B,H,N,D] -> contiguous [BH,N,D], as the reference does (triple.py:51-55)."""
    B, H, N, D = t.shape
    return t.reshape(B * H, N, D).contiguous()


def _outer(a, b, c, alpha):
    BH, N, Da = a.shape
    Db, Dc = b.shape[-1], c.shape[-1]
    out = torch.empty(BH, Da, Db, Dc, dtype=torch.float32, device=a.device)
    ws = torch.empty(lib.flare_triple_workspace_bytes(BH, N, Da, Db, Dc), dtype=torch.uint8, device=a.device)
    check(lib.flare_triple_outer(BH, N, Da, Db, Dc, _cabi.DTYPE_CODE[a.dtype], ptr(a), ptr(b), ptr(c), float(alpha),
                                 ptr(out), ptr(ws), stream_of(a)), "flare_triple_outer")
    return out


def _contract(t, perm, a, b, alpha):
    """out[n,x] = alpha * sum_{y,z} t.permute(perm)[x,y,z] a[n,y] b[n,z]; t is [BH,D0,D1,D2] fp32 contiguous."""
    BH, N, Dy = a.shape
    Dz = b.shape[-1]
    dims, strides = t.shape[1:], t.stride()[1:]
    Dx = dims[perm[0]]
    assert (dims[perm[1]], dims[perm[2]]) == (Dy, Dz)
    out = torch.empty(BH, N, Dx, dtype=a.dtype, device=a.device)
    check(lib.flare_triple_contract(BH, N, Dx, Dy, Dz, _cabi.DTYPE_CODE[a.dtype], ptr(t), strides[perm[0]],
                                    strides[perm[1]], strides[perm[2]], ptr(a), ptr(b), float(alpha), ptr(out),
                                    stream_of(a)), "flare_triple_contract")
    return out


class _TripleFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q1, q2, k1, k2, v):
        _need_cuda(q1, q2, k1, k2, v)
        if not (q1.dtype == q2.dtype == k1.dtype == k2.dtype == v.dtype):
            raise TypeError("q1, q2, k1, k2, v must share a dtype")
        B, H, N, Dq = q1.shape
        Dv = v.shape[-1]
        with torch.cuda.device(v.device):
            fq1, fq2, fk1, fk2, fv = (_flat(t) for t in (q1, q2, k1, k2, v))
            state = _outer(fk1, fv, fk2, 1.0 / N)                         # [BH, Dq, Dv, Dq]
            o = _contract(state, (1, 0, 2), fq1, fq2, 1.0)                # x = j, y = i, z = k
        ctx.save_for_backward(fq1, fq2, fk1, fk2, fv, state)
        ctx.shape = (B, H, N, Dq, Dv)
        return state.view(B, H, Dq, Dv, Dq), o.view(B, H, N, Dv)

    @staticmethod
    def backward(ctx, dstate_out, do):
        fq1, fq2, fk1, fk2, fv, state = ctx.saved_tensors
        B, H, N, Dq, Dv = ctx.shape
        with torch.cuda.device(fv.device):
            if do is None:
                do = torch.zeros(B, H, N, Dv, dtype=fv.dtype, device=fv.device)
            fdo = _flat(do.to(fv.dtype))
            dstate = _outer(fq1, fdo, fq2, 1.0)
            if dstate_out is not None:
                dstate = dstate + dstate_out.reshape(B * H, Dq, Dv, Dq).float()
            dq1 = _contract(state, (0, 1, 2), fdo, fq2, 1.0)              # x = i, y = j, z = k
            dq2 = _contract(state, (2, 0, 1), fq1, fdo, 1.0)              # x = k, y = i, z = j
            dk1 = _contract(dstate, (0, 1, 2), fv, fk2, 1.0 / N)
            dk2 = _contract(dstate, (2, 0, 1), fk1, fv, 1.0 / N)
            dv = _contract(dstate, (1, 0, 2), fk1, fk2, 1.0 / N)
        return (dq1.view(B, H, N, Dq), dq2.view(B, H, N, Dq), dk1.view(B, H, N, Dq), dk2.view(B, H, N, Dq),
                dv.view(B, H, N, Dv))


def triple_attention(q1, q2, k1, k2, v):
    """(STATE [B,H,Dq,Dv,Dq] fp32, O [B,H,N,Dv]); q1, q2, k1, k2: [B,H,N,Dq], v: [B,H,N,Dv]."""
    return _TripleFn.apply(q1, q2, k1, k2, v)


def causal_linear(q, k, v):
    """Y [B,H,N,Dv] = Q_t . sum_{n<=t} K_n^T V_n / N; q, k: [B,H,N,Dk], v: [B,H,N,Dv]."""
    _need_cuda(q, k, v)
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k, v must share a dtype")
    q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
    B, H, N, Dk = k.shape
    Dv = v.shape[-1]
    i64x3 = _cabi.C.c_int64 * 3
    with torch.cuda.device(k.device):
        y = torch.empty(B, H, N, Dv, dtype=v.dtype, device=v.device)
        ws = torch.empty(lib.flare_causal_linear_workspace_bytes(B, H, N, Dk, Dv), dtype=torch.uint8, device=k.device)
        check(lib.flare_causal_linear(B, H, N, Dk, Dv, _cabi.DTYPE_CODE[k.dtype],
                                      ptr(q), i64x3(*q.stride()[:3]), ptr(k), i64x3(*k.stride()[:3]),
                                      ptr(v), i64x3(*v.stride()[:3]), ptr(y), i64x3(*y.stride()[:3]),
                                      ptr(ws), stream_of(k)), "flare_causal_linear")
    return y
