"""CPU oracle for the FLARE gather-scatter token mixer.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file;
it is the checker used by ``tests/``, by the smoke entry and by the CPU
baseline leg of ``bench.py``.  It restates, in plain PyTorch on the CPU, the
algorithm of the reference project (vpuri3/FLARE.py):

* ``mixer_sdpa``      -- the two back-to-back SDPA calls of
                         ``README.md:37-53`` / ``pdebench/models/flare.py:136-138``.
* ``mixer_explicit``  -- the explicit softmax form of
                         ``pdebench/models/flare.py:141-150`` (with the scale
                         applied, which that branch of the reference omits).
* ``mixer_lra``       -- the masked variant of ``lra/models/backends.py:588-622``.
* closed-form backward, split-N partials with the log-sum-exp combine, the
  causal / recurrent form, triple attention (``lra/models/triton/triple.py:846-860``)
  and causal linear attention (``lra/models/triton/causal_linear.py:317-336``).

The arithmetic of the first item lives in a third-party dependency of the
reference that is not vendored in it: ``torch.nn.functional.
scaled_dot_product_attention`` (reference pin torch==2.8.0, ``uv.lock:3427``).
Parity pin: the functions here are checked in ``tests/test_oracle.py`` against
golden vectors produced by importing the reference's own
``pdebench/models/flare.py`` and ``lra/models/backends.py`` (script and vectors
under ``tests/golden/``).  The causal form and the context-parallel combine have
no counterpart in the reference: for those, parity is unpinned and the checks
are self-consistency ones (recurrent == dense masked, sharded == unsharded).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

__all__ = [
    "mixer_sdpa", "mixer_explicit", "mixer_lra", "dropout_keep_masks", "mixer_dropout", "gather", "scatter",
    "mixer_fwd_stats", "mixer_bwd_closed_form", "mixer_fwd_bwd_streamed", "gather_partials",
    "lse_combine", "causal_dense", "causal_recurrent", "causal_chunked", "causal_bwd_autograd", "causal_bwd_chunked",
    "triple_attention", "triple_attention_bwd", "causal_linear", "rel_l2",
]


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a-b||_2 / ||b||_2 in float64 (the acceptance measure)."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    den = b.norm().item()
    return (a - b).norm().item() / (den if den > 0 else 1.0)


def _expand_q(q: torch.Tensor, B: int) -> torch.Tensor:
    if q.dim() == 3:
        q = q.unsqueeze(0).expand(B, -1, -1, -1)
    return q


# ---------------------------------------------------------------------------
# forward
# ---------------------------------------------------------------------------
def mixer_sdpa(q, k, v, scale: float = 1.0):
    """README.md:37-53: z = SDPA(q,k,v); y = SDPA(k,q,z)."""
    qe = _expand_q(q, k.shape[0])
    z = F.scaled_dot_product_attention(qe, k, v, scale=scale)
    y = F.scaled_dot_product_attention(k, qe, z, scale=scale)
    return y


def gather(q, k, v, scale: float = 1.0, key_mask: Optional[torch.Tensor] = None):
    """z[B,H,M,D] = softmax_N(scale q k^T) v, and the row log-sum-exp L[B,H,M]."""
    qe = _expand_q(q, k.shape[0])
    s = scale * (qe @ k.transpose(-2, -1))            # [B,H,M,N]
    if key_mask is not None:
        s = s.masked_fill(~key_mask[:, None, None, :], float("-inf"))
    L = torch.logsumexp(s, dim=-1)
    z = torch.softmax(s, dim=-1) @ v
    return z, L


def scatter(q, k, z, scale: float = 1.0):
    """y[B,H,N,D] = softmax_M(scale k q^T) z, and the column log-sum-exp C[B,H,N]."""
    qe = _expand_q(q, k.shape[0])
    st = scale * (k @ qe.transpose(-2, -1))           # [B,H,N,M]
    C = torch.logsumexp(st, dim=-1)
    y = torch.softmax(st, dim=-1) @ z
    return y, C


def mixer_explicit(q, k, v, scale: float = 1.0):
    """pdebench/models/flare.py:141-150 with the scale applied to the scores."""
    z, _ = gather(q, k, v, scale)
    y, _ = scatter(q, k, z, scale)
    return y


def mixer_lra(q, k, v, scale: float = 1.0, key_mask: Optional[torch.Tensor] = None):
    """lra/models/backends.py:588-622: key_mask[B,N] bool, True = keep.

    Gather ignores masked tokens; masked tokens' own output rows are zero
    (what the installed torch returns for an all-masked SDPA row).
    """
    z, _ = gather(q, k, v, scale, key_mask)
    y, _ = scatter(q, k, z, scale)
    if key_mask is not None:
        y = y * key_mask[:, None, :, None].to(y.dtype)
    return y


def dropout_keep_masks(B, H, M, N, p: float, seed: int):
    """The keep masks the CUDA kernels draw for attention dropout, recomputed on the host: element
    (which, b, h, m, n) is kept iff hash(n, (which*B*H + b*H + h)*M + m, seed) >= p * 2^32 (32-bit
    wrap-around arithmetic; which = 1 for the gather weights, 2 for the scatter weights).
    Returns two bool tensors [B,H,M,N]."""
    import numpy as np
    u = np.uint32
    seed_lo, seed_hi = u(seed & 0xFFFFFFFF), u((seed >> 32) & 0xFFFFFFFF)
    thresh = min(int(p * 4294967296.0), 4294967295)
    n = np.arange(N, dtype=np.uint32)[None, :]
    out = []
    with np.errstate(over="ignore"):
        for which in (1, 2):
            rows = (np.arange(B * H, dtype=np.uint32)[:, None] + u(which * B * H)) * u(M) + np.arange(M, dtype=np.uint32)[None, :]
            row = rows.reshape(-1, 1)
            x = (n * u(0x9E3779B1)) ^ seed_lo
            y = (row * u(0x85EBCA77)) ^ seed_hi
            x = x ^ (y + u(0x165667B1) + (x << u(6)) + (x >> u(2)))
            x ^= x >> u(16); x *= u(0x85EBCA6B); x ^= x >> u(13); x *= u(0xC2B2AE35); x ^= x >> u(16)
            out.append(torch.from_numpy((x >= u(thresh)).reshape(B, H, M, N)))
    return out[0], out[1]


def mixer_dropout(q, k, v, scale: float, keep1, keep2, p: float, key_mask: Optional[torch.Tensor] = None):
    """The two SDPA calls with dropout_p = p (lra/models/backends.py:604-606) for GIVEN keep masks: dropout
    acts on the normalised softmax weights, survivors scaled by 1/(1-p)."""
    qe = _expand_q(q, k.shape[0])
    s = scale * (qe @ k.transpose(-2, -1))
    sg = s if key_mask is None else s.masked_fill(~key_mask[:, None, None, :], float("-inf"))
    P = torch.softmax(sg, dim=-1) * keep1 / (1.0 - p)
    z = P @ v
    A = torch.softmax(s, dim=-2) * keep2 / (1.0 - p)
    y = A.transpose(-2, -1) @ z
    if key_mask is not None:
        y = y * key_mask[:, None, :, None].to(y.dtype)
    return y


def mixer_fwd_stats(q, k, v, scale: float = 1.0):
    """(y, z, L, C): outputs plus both log-sum-exp vectors."""
    z, L = gather(q, k, v, scale)
    y, C = scatter(q, k, z, scale)
    return y, z, L, C


# ---------------------------------------------------------------------------
# backward (closed form; equals autograd of mixer_sdpa)
# ---------------------------------------------------------------------------
def mixer_bwd_closed_form(q, k, v, dy, scale: float = 1.0):
    """dq[H,M,D] (summed over B when q is 3-D), dk, dv for the encoder mixer.

    S = scale q k^T; P = softmax_N(S); A = softmax_M(S) (column-wise);
    dZ = A dY;  dV = P^T dZ;
    dS = P*(dZ V^T - rowsum(dZ*Z)) + A*(Z dY^T - colsum(dY*Y));
    dQ = scale dS K;  dK = scale dS^T Q.
    """
    B = k.shape[0]
    qe = _expand_q(q, B)
    S = scale * (qe @ k.transpose(-2, -1))            # [B,H,M,N]
    P = torch.softmax(S, dim=-1)
    A = torch.softmax(S, dim=-2)
    Z = P @ v                                         # [B,H,M,D]
    Y = A.transpose(-2, -1) @ Z                       # [B,H,N,D]
    dZ = A @ dy
    delta_n = (dy * Y).sum(-1)                        # [B,H,N]
    Delta_m = (dZ * Z).sum(-1)                        # [B,H,M]
    dV = P.transpose(-2, -1) @ dZ
    dS = P * (dZ @ v.transpose(-2, -1) - Delta_m[..., None]) \
        + A * (Z @ dy.transpose(-2, -1) - delta_n[..., None, :])
    dQ = scale * (dS @ k)
    dK = scale * (dS.transpose(-2, -1) @ qe)
    if q.dim() == 3:
        dQ = dQ.sum(0)
    return dQ, dK, dV


def mixer_bwd_autograd(q, k, v, dy, scale: float = 1.0, fn=None):
    """dq, dk, dv by autograd through ``fn`` (default: the two-SDPA form)."""
    fn = fn or mixer_sdpa
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    y = fn(q, k, v, scale)
    y.backward(dy)
    return q.grad, k.grad, v.grad


def mixer_fwd_bwd_streamed(q, k, v, dy, scale: float = 1.0, chunk: int = 65536):
    """(y, dq, dk, dv) of the encoder mixer with the token axis walked in chunks.

    The same arithmetic as ``mixer_sdpa`` + ``mixer_bwd_closed_form`` (README.md:37-53 and its
    autograd), arranged so that no more than M x chunk scores exist at a time: the oracle for
    token counts where the dense M x N matrices do not fit (one (b, h) of the million-token case).
    Three sweeps: records of the gather + log-sum-exp combine -> Z, L; then Y and dZ; then dV, dK, dQ.
    """
    B, H, N, D = k.shape
    qe = _expand_q(q, B)
    bounds = [(n0, min(N, n0 + chunk)) for n0 in range(0, N, chunk)]
    m, l, acc = gather_partials(q, k, v, scale, bounds)
    Z, L = lse_combine(m, l, acc)                      # [B,H,M,D], [B,H,M]
    y = torch.empty_like(v)
    dZ = torch.zeros_like(Z)
    for n0, n1 in bounds:
        S = scale * (qe @ k[:, :, n0:n1].transpose(-2, -1))
        A = torch.softmax(S, dim=-2)
        y[:, :, n0:n1] = A.transpose(-2, -1) @ Z
        dZ += A @ dy[:, :, n0:n1]
    Delta_m = (dZ * Z).sum(-1)
    dQ = torch.zeros_like(qe)
    dK, dV = torch.empty_like(k), torch.empty_like(v)
    for n0, n1 in bounds:
        kk, vv, gg = k[:, :, n0:n1], v[:, :, n0:n1], dy[:, :, n0:n1]
        S = scale * (qe @ kk.transpose(-2, -1))
        P = torch.exp(S - L[..., None])
        A = torch.softmax(S, dim=-2)
        delta_n = (gg * y[:, :, n0:n1]).sum(-1)
        dV[:, :, n0:n1] = P.transpose(-2, -1) @ dZ
        dS = P * (dZ @ vv.transpose(-2, -1) - Delta_m[..., None]) + A * (Z @ gg.transpose(-2, -1) - delta_n[..., None, :])
        dQ += scale * (dS @ kk)
        dK[:, :, n0:n1] = scale * (dS.transpose(-2, -1) @ qe)
    if q.dim() == 3:
        dQ = dQ.sum(0)
    return y, dQ, dK, dV


# ---------------------------------------------------------------------------
# split-N partials and the log-sum-exp combine (single-GPU splits and the
# context-parallel exchange use the same record)
# ---------------------------------------------------------------------------
def gather_partials(q, k, v, scale: float, bounds) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-range partial records for token ranges ``bounds = [(n0,n1),...]``.

    Returns m[S,B,H,M] (running max), l[S,B,H,M] (sum of exp(s-m)) and
    acc[S,B,H,M,D] (sum of exp(s-m) v).  An empty range gives m=-inf, l=0, acc=0.
    """
    B = k.shape[0]
    qe = _expand_q(q, B)
    ms, ls, accs = [], [], []
    for (n0, n1) in bounds:
        kk, vv = k[:, :, n0:n1], v[:, :, n0:n1]
        s = scale * (qe @ kk.transpose(-2, -1))
        if n1 > n0:
            m = s.max(dim=-1).values
            e = torch.exp(s - m[..., None])
            l = e.sum(-1)
            acc = e @ vv
        else:
            m = torch.full(s.shape[:-1], float("-inf"), dtype=s.dtype)
            l = torch.zeros_like(m)
            acc = torch.zeros(*m.shape, v.shape[-1], dtype=s.dtype)
        ms.append(m); ls.append(l); accs.append(acc)
    return torch.stack(ms), torch.stack(ls), torch.stack(accs)


def lse_combine(m, l, acc):
    """Combine records along dim 0: returns z[B,H,M,D] and L[B,H,M]."""
    mx = m.max(dim=0).values
    w = torch.exp(m - mx)                              # exp(-inf - finite) = 0
    w = torch.where(torch.isfinite(m), w, torch.zeros_like(w))
    lt = (l * w).sum(0)
    at = (acc * w[..., None]).sum(0)
    return at / lt[..., None], mx + torch.log(lt)


# ---------------------------------------------------------------------------
# causal FLARE (no reference code; self-consistency only)
# ---------------------------------------------------------------------------
def causal_dense(q, k, v, scale: float = 1.0):
    """y_t = softmax_M(S[:,t]) . z_t,  z_t = softmax_{n<=t}(S) v  (dense, small N)."""
    B, H, N, D = k.shape
    qe = _expand_q(q, B)
    S = scale * (qe @ k.transpose(-2, -1))            # [B,H,M,N]
    A = torch.softmax(S, dim=-2)                       # over M, per token
    ys = []
    for t in range(N):
        P = torch.softmax(S[..., : t + 1], dim=-1)
        z = P @ v[:, :, : t + 1]                       # [B,H,M,D]
        ys.append(torch.einsum("bhm,bhmd->bhd", A[..., t], z))
    return torch.stack(ys, dim=2)


def causal_recurrent(q, k, v, scale: float = 1.0, state=None):
    """Token-by-token recurrence on the state (m[M], l[M], acc[M,D])."""
    B, H, N, D = k.shape
    qe = _expand_q(q, B)
    M = qe.shape[2]
    if state is None:
        m = torch.full((B, H, M), float("-inf"), dtype=k.dtype)
        l = torch.zeros(B, H, M, dtype=k.dtype)
        acc = torch.zeros(B, H, M, D, dtype=k.dtype)
    else:
        m, l, acc = state
    ys = []
    for t in range(N):
        s = scale * torch.einsum("bhmd,bhd->bhm", qe, k[:, :, t])
        mn = torch.maximum(m, s)
        a = torch.where(torch.isfinite(m), torch.exp(m - mn), torch.zeros_like(m))
        e = torch.exp(s - mn)
        l = a * l + e
        acc = a[..., None] * acc + e[..., None] * v[:, :, t, None, :]
        m = mn
        w = torch.softmax(s, dim=-1)
        ys.append(torch.einsum("bhm,bhmd->bhd", w / l, acc))
    return torch.stack(ys, dim=2), (m, l, acc)


def causal_chunked(q, k, v, scale: float = 1.0, chunk: int = 64):
    """Chunked prefill: carry (m,l,acc) across chunks, matmuls inside a chunk."""
    B, H, N, D = k.shape
    qe = _expand_q(q, B)
    M = qe.shape[2]
    m0 = torch.full((B, H, M), float("-inf"), dtype=k.dtype)
    l0 = torch.zeros(B, H, M, dtype=k.dtype)
    a0 = torch.zeros(B, H, M, D, dtype=k.dtype)
    out = []
    for c0 in range(0, N, chunk):
        kk, vv = k[:, :, c0:c0 + chunk], v[:, :, c0:c0 + chunk]
        T = kk.shape[2]
        S = scale * (qe @ kk.transpose(-2, -1))        # [B,H,M,T]
        mu = torch.maximum(m0, S.max(-1).values)
        a = torch.where(torch.isfinite(m0), torch.exp(m0 - mu), torch.zeros_like(mu))
        E = torch.exp(S - mu[..., None])
        lmt = (a * l0)[..., None] + torch.cumsum(E, dim=-1)   # [B,H,M,T]
        G = (torch.softmax(S, dim=-2) / lmt).transpose(-2, -1)  # [B,H,T,M]
        inter = G @ (a[..., None] * a0)
        W = torch.tril(G @ E)                           # [B,H,T,T]
        out.append(inter + W @ vv)
        l0 = a * l0 + E.sum(-1)
        a0 = a[..., None] * a0 + E @ vv
        m0 = mu
    return torch.cat(out, dim=2), (m0, l0, a0)


def causal_bwd_autograd(q, k, v, dy, scale: float = 1.0):
    """dq, dk, dv of causal FLARE by autograd through the dense masked-softmax form (small N)."""
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    causal_dense(q, k, v, scale).backward(dy)
    return q.grad, k.grad, v.grad


def causal_bwd_chunked(q, k, v, dy, scale: float = 1.0, chunk: int = 64):
    """dq, dk, dv of causal FLARE as a reverse scan over chunks: the algorithm of the CUDA backward.

    Forward states (m, l, acc) at the chunk starts come from the same exclusive log-sum-exp prefix the
    prefill uses.  Walking the chunks from the last to the first, the suffix state
    R_m = sum_{t > chunk} G_tm g_t (M x D) and r_m = -sum_{t > chunk} G_tm (g_t . z_tm), G = A / l, is
    carried relative to the running maximum mu of the chunk that produced it, so that every factor that
    multiplies it is at most one.  Inside a chunk (E' = e^{S - mu}, l' = a l0 + cumsum E', G' = A / l',
    X_nt = v_n . g_t, c_mt = g_t . z_tm = (a (acc0 g^T) + E' triu(X)) / l'):
        dS2 = A (c - delta),  delta_t = sum_m A_mt c_mt
        dV  = E'^T Rin + tril(G'^T E')^T-masked g
        dS1 = E' (Rin V^T + rin + G' tril(X^T) - revcumsum(G' c))
        dQ += scale dS K,  dK = scale dS^T Q.
    """
    B, H, N, D = k.shape
    qe = _expand_q(q, B)
    M = qe.shape[2]
    bounds = [(c0, min(N, c0 + chunk)) for c0 in range(0, N, chunk)]
    # forward: exclusive prefix of the per-chunk records
    m, l, acc = gather_partials(q, k, v, scale, bounds)
    starts = []
    m0 = torch.full((B, H, M), float("-inf"), dtype=k.dtype)
    l0 = torch.zeros(B, H, M, dtype=k.dtype)
    a0 = torch.zeros(B, H, M, D, dtype=k.dtype)
    for c in range(len(bounds)):
        starts.append((m0, l0, a0))
        mn = torch.maximum(m0, m[c])
        wa = torch.where(torch.isfinite(m0), torch.exp(m0 - mn), torch.zeros_like(mn))
        wc = torch.where(torch.isfinite(m[c]), torch.exp(m[c] - mn), torch.zeros_like(mn))
        l0 = wa * l0 + wc * l[c]
        a0 = wa[..., None] * a0 + wc[..., None] * acc[c]
        m0 = mn
    dq = torch.zeros_like(qe)
    dk, dv = torch.zeros_like(k), torch.zeros_like(v)
    Rh = torch.zeros(B, H, M, D, dtype=k.dtype)
    rh = torch.zeros(B, H, M, dtype=k.dtype)
    nu = torch.full((B, H, M), float("inf"), dtype=k.dtype)
    for c in reversed(range(len(bounds))):
        n0, n1 = bounds[c]
        kk, vv, gg = k[:, :, n0:n1], v[:, :, n0:n1], dy[:, :, n0:n1]
        T = n1 - n0
        m0, l0, a0 = starts[c]
        S = scale * (qe @ kk.transpose(-2, -1))                    # [B,H,M,T]
        mu = torch.maximum(m0, S.max(-1).values)
        a = torch.where(torch.isfinite(m0), torch.exp(m0 - mu), torch.zeros_like(mu))
        E = torch.exp(S - mu[..., None])
        lp = (a * l0)[..., None] + torch.cumsum(E, dim=-1)
        A = torch.softmax(S, dim=-2)
        G = A / lp
        X = vv @ gg.transpose(-2, -1)                               # [B,H,T(n),T(t)]
        cm = (a[..., None] * (a0 @ gg.transpose(-2, -1)) + E @ torch.triu(X)) / lp      # c_mt
        delta = (A * cm).sum(-2, keepdim=True)
        dS2 = A * (cm - delta)
        w = torch.where(torch.isfinite(nu), torch.exp(mu - nu), torch.zeros_like(mu))  # rescale the carry-in
        Rin, rin = w[..., None] * Rh, w * rh
        W = G.transpose(-2, -1) @ E                                 # [B,H,T(t),T(n)]
        dv[:, :, n0:n1] = E.transpose(-2, -1) @ Rin + torch.tril(W).transpose(-2, -1) @ gg
        Gc = G * cm
        rev = torch.flip(torch.cumsum(torch.flip(Gc, [-1]), dim=-1), [-1])             # sum_{t >= n}
        de = Rin @ vv.transpose(-2, -1) + rin[..., None] + G @ torch.tril(X.transpose(-2, -1)) - rev
        dS = E * de + dS2
        dq += scale * (dS @ kk)
        dk[:, :, n0:n1] = scale * (dS.transpose(-2, -1) @ qe)
        Rh = Rin + G @ gg
        rh = rin - Gc.sum(-1)
        nu = mu
    if q.dim() == 3:
        dq = dq.sum(0)
    return dq, dk, dv


# ---------------------------------------------------------------------------
# the two Triton-kernel operators of the reference, as einsums
# ---------------------------------------------------------------------------
def triple_attention(q1, q2, k1, k2, v):
    """lra/models/triton/triple.py:846-860: STATE = K1 (x) V (x) K2 / N ; O = Q1 STATE Q2."""
    N = k1.shape[-2]
    state = torch.einsum("bhni,bhnj,bhnk->bhijk", k1.float(), v.float(), k2.float()) / N
    o = torch.einsum("bhni,bhijk,bhnk->bhnj", q1.float(), state, q2.float())
    return state, o


def triple_attention_bwd(q1, q2, k1, k2, v, do):
    """lra/models/triton/triple.py:887-931 (grad of O only)."""
    N = k1.shape[-2]
    q1, q2, k1, k2, v, do = (t.float() for t in (q1, q2, k1, k2, v, do))
    state = torch.einsum("bhni,bhnj,bhnk->bhijk", k1, v, k2) / N
    dstate = torch.einsum("bhni,bhnj,bhnk->bhijk", q1, do, q2)
    dq1 = torch.einsum("bhnj,bhijk,bhnk->bhni", do, state, q2)
    dq2 = torch.einsum("bhni,bhijk,bhnj->bhnk", q1, state, do)
    dk1 = torch.einsum("bhijk,bhnj,bhnk->bhni", dstate, v, k2) / N
    dk2 = torch.einsum("bhijk,bhni,bhnj->bhnk", dstate, k1, v) / N
    dv = torch.einsum("bhijk,bhni,bhnk->bhnj", dstate, k1, k2) / N
    return dq1, dq2, dk1, dk2, dv


def causal_linear(q, k, v):
    """lra/models/triton/causal_linear.py:317-336: Y_t = Q_t sum_{n<=t} K_n^T V_n / N."""
    N = k.shape[-2]
    kv = torch.einsum("bhnd,bhne->bhnde", k.float(), v.float()) / N
    st = torch.cumsum(kv, dim=2)
    return torch.einsum("bhnd,bhnde->bhne", q.float(), st)


def make_inputs(B, H, N, M, D, dtype=torch.float32, seed=0, std_pow=-0.25, q4d=False):
    """Seeded inputs: q,k,v = randn * D**std_pow (unit-variance logits at scale 1), dy = randn."""
    g = torch.Generator().manual_seed(seed)
    sd = float(D) ** std_pow
    q = torch.randn(H, M, D, generator=g) * sd
    k = torch.randn(B, H, N, D, generator=g) * sd
    v = torch.randn(B, H, N, D, generator=g) * sd
    dy = torch.randn(B, H, N, D, generator=g)
    return tuple(t.to(dtype) for t in (q, k, v, dy))
