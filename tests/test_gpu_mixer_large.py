"""Parity of the tensor-core kernels against the CPU oracle at sizes where a token range spans many tiles.

* the benchmark's own problem (B=1, H=8, N=2^20, M=256, D=32, bf16): one head of the GPU result against
  the token-chunked oracle (``oracle.mixer_fwd_bwd_streamed``), forward and all three gradients;
* N ~ 65 536 with 256 and 192 latents, bf16 and fp16: several ranges of >= 64 tiles each, so the TMA
  rings wrap and every pipeline reaches steady state;
* the gather's lazy running maximum: one token range (n_splits = 1) whose row maxima grow along the
  token axis, a little (no rescale is ever needed) and a lot (the accumulator must be rescaled),
  for all rows or only for some, with a ragged last tile.

Tolerance: relative L2 <= 2e-2 against the fp32 oracle on the same rounded inputs.
"""
import ctypes as C

import pytest
import torch

from oracle import flare_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fb(cuda_dev):
    import __graft_entry__
    __graft_entry__.build()
    import flare_b200
    return flare_b200


def _run(fb, q, k, v, dy, scale, dev):
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    y = fb.flare_multihead_mixer(qd, kd, vd, scale=scale)
    y.backward(dy.to(dev))
    torch.cuda.synchronize()
    return y.detach(), qd.grad, kd.grad, vd.grad


def test_million_tokens_one_head_against_the_oracle(fb, cuda_dev):
    B, H, N, M, D = 1, 8, 1 << 20, 256, 32
    g = torch.Generator().manual_seed(99)
    sd = D ** -0.25
    q = (torch.randn(H, M, D, generator=g) * sd).bfloat16()
    k = (torch.randn(B, H, N, D, generator=g) * sd).bfloat16()
    v = (torch.randn(B, H, N, D, generator=g) * sd).bfloat16()
    dy = torch.randn(B, H, N, D, generator=g).bfloat16()
    y, dq, dk, dv = _run(fb, q, k, v, dy, 1.0, cuda_dev)
    assert fb.device_status() == 0
    h = 5
    ref = O.mixer_fwd_bwd_streamed(q[h:h + 1].float(), k[:, h:h + 1].float(), v[:, h:h + 1].float(),
                                   dy[:, h:h + 1].float(), 1.0, chunk=32768)
    got = (y[:, h:h + 1], dq[h:h + 1], dk[:, h:h + 1], dv[:, h:h + 1])
    errs = {n: O.rel_l2(a.float().cpu(), b) for n, a, b in zip(("y", "dq", "dk", "dv"), got, ref)}
    assert all(e <= 2e-2 for e in errs.values()), errs
    # token rows on both sides of every boundary between two token ranges of the split passes
    from flare_b200.mixer import make_problem
    p = make_problem(q.to(cuda_dev), k.to(cuda_dev), 1.0)
    S = fb._cabi.lib.flare_pick_splits(C.byref(p))
    chunk = -(-(-(-N // S)) // 128) * 128
    rows = torch.cat([torch.arange(max(0, b0 - 128), min(N, b0 + 128)) for b0 in range(chunk, N, chunk)])
    for name, a, b in zip(("y", "dk", "dv"), (got[0], got[2], got[3]), (ref[0], ref[2], ref[3])):
        e = O.rel_l2(a.float().cpu()[:, :, rows], b[:, :, rows])
        assert e <= 2e-2, (name, e)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,N,M,D", [
    (1, 2, 65536 + 77, 256, 32),
    (1, 2, 65536, 192, 32),
    (2, 1, 40000, 64, 16),
])
def test_many_tiles_per_range(fb, cuda_dev, dtype, B, H, N, M, D):
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=N + M)
    got = _run(fb, q, k, v, dy, 1.0, cuda_dev)
    assert fb.device_status() == 0
    ref = O.mixer_fwd_bwd_streamed(q.float(), k.float(), v.float(), dy.float(), 1.0, chunk=16384)
    errs = {n: O.rel_l2(a.float().cpu(), b) for n, a, b in zip(("y", "dq", "dk", "dv"), got, ref)}
    assert all(e <= 2e-2 for e in errs.values()), errs


def _ramp_inputs(N, M, D, top, some_rows_only, seed):
    """Scores whose row maximum grows along n: k_n = r(n) u + noise, q_m = a_m u + noise, r from 0 to `top`
    (natural-log units of the score).  a_m = 1, or +-1 alternating so that only half of the rows grow."""
    g = torch.Generator().manual_seed(seed)
    u = torch.zeros(D)
    u[0] = 1.0
    ramp = torch.linspace(0.0, top, N)
    k = ramp[:, None] * u[None, :] + 0.3 * torch.randn(N, D, generator=g)
    a = torch.ones(M)
    if some_rows_only:
        a[1::2] = -1.0
    q = a[:, None] * u[None, :] + 0.3 * torch.randn(M, D, generator=g)
    v = torch.randn(N, D, generator=g)
    dy = torch.randn(N, D, generator=g)
    f = lambda t: t.bfloat16()
    return f(q)[None], f(k)[None, None], f(v)[None, None], f(dy)[None, None]


@pytest.mark.parametrize("D", [32, 16])
@pytest.mark.parametrize("top,some_rows_only", [(12.0, False), (80.0, False), (80.0, True), (45.0, True)])
def test_gather_running_maximum_over_one_long_range(fb, cuda_dev, D, top, some_rows_only):
    from flare_b200 import _cabi
    from flare_b200.mixer import make_problem
    N, M = 2048 + 77, 256
    q, k, v, dy = _ramp_inputs(N, M, D, top, some_rows_only, seed=int(top) + D)
    dev = cuda_dev
    qd, kd, vd, dyd = (t.to(dev) for t in (q, k, v, dy))
    p = make_problem(qd, kd, 1.0, n_splits=1, v=vd, dy=dyd)
    rec = torch.empty(1, 1, 1, M, D + 2, device=dev)
    z32 = torch.empty(1, 1, M, D, device=dev)
    lse = torch.empty(1, 1, M, device=dev)
    _cabi.check(_cabi.lib.flare_gather_partial(C.byref(p), qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), None,
                                               rec.data_ptr(), None), "gather_partial")
    _cabi.check(_cabi.lib.flare_combine(C.byref(p), rec.data_ptr(), 1, z32.data_ptr(), None, lse.data_ptr(), None, None),
                "combine")
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    z_ref, L_ref = O.gather(q.float(), k.float(), v.float(), 1.0)
    assert O.rel_l2(z32.cpu(), z_ref) <= 2e-2
    assert (lse.cpu() - L_ref).abs().max() <= 2e-2 * max(1.0, L_ref.abs().max().item())
    # control: the dZ pass (same kernel, no running maximum) on the same scores
    _, Cn = O.scatter(q.float(), k.float(), z_ref, 1.0)
    dz = torch.empty(1, 1, 1, M, D, device=dev)
    _cabi.check(_cabi.lib.flare_bwd_dz_partial(C.byref(p), qd.data_ptr(), kd.data_ptr(), dyd.data_ptr(), None,
                                               Cn.contiguous().to(dev).data_ptr(), dz.data_ptr(), None), "dz_partial")
    torch.cuda.synchronize()
    S = (q.float()[None] @ k.float().transpose(-2, -1))
    dz_ref = torch.softmax(S, dim=-2) @ dy.float()
    assert O.rel_l2(dz[0].cpu(), dz_ref) <= 2e-2
