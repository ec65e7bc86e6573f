"""flare_gather_noalloc: the gather pass for callers that cannot allocate device memory.

Some users of the library sit where allocation is not allowed at call time -- a plugin inside a
framework that planned its memory up front, or a latency-critical thread that must not enter the
CUDA allocator.  For them the library keeps the split-N partial records in a fixed built-in array.
This test drives that entry point through the C ABI, twice in a row (the array keeps the first
call's records, so the second call proves stale contents do not leak into the result), and
compares with the workspace-based entry points (flare_gather_partial + flare_combine).

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import pytest
import torch

from oracle import flare_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def env(cuda_dev):
    import __graft_entry__
    __graft_entry__.build()
    import flare_b200  # noqa: F401
    from flare_b200 import _cabi
    from flare_b200.mixer import make_problem
    return _cabi, make_problem


def _existing_path(cabi, make_problem, q, k, v, scale):
    B, H, N, D = k.shape
    M = q.shape[-2]
    p = make_problem(q, k, scale, v=v)
    p.n_splits = cabi.lib.flare_pick_splits(C.byref(p))
    rec = torch.empty(p.n_splits, B, H, M, D + 2, dtype=torch.float32, device=k.device)
    z32 = torch.empty(B, H, M, D, dtype=torch.float32, device=k.device)
    lse = torch.empty(B, H, M, dtype=torch.float32, device=k.device)
    cabi.check(cabi.lib.flare_gather_partial(C.byref(p), q.data_ptr(), k.data_ptr(), v.data_ptr(), None,
                                             rec.data_ptr(), None), "flare_gather_partial")
    cabi.check(cabi.lib.flare_combine(C.byref(p), rec.data_ptr(), p.n_splits, z32.data_ptr(), None,
                                      lse.data_ptr(), None, None), "flare_combine")
    torch.cuda.synchronize()
    return z32, lse


def _noalloc(cabi, make_problem, q, k, v, scale, n_splits=0):
    B, H, N, D = k.shape
    M = q.shape[-2]
    p = make_problem(q, k, scale, v=v, n_splits=n_splits)
    z32 = torch.full((B, H, M, D), float("nan"), dtype=torch.float32, device=k.device)
    z = torch.empty(B, H, M, D, dtype=k.dtype, device=k.device)
    lse = torch.full((B, H, M), float("nan"), dtype=torch.float32, device=k.device)
    cabi.check(cabi.lib.flare_gather_noalloc(C.byref(p), q.data_ptr(), k.data_ptr(), v.data_ptr(), None,
                                             z32.data_ptr(), z.data_ptr(), lse.data_ptr(), None),
               "flare_gather_noalloc")
    torch.cuda.synchronize()
    return z32, z, lse


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_workspace_entry_points(env, cuda_dev, dtype):
    cabi, make_problem = env
    tol = TOL[dtype]
    # two different problems back to back: the second must not see the first one's records
    for (B, H, N, M, D, scale, seed) in [(2, 4, 3000, 64, 32, 1.0, 1), (1, 8, 777, 128, 16, 0.5, 2)]:
        q, k, v, _ = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=seed)
        qd, kd, vd = (t.to(cuda_dev) for t in (q, k, v))
        z_ref, lse_ref = _existing_path(cabi, make_problem, qd, kd, vd, scale)
        z32, z, lse = _noalloc(cabi, make_problem, qd, kd, vd, scale)
        assert O.rel_l2(z32, z_ref) <= tol
        assert O.rel_l2(lse, lse_ref) <= max(tol * 1e-2, 1e-6)
        assert O.rel_l2(z.float(), z_ref) <= max(tol, 1e-5)
        # and against the CPU oracle, like every other parity test
        z_o, L_o = O.gather(q.float(), k.float(), v.float(), scale)
        assert O.rel_l2(z32.cpu(), z_o) <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_more_ranges_asked_for_than_fit(env, cuda_dev, dtype):
    """B=8, H=8, M=256, D=32: one record set is 2.1 MiB, seven fit in the 16 MiB array.  Asking for 16
    token ranges makes the entry point fall back to 7; N = 2000 rounds each range up to 384 tokens, so
    only 6 of the 7 are non-empty and the last one must come out as a neutral record, not as whatever
    the previous call left there (large finite records, written first on purpose)."""
    cabi, make_problem = env
    B, H, N, M, D = 8, 8, 2000, 256, 32
    big_q, big_k, big_v, _ = O.make_inputs(B, H, 4000, M, D, dtype=dtype, seed=5)
    _noalloc(cabi, make_problem, (big_q * 3).to(cuda_dev), (big_k * 3).to(cuda_dev), (big_v * 100).to(cuda_dev), 1.0)
    q, k, v, _ = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=6)
    qd, kd, vd = (t.to(cuda_dev) for t in (q, k, v))
    z_ref, lse_ref = _existing_path(cabi, make_problem, qd, kd, vd, 1.0)
    z32, z, lse = _noalloc(cabi, make_problem, qd, kd, vd, 1.0, n_splits=16)
    tol = TOL[dtype]
    assert torch.isfinite(z32).all() and torch.isfinite(lse).all()
    assert O.rel_l2(z32, z_ref) <= tol
    assert O.rel_l2(lse, lse_ref) <= max(tol * 1e-2, 1e-6)


def test_sizes_beyond_the_built_in_scratch_are_refused(env, cuda_dev):
    cabi, make_problem = env
    # B*H*M*(D+2) = 64*64*512*34 floats = 272 MiB of records: far beyond the 16 MiB array
    p = cabi.FlareProblem()
    p.B, p.H, p.N, p.M, p.D = 64, 64, 128, 512, 32
    p.dtype, p.scale = cabi.F32, 1.0
    rc = cabi.lib.flare_gather_noalloc(C.byref(p), 16, 16, 16, None, 16, None, None, None)
    assert rc == -3
    assert b"built-in scratch" in cabi.lib.flare_last_error()
