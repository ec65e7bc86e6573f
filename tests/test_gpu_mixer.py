"""Parity of the CUDA mixer (through the C ABI) with the CPU oracle and the reference's golden vectors.

Tolerances are the acceptance ones: relative L2 <= 1e-5 for fp32 and <= 2e-2 for
bf16/fp16 against an fp32 oracle evaluated on the same (rounded) inputs.
"""
import pytest
import torch

from conftest import load_golden
from oracle import flare_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


@pytest.fixture(scope="module")
def fb(cuda_dev):
    import __graft_entry__
    __graft_entry__.build()
    import flare_b200
    return flare_b200


def run_mixer(fb, q, k, v, dy, scale, dev, key_mask=None):
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    y = fb.flare_multihead_mixer(qd, kd, vd, scale=scale, key_mask=None if key_mask is None else key_mask.to(dev))
    y.backward(dy.to(dev))
    torch.cuda.synchronize()
    return [t.float().cpu() for t in (y, qd.grad, kd.grad, vd.grad)]


def oracle_all(q, k, v, dy, scale):
    qf, kf, vf, dyf = (t.float() for t in (q, k, v, dy))
    y = O.mixer_sdpa(qf, kf, vf, scale)
    return [y, *O.mixer_bwd_closed_form(qf, kf, vf, dyf, scale)]


def assert_close(got, ref, tol, names=("y", "dq", "dk", "dv")):
    errs = {n: O.rel_l2(g, r) for n, g, r in zip(names, got, ref)}
    assert all(e <= tol for e in errs.values()), errs


@pytest.mark.parametrize("name", ["pde_mixer_s1", "pde_mixer_sqrt"])
def test_golden_vectors_from_reference(fb, cuda_dev, name):
    g = load_golden(name)
    got = run_mixer(fb, g["q"], g["k"], g["v"], g["dy"], g["scale"], cuda_dev)
    assert_close(got, [g["y"], g["dq"], g["dk"], g["dv"]], 1e-5)


def test_golden_masked_lra(fb, cuda_dev):
    g = load_golden("lra_mixer_mask")
    got = run_mixer(fb, g["q"], g["k"], g["v"], g["dy"], g["scale"], cuda_dev, key_mask=g["mask"].bool())
    assert_close(got, [g["y"], g["dq"], g["dk"], g["dv"]], 1e-5)


@pytest.mark.parametrize("path", ["simt", "auto"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,N,M,D,scale", [
    (2, 8, 4096, 64, 16, 1.0),          # the reference's CPU-runnable case
    (1, 2, 777, 100, 32, 32 ** -0.5),   # ragged N, M not a multiple of the tile
    (2, 3, 130, 16, 8, 1.0),
    (1, 2, 515, 48, 64, 0.5),
    (1, 1, 300, 24, 128, 0.25),
    (1, 4, 2048, 256, 32, 1.0),         # latent count and head dim of the headline case
    (1, 2, 1500, 512, 32, 1.0),         # more than 256 latents: blocks of 256 merged by log-sum-exp
    (2, 1, 700, 320, 32, 0.7),          # a full block and a 64-latent one
])
def test_parity_fwd_bwd(fb, cuda_dev, path, dtype, B, H, N, M, D, scale):
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=N + M)
    prev = fb.set_kernel_path(path)
    try:
        got = run_mixer(fb, q, k, v, dy, scale, cuda_dev)
    finally:
        fb.set_kernel_path(prev)
    assert_close(got, oracle_all(q, k, v, dy, scale), TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,N,M,D", [
    (1, 2, 1000, 256, 32),      # ragged last tile, two 128-latent blocks
    (2, 2, 2048, 192, 32),      # second latent block half full
    (1, 3, 700, 128, 32),       # one block
    (1, 1, 128 * 37 + 5, 256, 32),
    (2, 1, 300, 64, 16),
    (1, 2, 900, 640, 32),       # more than 256 latents: blocks of 256 that add into dk, dv
])
def test_general_tensor_core_backward(fb, cuda_dev, dtype, B, H, N, M, D):
    """The two-exponential tensor-core backward on its own (it otherwise only takes the (b, h) the range
    check hands it, masks, single terms and fp16)."""
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=11)
    prev = fb.set_kernel_path("tc_exact")
    try:
        tc0, simt0 = fb.pass_counts()
        got = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev)
        tc1, simt1 = fb.pass_counts()
    finally:
        fb.set_kernel_path(prev)
    assert simt1 == simt0 and tc1 - tc0 == 4      # gather, scatter, dZ, main backward
    assert_close(got, oracle_all(q, k, v, dy, 1.0), 2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_lra_shape_with_mask_stays_on_tensor_cores(fb, cuda_dev, dtype):
    """The LRA configuration (out/lra/run.sh:32-93: C=128, H=8, M=128, N up to 4096) with the key-padding
    mask every LRA batch carries (lra/models/backends.py:602-622); a smaller batch than 32 keeps the
    oracle quick."""
    B, H, N, M, D = 4, 8, 4096, 128, 16
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=31)
    lens = torch.tensor([N, 3000, 1025, 130])
    mask = torch.arange(N)[None, :] < lens[:, None]
    tc0, simt0 = fb.pass_counts()
    got = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev, key_mask=mask)
    tc1, simt1 = fb.pass_counts()
    assert simt1 == simt0 and tc1 - tc0 == 4
    assert fb.device_status() == 0
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    y = O.mixer_lra(qf, kf, vf, 1.0, mask)
    y.backward(dy.float())
    assert_close(got, [y.detach(), qf.grad, kf.grad, vf.grad], 2e-2)


def test_scattered_mask_bits(fb, cuda_dev):
    """A mask that is not a prefix: kept and dropped tokens alternate irregularly inside tiles."""
    B, H, N, M, D = 2, 2, 1000, 96, 32
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=torch.bfloat16, seed=41)
    mask = torch.rand(B, N, generator=torch.Generator().manual_seed(1)) < 0.6
    mask[1, :300] = False                        # whole tiles dropped, first ones included
    got = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev, key_mask=mask)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    y = O.mixer_lra(qf, kf, vf, 1.0, mask)
    y.backward(dy.float())
    assert_close(got, [y.detach(), qf.grad, kf.grad, vf.grad], 2e-2)


def test_single_token(fb, cuda_dev):
    # N = 1: z = v, y = v and every gradient of q and k vanishes identically
    q, k, v, dy = O.make_inputs(3, 2, 1, 16, 16, seed=17)
    y, dq, dk, dv = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev)
    ref = oracle_all(q, k, v, dy, 1.0)
    assert O.rel_l2(y, ref[0]) <= 1e-5 and O.rel_l2(dv, ref[3]) <= 1e-5
    assert dq.abs().max() <= 1e-5 and dk.abs().max() <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_strided_head_views_and_expanded_q(fb, cuda_dev, dtype):
    # k, v as the 'b n (h d) -> b h n d' views of flare.py:127-128; q expanded as in flare.py:136
    B, H, N, M, D = 2, 4, 600, 32, 16
    g = torch.Generator().manual_seed(11)
    kx = (torch.randn(B, N, H * D, generator=g) * D ** -0.25).to(dtype)
    vx = (torch.randn(B, N, H * D, generator=g) * D ** -0.25).to(dtype)
    q = (torch.randn(H, M, D, generator=g) * D ** -0.25).to(dtype)
    dy = torch.randn(B, N, H * D, generator=g).to(dtype)
    dev = cuda_dev
    kd, vd, qd = (t.to(dev).requires_grad_(True) for t in (kx, vx, q))
    k4 = kd.view(B, N, H, D).permute(0, 2, 1, 3)
    v4 = vd.view(B, N, H, D).permute(0, 2, 1, 3)
    y = fb.flare_multihead_mixer(qd.unsqueeze(0).expand(B, -1, -1, -1), k4, v4)
    assert y.shape == (B, H, N, D)
    yc = y.permute(0, 2, 1, 3).reshape(B, N, H * D)
    yc.backward(dy.to(dev))
    torch.cuda.synchronize()
    ko = kx.view(B, N, H, D).permute(0, 2, 1, 3)
    vo = vx.view(B, N, H, D).permute(0, 2, 1, 3)
    dyo = dy.view(B, N, H, D).permute(0, 2, 1, 3)
    ref = oracle_all(q, ko, vo, dyo, 1.0)
    got = [y.float().cpu(), qd.grad.float().cpu(),
           kd.grad.float().cpu().view(B, N, H, D).permute(0, 2, 1, 3),
           vd.grad.float().cpu().view(B, N, H, D).permute(0, 2, 1, 3)]
    assert_close(got, ref, TOL[dtype])


def test_batched_q(fb, cuda_dev):
    B, H, N, M, D = 2, 2, 200, 16, 16
    _, k, v, dy = O.make_inputs(B, H, N, M, D, seed=4)
    q = torch.randn(B, H, M, D, generator=torch.Generator().manual_seed(5)) * 0.5
    got = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev)
    y = O.mixer_sdpa(q, k, v, 1.0)
    ref = [y, *O.mixer_bwd_closed_form(q, k, v, dy, 1.0)]
    assert got[1].shape == (B, H, M, D)
    assert_close(got, ref, 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_key_mask(fb, cuda_dev, dtype):
    B, H, N, M, D = 3, 2, 333, 32, 32
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=9)
    lens = torch.tensor([N, 200, 1])
    mask = torch.arange(N)[None, :] < lens[:, None]
    got = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev, key_mask=mask)
    qf, kf, vf, dyf = (t.float().requires_grad_(True) if i < 3 else t.float() for i, t in enumerate((q, k, v, dy)))
    y = O.mixer_lra(qf, kf, vf, 1.0, mask)
    y.backward(dyf)
    assert_close(got, [y.detach(), qf.grad, kf.grad, vf.grad], TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gather_and_scatter_as_separate_ops(fb, cuda_dev, dtype):
    # BigFLARE (pdebench/models/flare_ablations.py:93-132) edits z between the two calls
    B, H, N, M, D = 2, 2, 500, 32, 16
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=21)
    dev = cuda_dev
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    z, lse = fb.flare_gather(qd, kd, vd, scale=0.7)
    z2 = z * 1.5 + 0.25
    y = fb.flare_scatter(qd, kd, z2, scale=0.7)
    y.backward(dy.to(dev))
    torch.cuda.synchronize()
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    zr, Lr = O.gather(qf, kf, vf, 0.7)
    yr, _ = O.scatter(qf, kf, zr * 1.5 + 0.25, 0.7)
    yr.backward(dy.float())
    tol = TOL[dtype]
    assert O.rel_l2(z.float().cpu(), zr.detach()) <= tol
    assert O.rel_l2(lse.cpu(), Lr.detach()) <= max(tol, 1e-5)
    got = [y.float().cpu(), qd.grad.float().cpu(), kd.grad.float().cpu(), vd.grad.float().cpu()]
    # z is rounded to the input dtype between the two ops, as in the reference
    assert_close(got, [yr.detach(), qf.grad, kf.grad, vf.grad], tol * (1 if dtype == torch.float32 else 1.5))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_separate_ops_backward_on_tensor_cores(fb, cuda_dev, dtype):
    """Gather-only and scatter-only backward terms (BigFLARE trains through them) at a size with several
    token ranges, served by the general tensor-core backward."""
    B, H, N, M, D = 1, 2, 65536, 256, 32
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=23)
    dev = cuda_dev
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    tc0, simt0 = fb.pass_counts()
    z, lse = fb.flare_gather(qd, kd, vd, scale=1.0)
    z2 = z * 1.5                                  # the latents are edited between the two operators
    y = fb.flare_scatter(qd, kd, z2, scale=1.0)
    y.backward(dy.to(dev))
    torch.cuda.synchronize()
    tc1, simt1 = fb.pass_counts()
    assert simt1 == simt0 and tc1 - tc0 == 5      # gather, scatter, dZ, scatter-term backward, gather-term backward
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    zr, _ = O.gather(qf, kf, vf, 1.0)
    zr2 = (zr.to(dtype) * 1.5).float()            # z crosses the boundary between the two operators in `dtype`
    yr, _ = O.scatter(qf, kf, zr2, 1.0)
    yr.backward(dy.float())
    got = [y.float().cpu(), qd.grad.float().cpu(), kd.grad.float().cpu(), vd.grad.float().cpu()]
    assert_close(got, [yr.detach(), qf.grad, kf.grad, vf.grad], 3e-2)


def test_partial_records_and_combine_match_oracle(fb, cuda_dev):
    import ctypes as C
    from flare_b200 import _cabi
    from flare_b200.mixer import make_problem
    B, H, N, M, D = 1, 2, 1000, 48, 16
    q, k, v, _ = O.make_inputs(B, H, N, M, D, seed=2)
    dev = cuda_dev
    qd, kd, vd = (t.to(dev) for t in (q, k, v))
    S = 5                                        # ranges of 256 tokens; the last one is empty
    p = make_problem(qd, kd, 1.0, n_splits=S, v=vd)
    rec = torch.full((S, B, H, M, D + 2), float("nan"), device=dev)
    _cabi.check(_cabi.lib.flare_gather_partial(C.byref(p), qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), None,
                                               rec.data_ptr(), None), "gather_partial")
    torch.cuda.synchronize()
    bounds = [(i * 256, min(N, (i + 1) * 256)) for i in range(S)]
    bounds[-1] = (N, N)
    m, l, acc = O.gather_partials(q, k, v, 1.0, bounds)
    r = rec.cpu()
    assert torch.equal(torch.isinf(r[..., D]), torch.isinf(m))
    z_ref, L_ref = O.lse_combine(m, l, acc)
    z_rec, L_rec = O.lse_combine(r[..., D], r[..., D + 1], r[..., :D])
    assert O.rel_l2(z_rec, z_ref) <= 1e-5 and O.rel_l2(L_rec, L_ref) <= 1e-5
    z32 = torch.empty(B, H, M, D, device=dev)
    lse = torch.empty(B, H, M, device=dev)
    merged = torch.empty(B, H, M, D + 2, device=dev)
    _cabi.check(_cabi.lib.flare_combine(C.byref(p), rec.data_ptr(), S, z32.data_ptr(), None, lse.data_ptr(),
                                        merged.data_ptr(), None), "combine")
    torch.cuda.synchronize()
    assert O.rel_l2(z32.cpu(), z_ref) <= 1e-5 and O.rel_l2(lse.cpu(), L_ref) <= 1e-5
    mm = merged.cpu()
    z_m, L_m = O.lse_combine(mm[None, ..., D], mm[None, ..., D + 1], mm[None, ..., :D])
    assert O.rel_l2(z_m, z_ref) <= 1e-5


def test_deterministic(fb, cuda_dev):
    q, k, v, dy = O.make_inputs(1, 4, 3000, 64, 32, dtype=torch.bfloat16, seed=1)
    a = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev)
    b = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_cpu_tensors_are_rejected(fb):
    q, k, v, _ = O.make_inputs(1, 1, 16, 8, 8)
    with pytest.raises(RuntimeError):
        fb.flare_multihead_mixer(q, k, v)


def test_large_scores_are_stable(fb, cuda_dev):
    # logits of magnitude ~60: exercises the running-max rescaling of the gather
    q, k, v, dy = O.make_inputs(1, 2, 700, 32, 16, seed=8)
    got = run_mixer(fb, q * 6, k * 6, v, dy, 1.0, cuda_dev)
    assert_close(got, oracle_all(q * 6, k * 6, v, dy, 1.0), 2e-5)


@pytest.mark.parametrize("M", [256, 512])
def test_wide_score_range_takes_the_exact_path(fb, cuda_dev, M):
    """bf16 logits of magnitude ~60: the on-device range check rejects the one-exponential backward; at
    M = 256 the exact tensor-core kernel takes over, above 256 latents the fp32 kernels do."""
    q, k, v, dy = O.make_inputs(1, 2, 900, M, 32, dtype=torch.bfloat16, seed=21)
    q, k = (q.float() * 4).bfloat16(), (k.float() * 4).bfloat16()
    got = run_mixer(fb, q, k, v, dy, 1.0, cuda_dev)
    assert_close(got, oracle_all(q, k, v, dy, 1.0), 2e-2)


def test_full_size_properties(fb, cuda_dev):
    """The benchmark's own size (B=1, H=8, N=2^20, M=256, D=32, bf16), where the CPU oracle is out of reach:
    (1) the tensor-core path agrees with the fp32 kernels (themselves checked against the oracle above);
    (2) the backward is linear in dy: doubling dy doubles every gradient bit for bit (powers of two scale
        exactly through every product, sum and bf16 rounding of the path)."""
    B, H, N, M, D = 1, 8, 1 << 20, 256, 32
    g = torch.Generator(device="cpu").manual_seed(99)
    sd = D ** -0.25
    q = (torch.randn(H, M, D, generator=g) * sd).bfloat16().to(cuda_dev)
    k = (torch.randn(B, H, N, D, generator=g) * sd).bfloat16().to(cuda_dev)
    v = (torch.randn(B, H, N, D, generator=g) * sd).bfloat16().to(cuda_dev)
    dy = torch.randn(B, H, N, D, generator=g).bfloat16().to(cuda_dev)

    def run(path, dy_):
        prev = fb.set_kernel_path(path)
        try:
            qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
            y = fb.flare_multihead_mixer(qd, kd, vd)
            y.backward(dy_)
            torch.cuda.synchronize()
            return y.detach(), qd.grad, kd.grad, vd.grad
        finally:
            fb.set_kernel_path(prev)

    def rel(a, b):
        a, b = a.float(), b.float()
        return ((a - b).norm() / b.norm()).item()

    tc = run("auto", dy)
    ref = run("simt", dy)
    errs = {n: rel(a, b) for n, a, b in zip(("y", "dq", "dk", "dv"), tc, ref)}
    assert all(e <= 2e-2 for e in errs.values()), errs
    tc2 = run("auto", dy * 2)
    assert torch.equal(tc2[0], tc[0])
    for n, a, b in zip(("dq", "dk", "dv"), tc2[1:], tc[1:]):
        assert torch.equal(a.float(), b.float() * 2), n


# ------------------------------------------------------------------------------------------------
# the call-site variants of the reference that share this path
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shared_latents_expanded_over_heads(fb, cuda_dev, dtype):
    """BigFLARE's shared_latents (pdebench/models/flare_ablations.py:100-101): one [M,D] latent set expanded
    (stride 0) over the heads; its gradient is the sum over heads."""
    B, H, N, M, D = 2, 4, 700, 64, 32
    _, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=51)
    q1 = (torch.randn(1, M, D, generator=torch.Generator().manual_seed(52)) * D ** -0.25).to(dtype)
    dev = cuda_dev
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q1, k, v))
    tc0, simt0 = fb.pass_counts()
    y = fb.flare_multihead_mixer(qd.expand(H, -1, -1).unsqueeze(0).expand(B, -1, -1, -1), kd, vd)
    y.backward(dy.to(dev))
    torch.cuda.synchronize()
    tc1, simt1 = fb.pass_counts()
    if dtype == torch.bfloat16:
        assert simt1 == simt0 and tc1 - tc0 == 4
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q1, k, v))
    yr = O.mixer_sdpa(qf.expand(H, -1, -1), kf, vf, 1.0)
    yr.backward(dy.float())
    got = [y.float().cpu(), qd.grad.float().cpu(), kd.grad.float().cpu(), vd.grad.float().cpu()]
    assert got[1].shape == (1, M, D)
    assert_close(got, [yr.detach(), qf.grad, kf.grad, vf.grad], TOL[dtype])


def test_qk_norm_and_output_gate_variants(fb, cuda_dev):
    """qk_norm (pdebench/models/flare.py:130-132: a LayerNorm over D on q and k in front of the two calls) and
    the sigmoid output gate of pdebench/models/unloopy.py:98-101: both stay in torch around the operator and
    must differentiate through it."""
    torch.manual_seed(3)
    B, N, C, H, M = 2, 300, 64, 4, 32
    D = C // H
    dev = cuda_dev
    att = fb.FLARE(channel_dim=C, num_heads=H, num_latents=M, qk_norm=True).to(dev)
    gate = torch.nn.Linear(C, C).to(dev)
    x = torch.randn(B, N, C, device=dev, requires_grad=True)

    def run(fused):
        x.grad = None
        att.zero_grad(set_to_none=True)
        gate.zero_grad(set_to_none=True)
        y, _ = att(x, return_scores=not fused)              # the materialising branch is plain torch (attn_scale = 1)
        out = (y * gate(x).sigmoid()).square().mean()
        out.backward()
        return out.item(), x.grad.clone(), att.latent_q.grad.clone(), att.k_norm.weight.grad.clone()

    a, b = run(True), run(False)
    assert abs(a[0] - b[0]) <= 1e-5 * abs(b[0])
    for u, w in zip(a[1:], b[1:]):
        assert O.rel_l2(u.cpu(), w.cpu()) <= 1e-4
