"""Attention dropout inside the tensor-core kernels (lra/models/backends.py:604-606: dropout_p on both SDPA calls).

The keep masks are a counter hash, so the host can recompute them (oracle.dropout_keep_masks): the kernels are
checked exactly -- forward and backward -- against the dense two-softmax form with THOSE masks, and
statistically (keep rate, unbiasedness over seeds) as torch's own dropout would be.
"""
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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,N,M,D,p,masked", [
    (2, 2, 700, 64, 16, 0.1, False),
    (1, 2, 1100, 256, 32, 0.25, False),
    (2, 4, 500, 128, 16, 0.1, True),          # the LRA combination: key-padding mask and dropout
    (1, 1, 300, 320, 32, 0.5, False),         # more than 256 latents
])
def test_forward_and_backward_with_the_kernels_own_masks(fb, cuda_dev, dtype, B, H, N, M, D, p, masked):
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=N + M)
    seed = 0x1234_5678_9ABC_DEF0 + N
    mask = None
    if masked:
        mask = torch.arange(N)[None, :] < torch.tensor([N, N // 2 + 3][:B])[:, None]
    dev = cuda_dev
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    tc0, simt0 = fb.pass_counts()
    y = fb.flare_multihead_mixer(qd, kd, vd, key_mask=None if mask is None else mask.to(dev), dropout_p=p, dropout_seed=seed)
    y.backward(dy.to(dev))
    torch.cuda.synchronize()
    tc1, simt1 = fb.pass_counts()
    assert simt1 == simt0 and tc1 - tc0 == 4 and fb.device_status() == 0
    keep1, keep2 = O.dropout_keep_masks(B, H, M, N, p, seed)
    assert abs(keep1.float().mean().item() - (1 - p)) < 0.01 and abs(keep2.float().mean().item() - (1 - p)) < 0.01
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    yr = O.mixer_dropout(qf, kf, vf, 1.0, keep1, keep2, p, mask)
    yr.backward(dy.float())
    errs = {n: O.rel_l2(a.float().cpu(), b) for n, a, b in
            zip(("y", "dq", "dk", "dv"), (y, qd.grad, kd.grad, vd.grad), (yr.detach(), qf.grad, kf.grad, vf.grad))}
    assert all(e <= 2e-2 for e in errs.values()), errs


def test_dropout_is_unbiased_and_seeded(fb, cuda_dev):
    B, H, N, M, D, p = 1, 2, 512, 64, 32, 0.2
    q, k, v, _ = O.make_inputs(B, H, N, M, D, dtype=torch.bfloat16, seed=3)
    qd, kd, vd = (t.to(cuda_dev) for t in (q, k, v))
    y0 = fb.flare_multihead_mixer(qd, kd, vd).float()
    torch.manual_seed(7)
    a1 = fb.flare_multihead_mixer(qd, kd, vd, dropout_p=p)
    a2 = fb.flare_multihead_mixer(qd, kd, vd, dropout_p=p)
    assert not torch.equal(a1, a2)                                   # a new mask per call
    runs = [fb.flare_multihead_mixer(qd, kd, vd, dropout_p=p, dropout_seed=s).float() for s in range(64)]
    mean = torch.stack(runs).mean(0)
    # E[y] = y without dropout (both masks are independent and rescaled); 64 draws leave a few per cent of noise
    assert O.rel_l2(mean.cpu(), y0.cpu()) < 0.1
    assert O.rel_l2(runs[0].cpu(), y0.cpu()) > 0.1                   # a single draw is visibly perturbed
    again = fb.flare_multihead_mixer(qd, kd, vd, dropout_p=p, dropout_seed=5).float()
    assert torch.equal(again, runs[5])                               # same seed, same masks


def test_dropout_in_the_lra_module_only_while_training(fb, cuda_dev):
    from flare_b200.modules import LraFLARE
    torch.manual_seed(0)
    att = LraFLARE(channel_dim=64, num_heads=4, num_latents=32, kv_proj_hidden_dim=64, attn_drop=0.3).to(cuda_dev).bfloat16()
    x = torch.randn(2, 200, 64, device=cuda_dev).bfloat16()
    att.eval()
    assert torch.equal(att(x), att(x))
    att.train()
    assert not torch.equal(att(x), att(x))
