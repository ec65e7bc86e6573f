"""The registered torch operators on fake tensors: the shapes, strides and dtypes torch.compile will see,
without a GPU.  (The autograd engine itself needs a live device for CUDA tensors, so the backward operators
are called directly here; differentiation end to end is covered by the GPU tests.)"""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import flare_b200 as fb

ops = torch.ops.flare_b200


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_mixer_operator_shapes_on_fake_tensors(dtype):
    B, H, N, M, D = 2, 4, 300, 32, 16
    with FakeTensorMode():
        x = torch.empty(B, N, H * D, dtype=dtype, device="cuda")
        k = x.view(B, N, H, D).permute(0, 2, 1, 3)           # the 'b n (h d) -> b h n d' view of the reference
        v = (x * 2).view(B, N, H, D).permute(0, 2, 1, 3)
        q = torch.empty(H, M, D, dtype=dtype, device="cuda", requires_grad=True)
        y = fb.flare_multihead_mixer(q.unsqueeze(0).expand(B, -1, -1, -1), k, v, scale=0.5)
        assert y.shape == (B, H, N, D) and y.dtype == dtype and y.requires_grad
        assert y.stride() == k.stride()                      # 'b h n d -> b n (h d)' stays a free view
        y0, z32, lse_m, lse_n = ops.mixer_fwd(q, k, v, 0.5, None, 0.0, 0)
        assert z32.shape == (B, H, M, D) and lse_m.shape == (B, H, M) and lse_n.shape == (B, H, N)
        dq, dk, dv = ops.mixer_bwd(q, k, v, torch.empty_like(y0), y0, z32, lse_m, lse_n, 0.5, None, 0.0, 0)
        assert dq.shape == q.shape and dq.dtype == torch.float32
        assert dk.shape == k.shape and dk.stride() == k.stride() and dv.dtype == dtype


def test_separate_operators_on_fake_tensors():
    B, H, N, M, D = 1, 2, 100, 16, 32
    with FakeTensorMode():
        q = torch.empty(H, M, D, device="cuda", requires_grad=True)
        k = torch.empty(B, H, N, D, device="cuda")
        v = torch.empty(B, H, N, D, device="cuda")
        mask = torch.ones(B, N, dtype=torch.bool, device="cuda")
        z, lse = fb.flare_gather(q, k, v, key_mask=mask)
        assert z.shape == (B, H, M, D) and lse.shape == (B, H, M) and not lse.requires_grad
        y = fb.flare_scatter(q, k, z * 2, key_mask=mask)
        assert y.shape == (B, H, N, D) and y.requires_grad
        dq, dk, dz = ops.scatter_bwd(q, k, z, torch.empty_like(y), y, torch.empty(B, H, N, device="cuda"), 1.0, mask)
        assert dq.shape == q.shape and dk.shape == k.shape and dz.shape == z.shape
        dq, dk, dv = ops.gather_bwd(q, k, v, dz, torch.empty(B, H, M, D, device="cuda"), lse, 1.0, mask)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape


def test_autocast_casts_the_latents_like_sdpa(monkeypatch):
    B, H, N, M, D = 1, 2, 64, 8, 16
    state = {"on": False}
    # torch.autocast("cuda") switches itself off on a machine without a GPU: stand in for its two queries
    monkeypatch.setattr(torch, "is_autocast_enabled", lambda *a: state["on"])
    monkeypatch.setattr(torch, "get_autocast_dtype", lambda *a: torch.float16)
    with FakeTensorMode():
        q = torch.empty(H, M, D, device="cuda", requires_grad=True)              # fp32 parameter
        k = torch.empty(B, H, N, D, device="cuda", dtype=torch.float16)
        v = torch.empty(B, H, N, D, device="cuda", dtype=torch.float16)
        state["on"] = True
        y = fb.flare_multihead_mixer(q, k, v)
        state["on"] = False
        assert y.dtype == torch.float16 and y.requires_grad
        with pytest.raises(TypeError):
            fb.flare_multihead_mixer(q, k, v)                                    # no autocast: dtypes must agree
        y = fb.flare_multihead_mixer(q.half(), k, v, dropout_p=0.1)               # dropout: a seed is drawn on the host
        assert y.shape == k.shape
        with pytest.raises(NotImplementedError):
            fb.flare_multihead_mixer(q, k.float(), v.float(), dropout_p=0.1)      # fp32 has no dropout kernels
        with pytest.raises(ValueError):
            fb.flare_multihead_mixer(q.half(), k, v, dropout_p=1.0)
