"""Causal FLARE on the GPU against the CPU oracle (dense and recurrent forms).

The reference has no code for this path, so the oracle itself is checked for self-consistency
(tests/test_oracle.py); here the CUDA prefill and decode are compared with it.
"""
import pytest
import torch

from oracle import flare_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2, torch.float16: 5e-3}


def _inputs(B, H, N, M, D, dtype, seed=0):
    q, k, v, _ = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=seed)
    return q, k, v


@pytest.mark.parametrize("B,H,N,M,D,dtype", [
    (1, 2, 64, 32, 32, torch.float32),
    (2, 2, 200, 64, 32, torch.float32),       # ragged: 1.56 chunks, partial sub-chunk
    (1, 2, 384, 128, 64, torch.float32),      # the serving shape's M and D
    (1, 2, 300, 256, 32, torch.bfloat16),
    (2, 3, 257, 128, 64, torch.bfloat16),
    (1, 1, 130, 64, 16, torch.float16),
])
def test_prefill_matches_oracle(cuda_dev, B, H, N, M, D, dtype):
    import flare_b200 as fb
    q, k, v = _inputs(B, H, N, M, D, dtype)
    y_ref, (m_ref, l_ref, a_ref) = O.causal_recurrent(q.double(), k.double(), v.double(), 1.0)
    y, st = fb.flare_causal_prefill(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev), 1.0)
    assert O.rel_l2(y.double().cpu(), y_ref) <= TOL[dtype]
    # the final record, compared through what it represents: z = acc / l and lse = m + log l
    st = st.double().cpu()
    z = st[..., :D] / st[..., D + 1:D + 2]
    lse = st[..., D] + torch.log(st[..., D + 1])
    assert O.rel_l2(z, a_ref / l_ref[..., None]) <= TOL[dtype]
    assert O.rel_l2(lse, m_ref + torch.log(l_ref)) <= TOL[dtype]


def test_prefill_dense_small(cuda_dev):
    import flare_b200 as fb
    q, k, v = _inputs(1, 2, 40, 16, 16, torch.float32, seed=3)
    y_ref = O.causal_dense(q.double(), k.double(), v.double(), 0.7)
    y, _ = fb.flare_causal_prefill(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev), 0.7)
    assert O.rel_l2(y.double().cpu(), y_ref) <= 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_continues_prefill(cuda_dev, dtype):
    """prefill(first part) then token-by-token decode == prefill(everything)."""
    import flare_b200 as fb
    B, H, N, M, D = 2, 2, 160, 64, 32
    q, k, v = _inputs(B, H, N, M, D, dtype, seed=5)
    qd, kd, vd = q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev)
    y_all, st_all = fb.flare_causal_prefill(qd, kd, vd, 1.0)
    n0 = 100
    y0, st = fb.flare_causal_prefill(qd, kd[:, :, :n0], vd[:, :, :n0], 1.0)
    ys = [y0]
    for t in range(n0, N - 8):
        ys.append(fb.flare_causal_decode(qd, kd[:, :, t:t + 1], vd[:, :, t:t + 1], st, 1.0))
    ys.append(fb.flare_causal_decode(qd, kd[:, :, N - 8:], vd[:, :, N - 8:], st, 1.0))   # several tokens in one call
    y_inc = torch.cat(ys, dim=2)
    y_ref, _ = O.causal_recurrent(q.double(), k.double(), v.double(), 1.0)
    assert O.rel_l2(y_inc.double().cpu(), y_ref) <= TOL[dtype]
    assert O.rel_l2(y_inc.double().cpu(), y_all.double().cpu()) <= TOL[dtype]


def test_decode_from_empty_state(cuda_dev):
    import flare_b200 as fb
    B, H, N, M, D = 1, 2, 24, 32, 32
    q, k, v = _inputs(B, H, N, M, D, torch.float32, seed=7)
    st = fb.causal_state_init(B, H, M, D, cuda_dev)
    y = fb.flare_causal_decode(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev), st, 1.0)
    y_ref, _ = O.causal_recurrent(q.double(), k.double(), v.double(), 1.0)
    assert O.rel_l2(y.double().cpu(), y_ref) <= 2e-5


def test_prefill_with_prior_state(cuda_dev):
    import flare_b200 as fb
    B, H, N, M, D = 1, 2, 300, 64, 32
    q, k, v = _inputs(B, H, N, M, D, torch.float32, seed=9)
    qd, kd, vd = q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev)
    _, st = fb.flare_causal_prefill(qd, kd[:, :, :128], vd[:, :, :128], 1.0)
    y2, _ = fb.flare_causal_prefill(qd, kd[:, :, 128:], vd[:, :, 128:], 1.0, state=st)
    y_ref, _ = O.causal_recurrent(q.double(), k.double(), v.double(), 1.0)
    assert O.rel_l2(y2.double().cpu(), y_ref[:, :, 128:]) <= 2e-5


def test_unsupported_shape_is_refused(cuda_dev):
    import flare_b200 as fb
    q, k, v = _inputs(1, 1, 16, 520, 64, torch.float32)
    with pytest.raises(Exception):
        fb.flare_causal_prefill(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev), 1.0)


def test_serving_shape_split_prefill(cuda_dev):
    """B=4, H=16, N=8192, D=64, M=128 bf16 (too large for the CPU oracle): prefilling the prompt in two pieces
    with the carried record, and decoding its last tokens one by one, give what one prefill gives."""
    import flare_b200 as fb
    B, H, N, M, D = 4, 16, 8192, 128, 64
    g = torch.Generator().manual_seed(31)
    q = (torch.randn(H, M, D, generator=g) * D ** -0.25).bfloat16().to(cuda_dev)
    k = (torch.randn(B, H, N, D, generator=g) * D ** -0.25).bfloat16().to(cuda_dev)
    v = torch.randn(B, H, N, D, generator=g).bfloat16().to(cuda_dev)
    y_all, st_all = fb.flare_causal_prefill(q, k, v, 1.0)
    n0 = 5000                                            # not a multiple of the chunk
    y0, st = fb.flare_causal_prefill(q, k[:, :, :n0], v[:, :, :n0], 1.0)
    y1, st = fb.flare_causal_prefill(q, k[:, :, n0:N - 16], v[:, :, n0:N - 16], 1.0, state=st)
    ys = [y0, y1]
    for t in range(N - 16, N):
        ys.append(fb.flare_causal_decode(q, k[:, :, t:t + 1], v[:, :, t:t + 1], st, 1.0))
    y_inc = torch.cat(ys, dim=2)
    err = ((y_inc.float() - y_all.float()).norm() / y_all.float().norm()).item()
    assert err <= 2e-2, err
    z_a = st_all[..., :D] / st_all[..., D + 1:D + 2]
    z_b = st[..., :D] / st[..., D + 1:D + 2]
    assert ((z_a - z_b).norm() / z_a.norm()).item() <= 2e-2


@pytest.mark.parametrize("B,H,N,M,D,shared", [
    (1, 2, 128, 128, 32, False),     # exactly one chunk
    (2, 2, 333, 128, 64, True),      # ragged last chunk, latents shared by the batch
    (1, 3, 700, 64, 64, False),      # fewer latents than tensor-memory lanes
    (2, 1, 130, 96, 32, True),
    (1, 1, 5, 32, 32, False),        # a handful of tokens
])
def test_prefill_tensor_core_walk_shapes(cuda_dev, B, H, N, M, D, shared):
    """bf16 with M <= 128 and D in {32, 64} takes the tensor-core walk; state carried from a prior prefill too."""
    import flare_b200 as fb
    q, k, v = _inputs(B, H, N, M, D, torch.bfloat16, seed=11)          # q: [H, M, D]
    if not shared:                                                      # one latent set per batch element
        q = (torch.randn(B, H, M, D, generator=torch.Generator().manual_seed(12)) * D ** -0.25).bfloat16()
    y_ref, (m_ref, l_ref, a_ref) = O.causal_recurrent(q.double(), k.double(), v.double(), 0.9)
    qd, kd, vd = q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev)
    y, st = fb.flare_causal_prefill(qd, kd, vd, 0.9)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    assert O.rel_l2(y.double().cpu(), y_ref) <= 2e-2
    if N > 64:                                           # split anywhere: the second call starts from a record
        n0 = N // 3
        y0, st0 = fb.flare_causal_prefill(qd, kd[:, :, :n0].contiguous(), vd[:, :, :n0].contiguous(), 0.9)
        y1, _ = fb.flare_causal_prefill(qd, kd[:, :, n0:].contiguous(), vd[:, :, n0:].contiguous(), 0.9, state=st0)
        assert O.rel_l2(torch.cat([y0, y1], 2).double().cpu(), y_ref) <= 2e-2


def test_prefill_replays_from_a_cuda_graph(cuda_dev):
    """The four chained launches of the tensor-core prefill (records, scan, walk, redo pass) recorded once and replayed
    on new inputs written into the same buffers."""
    import flare_b200 as fb
    B, H, N, M, D = 2, 2, 700, 128, 64
    q, k, v = _inputs(B, H, N, M, D, torch.bfloat16, seed=17)
    q2, k2, v2 = _inputs(B, H, N, M, D, torch.bfloat16, seed=18)
    qd, kd, vd = q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev)
    side = torch.cuda.Stream(device=cuda_dev)
    side.wait_stream(torch.cuda.current_stream(cuda_dev))
    with torch.cuda.stream(side):
        fb.flare_causal_prefill(qd, kd, vd, 1.0)                     # warm-up outside the recording
    torch.cuda.current_stream(cuda_dev).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y, st = fb.flare_causal_prefill(qd, kd, vd, 1.0)
    for qq, kk, vv in ((q, k, v), (q2, k2, v2)):
        qd.copy_(qq.to(cuda_dev)); kd.copy_(kk.to(cuda_dev)); vd.copy_(vv.to(cuda_dev))
        graph.replay()
        torch.cuda.synchronize()
        y_ref, _ = O.causal_recurrent(qq.double(), kk.double(), vv.double(), 1.0)
        assert O.rel_l2(y.double().cpu(), y_ref) <= 2e-2
    assert fb.device_status() == 0


def test_prefill_tensor_core_walk_hands_wide_chunks_to_the_fp32_walk(cuda_dev):
    """Scores that climb by hundreds of octaves inside one chunk: the tensor-core walk keeps one reference
    maximum per chunk, flags such chunks, and the fp32 walk with a running maximum redoes them."""
    import flare_b200 as fb
    B, H, N, M, D = 1, 2, 384, 64, 32
    q, k, v = _inputs(B, H, N, M, D, torch.bfloat16, seed=13)
    ramp = torch.ones(N)
    ramp[128:256] = torch.linspace(1.0, 60.0, 128)       # the middle chunk only
    k = (k.float() * ramp[None, None, :, None]).bfloat16()
    y_ref, _ = O.causal_recurrent(q.double(), k.double(), v.double(), 1.0)
    y, _ = fb.flare_causal_prefill(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev), 1.0)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    assert torch.isfinite(y.float()).all()
    assert O.rel_l2(y.double().cpu(), y_ref) <= 2e-2


# ---------------------------------------------------------------------------------------------------------
# backward (flare_causal_mixer): against autograd through the dense definition and the chunked restatement
# ---------------------------------------------------------------------------------------------------------
def _fb():
    import flare_b200 as fb
    return fb


def _bwd_case(fb, dev, B, H, N, M, D, dtype, scale, seed):
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=seed)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    y = fb.flare_causal_mixer(qd, kd, vd, scale)
    y.backward(dy.to(dev))
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    return (q, k, v, dy), (y.detach().cpu(), qd.grad.cpu(), kd.grad.cpu(), vd.grad.cpu())


@pytest.mark.parametrize("B,H,N,M,D", [(1, 2, 96, 16, 16), (2, 2, 300, 32, 32), (1, 1, 257, 64, 64), (1, 2, 129, 128, 64)])
def test_backward_matches_autograd_of_the_dense_definition(cuda_dev, B, H, N, M, D):
    """fp32 kernel against fp64 autograd through causal_dense: ragged ends (N not a multiple of 32 or 128),
    one to three chunks, every supported head dim."""
    fb = _fb()
    (q, k, v, dy), (y, dq, dk, dv) = _bwd_case(fb, cuda_dev, B, H, N, M, D, torch.float32, 0.8, seed=21)
    qf, kf, vf, dyf = (t.double() for t in (q, k, v, dy))
    dq_ref, dk_ref, dv_ref = O.causal_bwd_autograd(qf, kf, vf, dyf, 0.8)
    assert O.rel_l2(y.double(), O.causal_dense(qf, kf, vf, 0.8)) <= 1e-5
    assert O.rel_l2(dq.double(), dq_ref) <= 1e-4
    assert O.rel_l2(dk.double(), dk_ref) <= 1e-4
    assert O.rel_l2(dv.double(), dv_ref) <= 1e-4


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2), (torch.float16, 5e-3)])
def test_backward_long_sequence_against_the_chunked_restatement(cuda_dev, dtype, tol):
    """N = 2000 (16 chunks, ragged last one), latents shared by two batch entries: the carried suffix state
    crosses many chunk boundaries.  The yardstick is the oracle's reverse chunk scan in fp64 on the same
    rounded inputs (itself pinned to autograd on small cases in the CPU suite)."""
    fb = _fb()
    B, H, N, M, D = 2, 2, 2000, 32, 32
    (q, k, v, dy), (y, dq, dk, dv) = _bwd_case(fb, cuda_dev, B, H, N, M, D, dtype, 1.0, seed=22)
    qf, kf, vf, dyf = (t.double() for t in (q, k, v, dy))
    dq_ref, dk_ref, dv_ref = O.causal_bwd_chunked(qf, kf, vf, dyf, 1.0, chunk=64)
    assert O.rel_l2(dq.double(), dq_ref) <= tol
    assert O.rel_l2(dk.double(), dk_ref) <= tol
    assert O.rel_l2(dv.double(), dv_ref) <= tol


def test_backward_with_growing_logits(cuda_dev):
    """Keys whose norm grows along the sequence: the running maxima rise by tens of units from chunk to
    chunk, so the carried suffix state is rescaled by tiny factors and early tokens' weights underflow
    relative to late maxima -- finite results that match the fp64 restatement."""
    fb = _fb()
    B, H, N, M, D = 1, 2, 640, 32, 32
    q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=torch.float32, seed=23)
    k = k * torch.linspace(0.5, 6.0, N).view(1, 1, N, 1)
    qd, kd, vd = (t.to(cuda_dev).requires_grad_(True) for t in (q, k, v))
    y = fb.flare_causal_mixer(qd, kd, vd, 1.0)
    y.backward(dy.to(cuda_dev))
    qf, kf, vf, dyf = (t.double() for t in (q, k, v, dy))
    dq_ref, dk_ref, dv_ref = O.causal_bwd_chunked(qf, kf, vf, dyf, 1.0, chunk=32)
    for got, ref in ((qd.grad, dq_ref), (kd.grad, dk_ref), (vd.grad, dv_ref)):
        assert torch.isfinite(got).all()
        assert O.rel_l2(got.cpu().double(), ref) <= 2e-4


def test_backward_refuses_what_it_cannot_hold(cuda_dev):
    fb = _fb()
    q, k, v, dy = O.make_inputs(1, 1, 64, 64, 128, dtype=torch.float32, seed=1)   # forward: fine; backward: D = 128
    qd, kd, vd = (t.to(cuda_dev).requires_grad_(True) for t in (q, k, v))
    y = fb.flare_causal_mixer(qd, kd, vd, 1.0)
    with pytest.raises(RuntimeError, match="causal_bwd"):
        y.backward(dy.to(cuda_dev))


# ---------------------------------------------------------------------------------------------------------
# the call-site variants of the reference's FLARE modules on the serving path
# ---------------------------------------------------------------------------------------------------------
def test_decode_with_shared_latents_and_normalised_q_k(cuda_dev):
    """`shared_latents` (one latent set expand()-ed over the heads: stride 0) and `qk_norm` (q, k normalised
    by the caller before the mixer; pdebench/models/flare.py:130-132) on prefill + decode: the broadcast view is
    accepted as it is, and what comes out equals the oracle on the materialised, normalised tensors."""
    import flare_b200 as fb
    import torch.nn.functional as F
    B, H, N, M, D = 2, 4, 150, 32, 32
    g = torch.Generator().manual_seed(31)
    q1 = torch.randn(1, M, D, generator=g)
    k = torch.randn(B, H, N, D, generator=g)
    v = torch.randn(B, H, N, D, generator=g)
    qn = F.normalize(q1, dim=-1).expand(H, M, D)            # stride 0 over the heads
    kn = F.normalize(k, dim=-1)
    assert qn.stride(0) == 0
    scale = 4.0                                             # unit vectors: a sharper softmax than scale 1
    qd, kd, vd = qn.to(cuda_dev), kn.to(cuda_dev), v.to(cuda_dev)
    qd = qd[:1].expand(H, M, D)                             # (.to() materialises; make the device view broadcast again)
    n0 = 128
    y0, st = fb.flare_causal_prefill(qd, kd[:, :, :n0], vd[:, :, :n0], scale)
    ys = [y0] + [fb.flare_causal_decode(qd, kd[:, :, t:t + 1], vd[:, :, t:t + 1], st, scale) for t in range(n0, N)]
    y = torch.cat(ys, dim=2)
    y_ref, _ = O.causal_recurrent(qn.contiguous().double(), kn.double(), v.double(), scale)
    assert O.rel_l2(y.double().cpu(), y_ref) <= 2e-5


def test_training_step_with_shared_latents(cuda_dev):
    """flare_causal_mixer with the latents expand()-ed over the heads: autograd folds the per-head gradients
    back onto the single latent set, equal to autograd through the dense definition."""
    import flare_b200 as fb
    B, H, N, M, D = 1, 3, 100, 16, 16
    g = torch.Generator().manual_seed(32)
    q1 = (torch.randn(1, M, D, generator=g) * 0.5)
    k = torch.randn(B, H, N, D, generator=g) * 0.5
    v = torch.randn(B, H, N, D, generator=g)
    dy = torch.randn(B, H, N, D, generator=g)
    qd = q1.to(cuda_dev).requires_grad_(True)
    kd, vd = k.to(cuda_dev).requires_grad_(True), v.to(cuda_dev).requires_grad_(True)
    fb.flare_causal_mixer(qd.expand(H, M, D), kd, vd, 1.0).backward(dy.to(cuda_dev))
    qr = q1.double().requires_grad_(True)
    kr, vr = k.double().requires_grad_(True), v.double().requires_grad_(True)
    O.causal_dense(qr.expand(H, M, D), kr, vr, 1.0).backward(dy.double())
    assert O.rel_l2(qd.grad.double().cpu(), qr.grad) <= 1e-4
    assert O.rel_l2(kd.grad.double().cpu(), kr.grad) <= 1e-4
    assert O.rel_l2(vd.grad.double().cpu(), vr.grad) <= 1e-4


def test_decode_step_replays_from_a_cuda_graph(cuda_dev):
    """The serving loop: one decode step recorded in a CUDA graph over static k_t, v_t, y_t buffers and the
    state record, replayed once per token (the state lives in one fp32 tensor updated in place, so the
    recorded launch needs nothing new per step).  Equals the prefill over the same tokens."""
    import flare_b200 as fb
    B, H, N, M, D = 2, 4, 96, 64, 32
    q, k, v = _inputs(B, H, N, M, D, torch.bfloat16, seed=41)
    qd, kd, vd = q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev)
    n0 = 32
    _, st = fb.flare_causal_prefill(qd, kd[:, :, :n0], vd[:, :, :n0], 1.0)
    k_t = torch.empty(B, H, 1, D, dtype=torch.bfloat16, device=cuda_dev)
    v_t = torch.empty_like(k_t)
    k_t.copy_(kd[:, :, n0:n0 + 1]); v_t.copy_(vd[:, :, n0:n0 + 1])
    side = torch.cuda.Stream(device=cuda_dev)
    side.wait_stream(torch.cuda.current_stream(cuda_dev))
    st_warm = st.clone()
    with torch.cuda.stream(side):
        fb.flare_causal_decode(qd, k_t, v_t, st_warm, 1.0)          # warm-up outside the recording
    torch.cuda.current_stream(cuda_dev).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_t = fb.flare_causal_decode(qd, k_t, v_t, st, 1.0)
    ys = []
    for t in range(n0, N):
        k_t.copy_(kd[:, :, t:t + 1]); v_t.copy_(vd[:, :, t:t + 1])
        graph.replay()
        ys.append(y_t.clone())
    torch.cuda.synchronize()
    y_all, st_all = fb.flare_causal_prefill(qd, kd, vd, 1.0)
    assert O.rel_l2(torch.cat(ys, dim=2).float().cpu(), y_all[:, :, n0:].float().cpu()) <= 2e-2
    z = lambda s: (s[..., :D] / s[..., D + 1:D + 2]).cpu()
    assert O.rel_l2(z(st), z(st_all)) <= 2e-2          # (the prefill state comes from the bf16 tensor-core gather)
    assert fb.device_status() == 0
