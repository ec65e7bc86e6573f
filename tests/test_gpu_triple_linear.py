"""Triple attention and causal linear attention on the GPU against the oracle and the vectors recorded
from the reference's einsum forms (tests/golden/triple_ref.npz, causal_linear_ref.npz)."""
import pytest
import torch

from conftest import load_golden
from oracle import flare_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-3}


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def test_triple_golden(cuda_dev):
    import flare_b200 as fb
    g = load_golden("triple_ref")
    t = {k: torch.as_tensor(v).to(cuda_dev) for k, v in g.items()}
    state, o = fb.triple_attention(t["q1"], t["q2"], t["k1"], t["k2"], t["v"])
    assert O.rel_l2(state.cpu(), torch.as_tensor(g["state"])) <= 1e-5
    assert O.rel_l2(o.cpu(), torch.as_tensor(g["o"])) <= 1e-5


@pytest.mark.parametrize("B,H,N,Dq,Dv,dtype", [
    (1, 2, 300, 16, 16, torch.float32),
    (2, 2, 1000, 32, 32, torch.float32),      # the reference's tested head size
    (1, 1, 257, 32, 16, torch.float32),       # Dq != Dv, ragged N
    (1, 2, 5000, 32, 32, torch.bfloat16),     # several token ranges
    (1, 1, 200, 64, 64, torch.float32),       # state larger than one shared-memory slab
    (1, 2, 640, 32, 32, torch.float16),
])
def test_triple_fwd_bwd(cuda_dev, B, H, N, Dq, Dv, dtype):
    import flare_b200 as fb
    s = Dq ** -0.5
    q1, q2, k1, k2 = (_rand((B, H, N, Dq), dtype, i, s) for i in range(4))
    v = _rand((B, H, N, Dv), dtype, 4)
    do = _rand((B, H, N, Dv), dtype, 5)
    st_ref, o_ref = O.triple_attention(*(t.double() for t in (q1, q2, k1, k2, v)))
    grads_ref = O.triple_attention_bwd(*(t.double() for t in (q1, q2, k1, k2, v, do)))
    ins = [t.to(cuda_dev).requires_grad_(True) for t in (q1, q2, k1, k2, v)]
    state, o = fb.triple_attention(*ins)
    tol = TOL[dtype]
    assert O.rel_l2(state.double().cpu(), st_ref.double()) <= tol
    assert O.rel_l2(o.double().cpu(), o_ref.double()) <= tol
    o.backward(do.to(cuda_dev))
    for name, t, r in zip(("dq1", "dq2", "dk1", "dk2", "dv"), ins, grads_ref):
        assert O.rel_l2(t.grad.double().cpu(), r.double()) <= tol, name


def test_triple_state_gradient(cuda_dev):
    """A loss on STATE itself reaches k1, k2, v."""
    import flare_b200 as fb
    B, H, N, D = 1, 2, 128, 16
    q1, q2, k1, k2, v = (_rand((B, H, N, D), torch.float32, i, 0.5) for i in range(5))
    w = _rand((B, H, D, D, D), torch.float32, 9)
    ref_in = [t.double().requires_grad_(True) for t in (k1, k2, v)]
    st = torch.einsum("bhni,bhnj,bhnk->bhijk", ref_in[0], ref_in[2], ref_in[1]) / N
    (st * w.double()).sum().backward()
    ins = [t.to(cuda_dev).requires_grad_(True) for t in (q1, q2, k1, k2, v)]
    state, _ = fb.triple_attention(*ins)
    (state * w.to(cuda_dev)).sum().backward()
    for t, r in zip((ins[2], ins[3], ins[4]), ref_in):
        assert O.rel_l2(t.grad.double().cpu(), r.grad) <= 1e-5


@pytest.mark.parametrize("B,H,N,dtype", [
    (3, 5, 1000, torch.bfloat16),             # ragged N: a last tile of 104 tokens, 15 (b, h)
    (1, 2, 129, torch.float16),               # one full tile and one token
    (2, 80, 300, torch.float16),              # more (b, h) than SMs: one token range each
])
def test_triple_tensor_core_shapes(cuda_dev, B, H, N, dtype):
    """16-bit inputs with every feature dimension 32 run on the tensor-core kernels (the pair-axis operand
    built on the fly): ragged token counts, a loss on both outputs so that dSTATE carries an upstream term,
    inputs large enough that the rank-3 tensors leave fp16's comfortable range without the per-(b, h) scaling."""
    import flare_b200 as fb
    D = 32
    q1, q2, k1, k2 = (_rand((B, H, N, D), dtype, 10 + i, 0.5) for i in range(4))
    v = _rand((B, H, N, D), dtype, 14, 4.0)
    do = _rand((B, H, N, D), dtype, 15, 8.0)
    w = _rand((B, H, D, D, D), torch.float32, 16)
    ref_in = [t.double().requires_grad_(True) for t in (q1, q2, k1, k2, v)]
    st_ref = torch.einsum("bhni,bhnj,bhnk->bhijk", ref_in[2], ref_in[4], ref_in[3]) / N
    o_ref = torch.einsum("bhni,bhijk,bhnk->bhnj", ref_in[0], st_ref, ref_in[1])
    ((st_ref * w.double()).sum() + (o_ref * do.double()).sum()).backward()
    ins = [t.to(cuda_dev).requires_grad_(True) for t in (q1, q2, k1, k2, v)]
    state, o = fb.triple_attention(*ins)
    ((state * w.to(cuda_dev)).sum() + (o.float() * do.to(cuda_dev).float()).sum()).backward()
    tol = TOL[dtype]
    assert fb.device_status() == 0
    assert O.rel_l2(state.double().cpu(), st_ref.detach()) <= tol
    assert O.rel_l2(o.double().cpu(), o_ref.detach()) <= tol
    for name, t, r in zip(("dq1", "dq2", "dk1", "dk2", "dv"), ins, ref_in):
        assert torch.isfinite(t.grad).all(), name
        assert O.rel_l2(t.grad.double().cpu(), r.grad) <= tol, name


def test_causal_linear_golden(cuda_dev):
    import flare_b200 as fb
    g = load_golden("causal_linear_ref")
    y = fb.causal_linear(*(torch.as_tensor(g[k]).to(cuda_dev) for k in ("q", "k", "v")))
    assert O.rel_l2(y.cpu(), torch.as_tensor(g["y"])) <= 1e-5


@pytest.mark.parametrize("B,H,N,Dk,Dv,dtype", [
    (1, 2, 2048, 128, 32, torch.float32),     # the reference's default test shape
    (2, 3, 1000, 64, 64, torch.float32),      # N not a multiple of 64
    (1, 1, 70, 16, 8, torch.float32),
    (1, 4, 4096, 128, 32, torch.bfloat16),
    (1, 2, 512, 32, 32, torch.float16),
])
def test_causal_linear(cuda_dev, B, H, N, Dk, Dv, dtype):
    import flare_b200 as fb
    q = _rand((B, H, N, Dk), dtype, 0, Dk ** -0.5)
    k = _rand((B, H, N, Dk), dtype, 1)
    v = _rand((B, H, N, Dv), dtype, 2)
    y_ref = O.causal_linear(q.double(), k.double(), v.double())
    y = fb.causal_linear(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev))
    assert O.rel_l2(y.double().cpu(), y_ref.double()) <= TOL[dtype]


@pytest.mark.parametrize("B,H,N,Dv,dtype", [
    (2, 2, 1000, 64, torch.float16),          # ragged last chunk
    (1, 2, 130, 32, torch.bfloat16),
    (8, 8, 2048, 32, torch.bfloat16),         # the shape of the reference's main()
    (1, 1, 7, 32, torch.float16),
])
def test_causal_linear_tensor_core_shapes(cuda_dev, B, H, N, Dv, dtype):
    """16-bit inputs with Dk = 128 and Dv in {32, 64} run on the tensor cores; q, k, v as head-interleaved views."""
    import flare_b200 as fb
    Dk = 128
    qf = _rand((B, N, H * Dk), dtype, 0, Dk ** -0.5).to(cuda_dev)
    kf = _rand((B, N, H * Dk), dtype, 1).to(cuda_dev)
    vf = _rand((B, N, H * Dv), dtype, 2).to(cuda_dev)
    q, k = (t.view(B, N, H, Dk).permute(0, 2, 1, 3) for t in (qf, kf))
    v = vf.view(B, N, H, Dv).permute(0, 2, 1, 3)
    y = fb.causal_linear(q, k, v)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    y_ref = O.causal_linear(q.double().cpu(), k.double().cpu(), v.double().cpu())
    assert O.rel_l2(y.double().cpu(), y_ref.double()) <= TOL[dtype]


def test_causal_linear_strided_views(cuda_dev):
    """q, k, v as 'b n (h d) -> b h n d' views, as the lra blocks make them."""
    import flare_b200 as fb
    B, H, N, Dk, Dv = 2, 4, 300, 32, 16
    qf = _rand((B, N, H * Dk), torch.float32, 0, 0.2).to(cuda_dev)
    kf = _rand((B, N, H * Dk), torch.float32, 1).to(cuda_dev)
    vf = _rand((B, N, H * Dv), torch.float32, 2).to(cuda_dev)
    q, k = (t.view(B, N, H, Dk).permute(0, 2, 1, 3) for t in (qf, kf))
    v = vf.view(B, N, H, Dv).permute(0, 2, 1, 3)
    y = fb.causal_linear(q, k, v)
    y_ref = O.causal_linear(q.double().cpu(), k.double().cpu(), v.double().cpu())
    assert O.rel_l2(y.double().cpu(), y_ref.double()) <= 1e-5
