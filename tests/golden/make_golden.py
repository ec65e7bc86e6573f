"""Generate the golden vectors under tests/golden/ from the reference project.

Run once in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/FLARE.py

It imports the reference's own ``pdebench/models/flare.py`` and
``lra/models/backends.py`` by file path (the packages themselves need
dependencies that are not installed), runs them on seeded CPU inputs in fp32
and records, at the boundary of the two ``F.scaled_dot_product_attention``
calls the reference makes, what went in and what came out, together with the
gradients autograd produced.  The ``.npz`` files it writes are committed; the
tests never need the reference checkout.
"""
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from seeded_init import fill_parameters, pde_inputs, projections  # noqa: E402


def _load(path: Path, name: str, package: str | None = None):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    if package:
        mod.__package__ = package
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


class SdpaTap:
    """Records the arguments and results of every SDPA call made inside a block."""

    def __init__(self):
        self.calls = []
        self._orig = F.scaled_dot_product_attention

    def __enter__(self):
        tap = self

        def wrapped(q, k, v, *a, **kw):
            out = tap._orig(q, k, v, *a, **kw)
            if out.requires_grad:
                out.retain_grad()
            for t in (q, k, v):
                if t.requires_grad and not t.is_leaf:
                    t.retain_grad()
            tap.calls.append((q, k, v, kw, out))
            return out

        F.scaled_dot_product_attention = wrapped
        return self

    def __exit__(self, *exc):
        F.scaled_dot_product_attention = self._orig


def np32(t):
    return t.detach().to(torch.float32).contiguous().numpy()


def pde_mixer_case(ref, name, B, N, C, H, M, scale, seed):
    """FLARE.forward of pdebench/models/flare.py:122-156 on a seeded input."""
    torch.manual_seed(seed)
    att = ref.FLARE(channel_dim=C, num_heads=H, num_latents=M, attn_scale=scale)
    x = torch.randn(B, N, C)
    with SdpaTap() as tap:
        out, _ = att(x)
    g = torch.Generator().manual_seed(seed + 1)
    dout = torch.randn(out.shape, generator=g)
    out.backward(dout)
    (q1, k1, v1, _, z), (k2, q2, z2, _, y) = tap.calls
    assert z2 is z and k2 is k1
    D = C // H
    # explicit path of the same module (flare.py:141-150 applies no scale)
    with torch.no_grad():
        _, scores = att(x, return_scores=True)
    np.savez_compressed(
        HERE / f"{name}.npz",
        q=np32(q1[0]), k=np32(k1), v=np32(v1), z=np32(z), y=np32(y),
        dy=np32(y.grad), dk=np32(k1.grad), dv=np32(v1.grad), dz=np32(z.grad),
        dq=np32(att.latent_q.grad.view(H, M, D)),
        scores=np32(scores), scale=np.float32(scale),
    )
    print(name, "k", tuple(k1.shape), "strides", k1.stride())


def lra_mixer_case(lra, name, B, N, C, H, M, scale, seed):
    """lra FLARE.forward (lra/models/backends.py:588-622) with a key-padding mask."""
    torch.manual_seed(seed)
    att = lra.FLARE(channel_dim=C, num_heads=H, num_latents=M, attn_scale=scale,
                    kv_proj_hidden_dim=C).eval()
    x = torch.randn(B, N, C)
    lens = torch.tensor([N, N - 5, N // 2, 1][:B])
    mask = torch.arange(N)[None, :] < lens[:, None]
    with SdpaTap() as tap:
        out = att(x, attention_mask=mask)
    g = torch.Generator().manual_seed(seed + 1)
    dout = torch.randn(out.shape, generator=g)
    out.backward(dout)
    (q1, k1, v1, _, z), (_, _, _, _, y) = tap.calls
    D = C // H
    np.savez_compressed(
        HERE / f"{name}.npz",
        q=np32(q1[0]), k=np32(k1), v=np32(v1), z=np32(z), y=np32(y),
        mask=mask.numpy(), dy=np32(y.grad), dk=np32(k1.grad), dv=np32(v1.grad),
        dq=np32(att.latent_q.grad.view(H, M, D)), scale=np.float32(scale),
    )
    print(name, "masked rows of y finite:", bool(torch.isfinite(y).all()))


def pde_model_case(ref, name, seed):
    """FLAREModel contract case (tests/pdebench/test_pdebench_model_contracts.py:21-132 sizes)."""
    torch.manual_seed(seed)
    model = ref.FLAREModel(in_dim=4, out_dim=3, channel_dim=32, num_blocks=2,
                           num_heads=4, num_latents=16).eval()
    x = torch.randn(2, 32, 4)
    with torch.no_grad():
        y = model(x)
    sd = {k: np32(v) for k, v in model.state_dict().items()}
    np.savez_compressed(HERE / f"{name}.npz", x=np32(x), y=np32(y),
                        **{"sd::" + k: v for k, v in sd.items()})
    print(name, "params", sum(v.size for v in sd.values()))


def pde_surrogate_case(ref, name):
    """The PDE-surrogate configuration (B=4, N=7225 = the 85 x 85 Darcy grid, C=128, 8 heads, 64 latents,
    8 blocks; pdebench/models/flare.py:251-349) trained one step with an MSE loss, fp32 on the CPU.
    Recorded: the loss, fingerprints of the output and of every parameter gradient (norm + 4 projections)
    and the full gradient of every block's latent queries.  Weights and inputs are functions of names
    and seeds (seeded_init.py), so the check rebuilds them instead of loading them."""
    model = ref.FLAREModel(in_dim=3, out_dim=1, channel_dim=128, num_blocks=8, num_heads=8, num_latents=64)
    fill_parameters(model)
    x, target = pde_inputs(4, 7225, seed=0)
    y = model(x)
    loss = F.mse_loss(y, target)
    loss.backward()
    out = {"loss": np.float64(loss.item()), "y_norm": np.float64(y.detach().double().norm().item()),
           "y_proj": projections("y", y).numpy()}
    for pname, prm in model.named_parameters():
        out["gnorm::" + pname] = np.float64(prm.grad.double().norm().item())
        out["gproj::" + pname] = projections(pname, prm.grad).numpy()
        if pname.endswith("latent_q"):
            out["grad::" + pname] = np32(prm.grad)
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, "loss", loss.item(), "params", sum(p.numel() for p in model.parameters()))


def lra_block_case(lra, name, seed):
    """lra FLAREBlock (lra/models/backends.py:624-672) with a key-padding mask, eval mode."""
    torch.manual_seed(seed)
    blk = lra.FLAREBlock(channel_dim=64, num_heads=4, num_latents=16, kv_proj_hidden_dim=64,
                         ffn_hidden_dim=64).eval()
    x = torch.randn(3, 24, 64)
    mask = torch.arange(24)[None, :] < torch.tensor([24, 17, 9])[:, None]
    with torch.no_grad():
        y = blk(x, attention_mask=mask)
    sd = {k: np32(v) for k, v in blk.state_dict().items()}
    np.savez_compressed(HERE / f"{name}.npz", x=np32(x), y=np32(y), mask=mask.numpy(),
                        **{"sd::" + k: v for k, v in sd.items()})
    print(name, "params", sum(v.size for v in sd.values()))


def triton_ref_cases(root: Path):
    """Einsum references of the two Triton operators (triple.py:846-860, causal_linear.py:317-336).

    Those files import triton at module level and define the references next to
    the kernels; only the pure-torch reference functions are executed here.
    """
    tri = _load(root / "lra/models/triton/triple.py", "_ref_triple")
    g = torch.Generator().manual_seed(7)
    B, H, N, D = 1, 2, 96, 16
    q1, q2, k1, k2, v = (torch.randn(B, H, N, D, generator=g) for _ in range(5))
    state, o = tri.triple_attn_einsum(q1, q2, k1, k2, v)
    # the file's own backward reference (triple.py:887-931) for a seeded upstream gradient of O
    do = torch.randn(B, H, N, D, generator=g)
    ctx = types.SimpleNamespace(saved_tensors=(q1, q2, k1, k2, v, o, state))
    dq1, dq2, dk1, dk2, dv = tri.triple_attn_bwd_einsum(ctx, None, do)
    np.savez_compressed(HERE / "triple_ref.npz", q1=np32(q1), q2=np32(q2), k1=np32(k1),
                        k2=np32(k2), v=np32(v), state=np32(state), o=np32(o), do=np32(do),
                        dq1=np32(dq1), dq2=np32(dq2), dk1=np32(dk1), dk2=np32(dk2), dv=np32(dv))
    cl = _load(root / "lra/models/triton/causal_linear.py", "_ref_causal_linear")
    B, H, N, Dk, Dv = 1, 2, 128, 32, 16
    q, k = (torch.randn(B, H, N, Dk, generator=g) for _ in range(2))
    v = torch.randn(B, H, N, Dv, generator=g)
    y = cl.linear_causal_reference(q, k, v)
    np.savez_compressed(HERE / "causal_linear_ref.npz", q=np32(q), k=np32(k), v=np32(v), y=np32(y))
    print("triton-file references written")


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of a FLARE.py checkout>")
    root = Path(sys.argv[1])
    ref = _load(root / "pdebench/models/flare.py", "_ref_pde_flare")
    pkg = types.ModuleType("_ref_lra_models")
    pkg.__path__ = [str(root / "lra/models")]
    sys.modules["_ref_lra_models"] = pkg
    _load(root / "lra/models/kernels.py", "_ref_lra_models.kernels", "_ref_lra_models")
    lra = _load(root / "lra/models/backends.py", "_ref_lra_models.backends", "_ref_lra_models")

    pde_mixer_case(ref, "pde_mixer_s1", B=2, N=48, C=32, H=4, M=16, scale=1.0, seed=0)
    pde_mixer_case(ref, "pde_mixer_sqrt", B=1, N=80, C=64, H=4, M=24, scale=16 ** -0.5, seed=1)
    lra_mixer_case(lra, "lra_mixer_mask", B=3, N=40, C=32, H=4, M=16, scale=1.0, seed=2)
    pde_model_case(ref, "pde_model_contract", seed=0)
    pde_surrogate_case(ref, "pde_surrogate_step")
    lra_block_case(lra, "lra_block_contract", seed=3)
    try:
        triton_ref_cases(root)
    except Exception as e:  # triton import without a GPU may fail on some images
        print("triton-file references skipped:", repr(e))


if __name__ == "__main__":
    main()
