"""Parameter values and inputs that depend only on a parameter's NAME and shape, so that the reference model
(when the golden vectors are recorded) and the drop-in model (when they are checked) hold the same numbers
without a multi-megabyte state_dict in the repository."""
import zlib

import torch


def _gen(name: str) -> torch.Generator:
    return torch.Generator().manual_seed(zlib.crc32(name.encode()))


@torch.no_grad()
def fill_parameters(model: torch.nn.Module) -> None:
    """Weights ~ N(0, 0.02) (the reference's init, pdebench/models/flare.py:321-333), small biases, latent
    queries ~ N(0, 0.1), norm weights near one: every value a function of the parameter's name."""
    for name, p in model.named_parameters():
        g = _gen(name)
        r = torch.randn(p.shape, generator=g)
        if name.endswith("latent_q"):
            p.copy_(0.1 * r)
        elif "norm" in name or name.startswith("out_proj.0"):
            p.copy_(1.0 + 0.1 * r if name.endswith("weight") else 0.05 * r)
        elif name.endswith("bias"):
            p.copy_(0.01 * r)
        else:
            p.copy_(0.02 * r)


def pde_inputs(B: int, N: int, seed: int = 0):
    """x[B,N,3]: two coordinates U[0,1) and one field N(0,1); target[B,N,1] ~ N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.cat([torch.rand(B, N, 2, generator=g), torch.randn(B, N, 1, generator=g)], -1)
    target = torch.randn(B, N, 1, generator=g)
    return x, target


def projections(name: str, t: torch.Tensor, n: int = 4) -> torch.Tensor:
    """n scalar products of t with unit-norm vectors derived from `name`: a few-number fingerprint of a
    tensor whose relative error follows the tensor's own."""
    g = _gen("proj::" + name)
    flat = t.detach().double().reshape(-1)
    r = torch.randn(n, flat.numel(), generator=g, dtype=torch.float64)
    r = r / r.norm(dim=1, keepdim=True)
    return r @ flat
