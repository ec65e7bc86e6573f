"""Drop-in FLARE modules whose token mixing runs on the flare_b200 kernels.

Constructor keywords, parameter names/shapes (hence ``state_dict`` keys) and
forward contracts follow the reference so that checkpoints load unchanged:

* pdebench surface: ``ResidualMLP`` (pdebench/models/flare.py:24-59), ``FLARE``
  (:64-156), ``FLAREBlock`` (:161-215), ``FLAREModel`` (:251-349).
* lra surface: ``LraFLARE`` / ``LraFLAREBlock`` (lra/models/backends.py:541-672),
  which add a key-padding mask, RoPE on k and output dropout.

Only the two SDPA calls are replaced; the pointwise layers stay in torch.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .mixer import flare_multihead_mixer

__all__ = ["ResidualMLP", "FLARE", "FLAREBlock", "FLAREModel", "LraFLARE", "LraFLAREBlock"]


def _activation(name):
    table = {"gelu": lambda: nn.GELU(approximate="tanh"), "silu": nn.SiLU}
    return table[name or "gelu"]()


def _norm(dim, rms):
    return nn.RMSNorm(dim) if rms else nn.LayerNorm(dim)


def _split_heads(t: torch.Tensor, heads: int) -> torch.Tensor:
    """[B,N,C] -> strided [B,H,N,D] view (no copy); the kernels take it as it is."""
    B, N, Cdim = t.shape
    return t.view(B, N, heads, Cdim // heads).permute(0, 2, 1, 3)


def _merge_heads(t: torch.Tensor) -> torch.Tensor:
    """[B,H,N,D] -> [B,N,C]; free when the mixer wrote into a [B,N,H,D]-backed buffer."""
    B, H, N, D = t.shape
    return t.permute(0, 2, 1, 3).reshape(B, N, H * D)


class ResidualMLP(nn.Module):
    """fc1 -> num_layers residual hidden layers -> fc2; ``num_layers == -1`` is a single Linear."""

    def __init__(self, in_dim: int, hidden_dim: int, out_dim: int, num_layers: int = 2, act: str = None,
                 input_residual: bool = False, output_residual: bool = False):
        super().__init__()
        if num_layers < -1:
            raise AssertionError(f"num_layers must be at least -1. Got {num_layers}.")
        self.num_layers = num_layers
        if num_layers == -1:
            self.fc = nn.Linear(in_dim, out_dim)
            self.residual = bool(input_residual and output_residual and in_dim == out_dim)
            return
        self.act = _activation(act)
        self.fc1 = nn.Linear(in_dim, hidden_dim)
        self.fcs = nn.ModuleList(nn.Linear(hidden_dim, hidden_dim) for _ in range(num_layers))
        self.fc2 = nn.Linear(hidden_dim, out_dim)
        self.input_residual = bool(input_residual and in_dim == hidden_dim)
        self.output_residual = bool(output_residual and hidden_dim == out_dim)

    def forward(self, x):
        if self.num_layers == -1:
            out = self.fc(x)
            return x + out if self.residual else out
        h = self.act(self.fc1(x))
        if self.input_residual:
            h = h + x
        for layer in self.fcs:
            h = h + self.act(layer(h))
        out = self.fc2(h)
        return h + out if self.output_residual else out


class _FlareCore(nn.Module):
    """State shared by the two surfaces: latent queries, head bookkeeping, the mixer call."""

    def _setup(self, channel_dim, num_heads, num_latents, attn_scale):
        heads = channel_dim // 8 if num_heads is None else num_heads
        if channel_dim % heads:
            raise AssertionError(
                f"channel_dim must be divisible by num_heads. Got {channel_dim} and {heads}.")
        if not attn_scale > 0.0:
            raise AssertionError(f"attn_scale must be greater than 0. Got {attn_scale}.")
        self.channel_dim, self.num_heads, self.num_latents = channel_dim, heads, num_latents
        self.head_dim = channel_dim // heads
        self.attn_scale = attn_scale
        # [C, M], reinterpreted (not transposed) as [H, M, D] at use: keeps checkpoints compatible
        self.latent_q = nn.Parameter(torch.empty(channel_dim, num_latents))
        nn.init.normal_(self.latent_q, mean=0.0, std=0.1)
        self.cp = None      # a cp_train.ContextParallel when the token axis is sharded over ranks

    def _mix(self, q, k, v, key_mask=None, dropout_p=0.0):
        if self.cp is not None:
            if key_mask is not None or dropout_p:
                raise NotImplementedError("the context-parallel mixer takes neither a mask nor dropout")
            from .parallel import flare_mixer_context_parallel
            # the latent gradient joins the other replicated weights in the group-wide gradient sum
            return flare_mixer_context_parallel(q, k, v, self.attn_scale, exchange=self.cp.exchange, reduce_dq=False)
        return flare_multihead_mixer(q, k, v, scale=self.attn_scale, key_mask=key_mask, dropout_p=dropout_p)

    def _latents(self):
        return self.latent_q.view(self.num_heads, self.num_latents, self.head_dim)


class FLARE(_FlareCore):
    def __init__(self, channel_dim: int, num_heads: int = 8, num_latents: int = 32, attn_scale: float = 1.0,
                 act: str = None, num_layers_k_proj: int = 3, num_layers_v_proj: int = 3,
                 k_proj_mlp_ratio: float = 1.0, v_proj_mlp_ratio: float = 1.0, qk_norm: bool = False,
                 rmsnorm: bool = False):
        super().__init__()
        self._setup(channel_dim, num_heads, num_latents, attn_scale)
        self.qk_norm = qk_norm
        if qk_norm:
            self.q_norm = _norm(self.head_dim, rmsnorm)
            self.k_norm = _norm(self.head_dim, rmsnorm)
        mk = lambda ratio, depth: ResidualMLP(channel_dim, int(channel_dim * ratio), channel_dim, depth, act, True, True)
        self.k_proj = mk(k_proj_mlp_ratio, num_layers_k_proj)
        self.v_proj = mk(v_proj_mlp_ratio, num_layers_v_proj)
        self.out_proj = nn.Linear(channel_dim, channel_dim)

    def forward(self, x, return_scores: bool = False):
        q = self._latents()
        k = _split_heads(self.k_proj(x), self.num_heads)
        v = _split_heads(self.v_proj(x), self.num_heads)
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        if return_scores:
            # materialising path kept for score inspection on small inputs; like the reference's
            # branch (pdebench/models/flare.py:141-150) it does not apply attn_scale
            scores = q @ k.transpose(-2, -1)
            z = F.softmax(scores, dim=-1) @ v
            y = F.softmax(scores.transpose(-2, -1), dim=-1) @ z
        else:
            scores = None
            y = self._mix(q, k, v)
        return self.out_proj(_merge_heads(y)), scores


class FLAREBlock(nn.Module):
    def __init__(self, channel_dim: int, num_heads: int = None, num_latents: int = None, attn_scale: float = 1.0,
                 act: str = None, rmsnorm: bool = False, num_layers_k_proj: int = 3, num_layers_v_proj: int = 3,
                 k_proj_mlp_ratio: float = 1.0, v_proj_mlp_ratio: float = 1.0, num_layers_ffn: int = 3,
                 ffn_mlp_ratio: float = 1.0, qk_norm: bool = False):
        super().__init__()
        self.norm1 = _norm(channel_dim, rmsnorm)
        self.norm2 = _norm(channel_dim, rmsnorm)
        self.att = FLARE(channel_dim=channel_dim, num_heads=num_heads, num_latents=num_latents,
                         attn_scale=attn_scale, act=act, num_layers_k_proj=num_layers_k_proj,
                         num_layers_v_proj=num_layers_v_proj, k_proj_mlp_ratio=k_proj_mlp_ratio,
                         v_proj_mlp_ratio=v_proj_mlp_ratio, qk_norm=qk_norm, rmsnorm=rmsnorm)
        self.mlp = ResidualMLP(channel_dim, int(channel_dim * ffn_mlp_ratio), channel_dim, num_layers_ffn, act,
                               True, True)

    def forward(self, x, return_scores: bool = False):
        mixed, scores = self.att(self.norm1(x), return_scores=return_scores)
        x = x + mixed
        return x + self.mlp(self.norm2(x)), scores


class FLAREModel(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, channel_dim: int = 64, num_blocks: int = 8, num_heads: int = None,
                 act: str = None, rmsnorm: bool = False, out_proj_norm: bool = True,
                 num_layers_in_out_proj: int = 2, attn_scale: float = 1.0, num_latents: int = None,
                 num_layers_k_proj: int = 3, num_layers_v_proj: int = 3, k_proj_mlp_ratio: float = 1.0,
                 v_proj_mlp_ratio: float = 1.0, num_layers_ffn: int = 3, ffn_mlp_ratio: float = 1.0,
                 qk_norm: bool = False):
        super().__init__()
        self.in_proj = ResidualMLP(in_dim, channel_dim, channel_dim, num_layers_in_out_proj, act, False, True)
        self.out_proj = nn.Sequential(
            _norm(channel_dim, rmsnorm) if out_proj_norm else nn.Identity(),
            ResidualMLP(channel_dim, channel_dim, out_dim, num_layers_in_out_proj, act, True, False),
        )
        self.blocks = nn.ModuleList(
            FLAREBlock(channel_dim=channel_dim, num_heads=num_heads, num_latents=num_latents, attn_scale=attn_scale,
                       act=act, rmsnorm=rmsnorm, num_layers_k_proj=num_layers_k_proj,
                       num_layers_v_proj=num_layers_v_proj, k_proj_mlp_ratio=k_proj_mlp_ratio,
                       v_proj_mlp_ratio=v_proj_mlp_ratio, num_layers_ffn=num_layers_ffn,
                       ffn_mlp_ratio=ffn_mlp_ratio, qk_norm=qk_norm)
            for _ in range(num_blocks))
        self.checkpoint_blocks = False      # recompute each block in the backward pass (cp_train.enable_context_parallel)
        self.initialize_weights()

    def initialize_weights(self):
        # Linear ~ N(0, 0.02) with zero bias, norms at identity; latent_q keeps its N(0, 0.1)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, (nn.LayerNorm, nn.RMSNorm)):
                if getattr(m, "weight", None) is not None:
                    nn.init.ones_(m.weight)
                if getattr(m, "bias", None) is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, x, return_scores: bool = False):
        collected = []
        h = self.in_proj(x)
        for blk in self.blocks:
            if self.checkpoint_blocks and self.training and not return_scores and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                h, s = checkpoint(blk, h, use_reentrant=False)
            else:
                h, s = blk(h, return_scores=return_scores)
            collected.append(s)
        out = self.out_proj(h)
        return (out, collected) if return_scores else out


class LraFLARE(_FlareCore):
    """lra/models/backends.py:541-622: shared kv-projection depth, key-padding mask, RoPE on k, dropout."""

    def __init__(self, channel_dim: int, num_heads: int = 8, num_latents: int = 32, act: str = None,
                 attn_scale: float = 1.0, num_layers_kv_proj: int = 3, kv_proj_hidden_dim: int = 1.0,
                 attn_drop: float = 0.0, proj_drop: float = 0.0, rope=None):
        super().__init__()
        self._setup(channel_dim, num_heads, num_latents, attn_scale)
        self.rope = rope
        self.attn_drop_p, self.proj_drop_p = attn_drop, proj_drop
        self.k_proj, self.v_proj = (
            ResidualMLP(channel_dim, kv_proj_hidden_dim, channel_dim, num_layers_kv_proj, act, True, True)
            for _ in range(2))
        self.out_proj = nn.Linear(channel_dim, channel_dim)

    def forward(self, x, attention_mask=None):
        k = _split_heads(self.k_proj(x), self.num_heads)
        v = _split_heads(self.v_proj(x), self.num_heads)
        if self.rope is not None:
            k = self.rope(k)
        drop = self.attn_drop_p if self.training else 0.0
        y = self._mix(self._latents(), k, v, key_mask=attention_mask, dropout_p=drop)
        y = self.out_proj(_merge_heads(y))
        return F.dropout(y, p=self.proj_drop_p if self.training else 0.0)


class LraFLAREBlock(nn.Module):
    def __init__(self, channel_dim: int, num_heads: int = None, num_latents: int = None, act: str = None,
                 rmsnorm: bool = False, attn_scale: float = 1.0, num_layers_kv_proj: int = 3,
                 num_layers_ffn: int = 3, kv_proj_hidden_dim: int = 1.0, ffn_hidden_dim: int = 1.0,
                 attn_drop: float = 0.0, proj_drop: float = 0.0, rope=None):
        super().__init__()
        self.norm1 = _norm(channel_dim, rmsnorm)
        self.norm2 = _norm(channel_dim, rmsnorm)
        self.att = LraFLARE(channel_dim=channel_dim, num_heads=num_heads, num_latents=num_latents, act=act,
                            attn_scale=attn_scale, num_layers_kv_proj=num_layers_kv_proj,
                            kv_proj_hidden_dim=kv_proj_hidden_dim, attn_drop=attn_drop, proj_drop=proj_drop,
                            rope=rope)
        self.mlp = ResidualMLP(channel_dim, ffn_hidden_dim, channel_dim, num_layers_ffn, act, True, True)

    def forward(self, x, attention_mask=None):
        x = x + self.att(self.norm1(x), attention_mask=attention_mask)
        return x + self.mlp(self.norm2(x))
