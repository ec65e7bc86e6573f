"""flare_b200: the FLARE gather-scatter token mixer for NVIDIA B200 (sm_100a).

The directory is named after the project it accelerates (``flare.py_b200``); the
importable name is ``flare_b200`` (see ``flare_b200.py`` at the repository root,
which registers this directory under that name).
"""
from .causal import causal_state_init, flare_causal_decode, flare_causal_mixer, flare_causal_prefill
from .mixer import (device_status, pass_counts, flare_gather, flare_multihead_mixer, flare_scatter, mixer_backward,
                    mixer_forward, set_kernel_path)
from .triple import causal_linear, triple_attention
from .modules import FLARE, FLAREBlock, FLAREModel, ResidualMLP
from .cp_train import ContextParallel, ShardedPointCloud, cp_train_step, enable_context_parallel

__all__ = [
    "flare_multihead_mixer", "flare_gather", "flare_scatter", "mixer_forward", "mixer_backward",
    "set_kernel_path", "device_status", "pass_counts", "flare_causal_prefill", "flare_causal_decode", "flare_causal_mixer", "causal_state_init", "triple_attention",
    "causal_linear", "FLARE", "FLAREBlock", "FLAREModel", "ResidualMLP",
    "ContextParallel", "ShardedPointCloud", "cp_train_step", "enable_context_parallel",
]
