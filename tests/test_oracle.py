"""Pins the CPU oracle to vectors recorded from the reference project itself."""
import pytest
import torch

from conftest import load_golden
from oracle import flare_oracle as O

MIXER_CASES = ["pde_mixer_s1", "pde_mixer_sqrt"]
TOL = 2e-6   # fp32 round-off between SDPA's fused kernel and the explicit form


@pytest.mark.parametrize("name", MIXER_CASES)
def test_forward_matches_reference(name):
    g = load_golden(name)
    for fn in (O.mixer_sdpa, O.mixer_explicit):
        y = fn(g["q"], g["k"], g["v"], g["scale"])
        assert O.rel_l2(y, g["y"]) < TOL
    z, _ = O.gather(g["q"], g["k"], g["v"], g["scale"])
    assert O.rel_l2(z, g["z"]) < TOL


@pytest.mark.parametrize("name", MIXER_CASES)
def test_explicit_scores_branch(name):
    # pdebench/models/flare.py:142 returns the unscaled scores q k^T
    g = load_golden(name)
    s = g["q"][None] @ g["k"].transpose(-2, -1)
    assert O.rel_l2(s, g["scores"]) < TOL


@pytest.mark.parametrize("name", MIXER_CASES)
def test_backward_matches_reference_autograd(name):
    g = load_golden(name)
    dq, dk, dv = O.mixer_bwd_closed_form(g["q"], g["k"], g["v"], g["dy"], g["scale"])
    assert O.rel_l2(dq, g["dq"]) < 1e-5
    assert O.rel_l2(dk, g["dk"]) < 1e-5
    assert O.rel_l2(dv, g["dv"]) < 1e-5
    dq2, dk2, dv2 = O.mixer_bwd_autograd(g["q"], g["k"], g["v"], g["dy"], g["scale"])
    assert O.rel_l2(dq2, g["dq"]) < 1e-5
    assert O.rel_l2(dk2, g["dk"]) < 1e-5
    assert O.rel_l2(dv2, g["dv"]) < 1e-5


def test_closed_form_backward_fp64():
    q, k, v, dy = O.make_inputs(2, 3, 70, 12, 8, dtype=torch.float64, seed=3)
    a = O.mixer_bwd_closed_form(q, k, v, dy, 0.7)
    b = O.mixer_bwd_autograd(q, k, v, dy, 0.7, fn=O.mixer_explicit)
    for x, y in zip(a, b):
        assert O.rel_l2(x, y) < 1e-12


def test_masked_variant_matches_lra_reference():
    g = load_golden("lra_mixer_mask")
    mask = g["mask"].bool()
    y = O.mixer_lra(g["q"], g["k"], g["v"], g["scale"], mask)
    assert O.rel_l2(y, g["y"]) < TOL
    z, _ = O.gather(g["q"], g["k"], g["v"], g["scale"], mask)
    assert O.rel_l2(z, g["z"]) < TOL


@pytest.mark.parametrize("bounds", [
    [(0, 48)], [(0, 7), (7, 48)], [(0, 16), (16, 16), (16, 33), (33, 48)],
])
def test_split_partials_combine(bounds):
    g = load_golden("pde_mixer_s1")
    m, l, acc = O.gather_partials(g["q"], g["k"], g["v"], g["scale"], bounds)
    z, L = O.lse_combine(m, l, acc)
    z0, L0 = O.gather(g["q"], g["k"], g["v"], g["scale"])
    assert O.rel_l2(z, g["z"]) < TOL
    assert O.rel_l2(L, L0) < TOL


def test_causal_forms_agree():
    q, k, v, _ = O.make_inputs(2, 2, 37, 6, 8, dtype=torch.float64, seed=5)
    yd = O.causal_dense(q, k, v, 0.9)
    yr, st = O.causal_recurrent(q, k, v, 0.9)
    yc, st2 = O.causal_chunked(q, k, v, 0.9, chunk=8)
    assert O.rel_l2(yr, yd) < 1e-12
    assert O.rel_l2(yc, yd) < 1e-12
    # last-token state equals the encoder gather over the whole sequence
    z, L = O.gather(q, k, v, 0.9)
    assert O.rel_l2(st[2] / st[1][..., None], z) < 1e-12
    assert O.rel_l2(st2[0] + torch.log(st2[1]), L) < 1e-12


def test_triple_and_causal_linear_references():
    g = load_golden("triple_ref")
    state, o = O.triple_attention(g["q1"], g["q2"], g["k1"], g["k2"], g["v"])
    assert O.rel_l2(state, g["state"]) < 1e-5
    assert O.rel_l2(o, g["o"]) < 1e-5
    g = load_golden("causal_linear_ref")
    y = O.causal_linear(g["q"], g["k"], g["v"])
    assert O.rel_l2(y, g["y"]) < 1e-5


def test_streamed_form_equals_dense_closed_form():
    """The token-chunked oracle used for the million-token check is the dense one, chunk by chunk."""
    q, k, v, dy = O.make_inputs(2, 3, 333, 20, 8, dtype=torch.float64, seed=5)
    y, dq, dk, dv = O.mixer_fwd_bwd_streamed(q, k, v, dy, 0.8, chunk=100)
    assert O.rel_l2(y, O.mixer_sdpa(q, k, v, 0.8)) < 1e-12
    for a, b in zip((dq, dk, dv), O.mixer_bwd_closed_form(q, k, v, dy, 0.8)):
        assert O.rel_l2(a, b) < 1e-12


def test_triple_backward_matches_the_reference_einsum_backward():
    """lra/models/triton/triple.py:887-931 (triple_attn_bwd_einsum) on the recorded inputs and upstream gradient."""
    g = load_golden("triple_ref")
    got = O.triple_attention_bwd(g["q1"], g["q2"], g["k1"], g["k2"], g["v"], g["do"])
    for name, a in zip(("dq1", "dq2", "dk1", "dk2", "dv"), got):
        assert O.rel_l2(a, g[name]) < 1e-5, name


def test_dropout_masks_have_the_right_rate_and_are_independent():
    keep1, keep2 = O.dropout_keep_masks(2, 3, 16, 4096, 0.3, seed=12345)
    assert keep1.shape == (2, 3, 16, 4096)
    for kmask in (keep1, keep2):
        assert abs(kmask.float().mean().item() - 0.7) < 5e-3
        rows = kmask.float().mean(-1)
        assert (rows - 0.7).abs().max() < 0.04                      # every (b, h, m) row on its own
    agree = (keep1 == keep2).float().mean().item()
    assert abs(agree - (0.7 * 0.7 + 0.3 * 0.3)) < 5e-3              # the two softmaxes draw independent masks
    k1b, _ = O.dropout_keep_masks(2, 3, 16, 4096, 0.3, seed=12346)
    assert abs((keep1 == k1b).float().mean().item() - 0.58) < 5e-3  # another seed, another mask
