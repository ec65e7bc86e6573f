"""CPU-side checks of the C ABI: the library loads, exports what the header declares, rejects bad requests."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def cabi():
    import __graft_entry__
    __graft_entry__.build()
    import flare_b200  # noqa: F401  (loads the shared library)
    from flare_b200 import _cabi
    return _cabi


def header_symbols():
    text = (ROOT / "include" / "flare_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flare_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(cabi):
    syms = header_symbols()
    assert len(syms) >= 15
    for s in syms:
        assert hasattr(cabi.lib, s), f"{s} declared in include/flare_b200.h but not exported"
        assert s in cabi.SIGNATURES, f"{s} has no ctypes signature"


def test_version_and_struct_layout(cabi):
    assert cabi.lib.flare_version() >= 100
    # 8 x 4-byte fields, 7 x 3 x int64, then the dropout probability (float, padded) and seed (uint64)
    assert C.sizeof(cabi.FlareProblem) == 32 + 7 * 24 + 16


def test_struct_sizes_match_the_header_as_a_c_compiler_sees_it(cabi, tmp_path):
    """The ctypes mirrors against sizeof/offsetof of the C declarations (gcc on the public header)."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    src = tmp_path / "sizes.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "flare_b200.h"\n'
        'int main(void) { printf("%zu %zu %zu %zu %zu\\n", sizeof(FlareProblem), offsetof(FlareProblem, dropout_p),\n'
        '  offsetof(FlareProblem, dropout_seed), sizeof(FlarePeers), offsetof(FlarePeers, epoch)); return 0; }\n')
    exe = tmp_path / "sizes"
    subprocess.check_call(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)])
    got = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    want = [C.sizeof(cabi.FlareProblem), cabi.FlareProblem.dropout_p.offset, cabi.FlareProblem.dropout_seed.offset,
            C.sizeof(cabi.FlarePeers), cabi.FlarePeers.epoch.offset]
    assert got == want


def _problem(cabi, **kw):
    p = cabi.FlareProblem()
    p.B, p.H, p.N, p.M, p.D = 1, 8, 4096, 64, 16
    p.dtype, p.scale, p.n_splits = cabi.F32, 1.0, 0
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_split_choice_and_workspace_are_host_only(cabi):
    p = _problem(cabi)
    s = cabi.lib.flare_pick_splits(C.byref(p))
    assert 1 <= s <= 4096 // 128
    assert cabi.lib.flare_fwd_workspace_bytes(C.byref(p)) >= s * 8 * 64 * 18 * 4
    assert cabi.lib.flare_bwd_workspace_bytes(C.byref(p)) >= s * 8 * 64 * 16 * 4 + 8 * 4096 * 4
    p = _problem(cabi, N=100)
    assert cabi.lib.flare_pick_splits(C.byref(p)) == 1


@pytest.mark.parametrize("kw,code", [
    (dict(D=24), -5), (dict(dtype=7), -1), (dict(scale=0.0), -1), (dict(M=0), -1),
])
def test_rejects_bad_problem_before_any_launch(cabi, kw, code):
    p = _problem(cabi, n_splits=1, **kw)
    rc = cabi.lib.flare_gather_partial(C.byref(p), 16, 16, 16, None, 16, None)
    assert rc == code
    assert cabi.lib.flare_last_error()


def test_rejects_misaligned_and_null(cabi):
    p = _problem(cabi, n_splits=1)
    p.q_stride[:] = (0, 64 * 16, 16)
    p.k_stride[:] = (8 * 4096 * 16, 4096 * 16, 16)
    p.v_stride[:] = (8 * 4096 * 16, 4096 * 16, 16)
    assert cabi.lib.flare_gather_partial(C.byref(p), 16, 24, 16, None, 16, None) == -2   # k pointer % 16
    assert cabi.lib.flare_gather_partial(C.byref(p), 16, None, 16, None, 16, None) == -1
    p.k_stride[:] = (8 * 4096 * 16, 4096 * 16, 18)
    assert cabi.lib.flare_gather_partial(C.byref(p), 16, 16, 16, None, 16, None) == -2   # row pitch
    with pytest.raises(cabi.FlareError):
        cabi.check(-2, "x")


def test_causal_prefill_workspace_size_and_alignment_are_host_checks(cabi):
    """The causal prefill's workspace holds fp32 records, the redo flags and the 16-bit records with their (m, l)
    pairs; a workspace that is not 16-byte aligned is refused before any launch."""
    p = _problem(cabi, B=2, H=4, N=1000, M=64, D=32)
    chunks, rows = 8, 2 * 4 * 64
    need = chunks * rows * (32 + 2) * 4 + chunks * 2 * 4 * 4 + chunks * rows * (32 * 2 + 8)
    assert cabi.lib.flare_causal_workspace_bytes(C.byref(p)) >= need
    rc = cabi.lib.flare_causal_prefill(C.byref(p), 16, 16, 16, 16, None, None, 24, None)
    assert rc == -1
    assert b"aligned" in cabi.lib.flare_last_error()


def test_whole_pass_checks_workspace(cabi):
    p = _problem(cabi)
    rc = cabi.lib.flare_mixer_fwd(C.byref(p), 16, 16, 16, None, 16, 16, 16, 16, 256, 8, None)
    assert rc == -3
