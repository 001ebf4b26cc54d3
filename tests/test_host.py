"""CPU tests of the host side: the C ABI exports what include/jvpfa.h declares, argument errors are
reported without touching a GPU, and the Python mirror raises the reference's exception types."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _declared_functions():
    text = (ROOT / "include" / "jvpfa.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jvpfa_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(built_library):
    from jvp_flash_attention_b200 import _lib
    names = _declared_functions()
    assert set(_lib.EXPORTED_SYMBOLS) <= set(names)
    for n in names:
        assert hasattr(built_library, n), f"{n} declared in jvpfa.h but not exported"


def test_version_and_error_strings(built_library):
    assert built_library.jvpfa_version() >= 100
    for code in range(0, 8):
        assert len(built_library.jvpfa_error_string(code)) > 0


def test_struct_layout_matches_header():
    """Sizes of the ctypes mirrors equal what a C compiler makes of the header."""
    import subprocess, tempfile
    from jvp_flash_attention_b200 import _lib
    src = '#include <stdio.h>\n#include "jvpfa.h"\nint main(){printf("%zu %zu %zu\\n", sizeof(jvpfa_mask), sizeof(jvpfa_fwd_args), sizeof(jvpfa_bwd_args));return 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "t.c").write_text(src)
        subprocess.run(["gcc", "-I", str(ROOT / "include"), "-o", f"{d}/t", f"{d}/t.c"], check=True)
        out = subprocess.run([f"{d}/t"], capture_output=True, text=True, check=True).stdout.split()
    assert [int(x) for x in out] == [C.sizeof(_lib.Mask), C.sizeof(_lib.FwdArgs), C.sizeof(_lib.BwdArgs)]


def test_bad_arguments_rejected_before_launch(built_library):
    from jvp_flash_attention_b200 import _lib
    L = built_library
    assert L.jvpfa_fwd(None, None) == _lib.ERR_BAD_ARG
    assert L.jvpfa_bwd(None, None) == _lib.ERR_BAD_ARG
    a = _lib.FwdArgs()
    a.B, a.H, a.N, a.D, a.dtype = 1, 1, 0, 64, _lib.BF16
    assert L.jvpfa_fwd(C.byref(a), None) == _lib.ERR_BAD_ARG           # N <= 0
    a.N = 128
    a.dtype = 9
    assert L.jvpfa_fwd(C.byref(a), None) == _lib.ERR_UNSUPPORTED       # unknown dtype
    a.dtype = _lib.BF16
    a.causal = 1
    a.mask.kind = _lib.MASK_BOOL
    a.mask.ptr = 16
    assert L.jvpfa_fwd(C.byref(a), None) == _lib.ERR_CAUSAL_MASK       # causal + mask
    a.causal = 0
    a.mask.kind = _lib.MASK_NONE
    assert L.jvpfa_fwd(C.byref(a), None) == _lib.ERR_WORKSPACE         # no workspace
    a.workspace, a.workspace_bytes = 256, 256
    assert L.jvpfa_fwd(C.byref(a), None) == _lib.ERR_BAD_ARG           # null tensors
    assert L.jvpfa_read_status(None, None, None) == _lib.ERR_BAD_ARG
    assert L.jvpfa_mask_summary(None, 1, 1, 64, None, None) == _lib.ERR_BAD_ARG
    m = _lib.Mask()
    m.ptr, m.kind, m.dtype = 4096, _lib.MASK_BOOL, 0
    m.stride[0], m.stride[1], m.stride[2], m.stride[3] = 64 * 64, 0, 64, 1
    # the summary buffer holds 64-bit words: it has to be 16-byte aligned (refused before anything is launched)
    assert L.jvpfa_mask_summary(C.byref(m), 1, 1, 64, C.c_void_p(4096 + 8), None) == _lib.ERR_BAD_ARG


def test_workspace_and_summary_sizes(built_library):
    from jvp_flash_attention_b200 import _lib
    b = _lib.BwdArgs()
    b.B, b.H, b.N, b.D, b.dtype = 2, 3, 100, 64, _lib.BF16
    assert built_library.jvpfa_bwd_workspace_bytes(C.byref(b)) == 256 + 2 * 3 * 100 * 16
    # 2 planes, 3 tiles of 64 along the sequence: tile flags (18 bytes, rounded up to 256) + the mask packed into 64-bit
    # words in both orientations (planes x tiles x 192 padded rows each) + one float per tile
    assert built_library.jvpfa_mask_summary_bytes(2, 1, 130) == 256 + 2 * (2 * 3 * 192 * 8) + 2 * 3 * 3 * 4


def test_python_api_error_behaviour():
    from jvp_flash_attention_b200.jvp_attention import JVPAttn, attention, MASK_CONST, MIN_SEQUENCE_LENGTH
    assert MASK_CONST == -100.0 and MIN_SEQUENCE_LENGTH == 32
    q = torch.randn(1, 2, 64, 64)
    big = torch.randn(1, 2, 64, 160)           # a head dimension of the CUDA-core kernels, which have no dropout
    with pytest.raises(NotImplementedError):
        attention(big, big, big, dropout_p=0.1)
    with pytest.raises(AssertionError):
        attention(q, q[..., :32], q)
    with pytest.raises(RuntimeError):          # CPU tensors: there is no CPU path
        attention(q, q, q)
    with pytest.raises(RuntimeError):
        JVPAttn.fwd_dual(q, q, q)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from jvp_flash_attention_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("JVPFA_LIBRARY", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no non-CUDA fallback"):
        _lib.lib()
