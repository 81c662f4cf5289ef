"""CPU-side checks: the shared library loads, exports every symbol include/kda_b200.h
declares, the ctypes mirror of KdaParams matches the C struct, and the backend contract
mirrors the reference's checks (tests/test_backends.py of the reference)."""
import ctypes as C
import os
import re
import subprocess
import sys
from types import ModuleType

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header():
    return open(os.path.join(ROOT, "include", "kda_b200.h")).read()


def test_library_exports_every_declared_symbol():
    from openkimi_b200 import _lib

    lib = _lib.load()
    declared = set(re.findall(r"\b(kda_[a-z0-9_]+)\s*\(", _header()))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.kda_abi_version() == 4
    assert lib.kda_guard_version() == 1 and lib.kda_guard_max_span() == 232.0
    assert lib.kda_guard_dot_precision() == b"tf32x3"
    assert b"NULL" in lib.kda_status_string(1)


def test_params_struct_matches_header(tmp_path):
    """Compile a tiny C program against the header and compare sizeof/offsetof with ctypes."""
    from openkimi_b200 import _lib

    fields = [f[0] for f in _lib.KdaParams._fields_]
    prog = '#include <stdio.h>\n#include <stddef.h>\n#include "kda_b200.h"\nint main(){printf("%zu\\n", sizeof(KdaParams));\n'
    prog += "".join(f'printf("%zu\\n", offsetof(KdaParams, {f}));\n' for f in fields) + "return 0;}\n"
    src = tmp_path / "probe.c"
    src.write_text(prog)
    exe = tmp_path / "probe"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert out[0] == C.sizeof(_lib.KdaParams)
    assert out[1:] == [getattr(_lib.KdaParams, f).offset for f in fields]


def test_validation_rejects_bad_arguments_without_a_gpu():
    """Argument checks run on the host before any launch."""
    from openkimi_b200 import _lib

    lib = _lib.load()
    p = _lib.KdaParams()
    assert lib.kda_fwd(None, None) == 1
    p.dtype = 7
    assert lib.kda_fwd(C.byref(p), None) == 3
    p.dtype = 1
    p.B, p.T, p.H, p.N, p.NT, p.dk, p.dv = 1, 64, 1, 1, 1, 96, 96
    assert lib.kda_fwd(C.byref(p), None) == 2
    p.dk = p.dv = 128
    assert lib.kda_fwd(C.byref(p), None) == 1  # NULL tensors
    fb, bb = C.c_size_t(), C.c_size_t()
    assert lib.kda_workspace_bytes(C.byref(p), C.byref(fb), C.byref(bb)) == 0
    assert fb.value > 0 and bb.value > 0 and fb.value % 256 == 0
    # a forward-only call (KDA_FLAG_NO_SAVE) needs less than half of the saving forward's workspace
    full = fb.value
    p.flags = _lib.FLAG_NO_SAVE
    assert lib.kda_workspace_bytes(C.byref(p), C.byref(fb), C.byref(bb)) == 0
    assert 0 < fb.value < full // 2


def test_fused_convolution_arguments_are_validated_without_a_gpu():
    """The fused short convolution (KdaParams.conv_*): all three filters or none, 1..4 taps, BF16 with
    dk = 128 only, and a larger workspace.  Every case fails before any launch, so fake (aligned,
    never dereferenced) addresses stand in for the tensors."""
    from openkimi_b200 import _lib

    lib = _lib.load()
    p = _lib.KdaParams()
    p.B, p.T, p.H, p.N, p.NT, p.dk, p.dv = 1, 64, 1, 1, 1, 128, 128
    p.dtype, p.guard_span = _lib.DTYPE_BF16, 232.0
    for name in ("q", "k", "v", "g", "beta", "o", "workspace"):
        setattr(p, name, 4096)
    fb0, fb1, bb = C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert lib.kda_workspace_bytes(C.byref(p), C.byref(fb0), C.byref(bb)) == 0
    p.conv_q = 4096
    assert lib.kda_fwd(C.byref(p), None) == 1            # conv_k, conv_v missing
    p.conv_k = p.conv_v = 4096
    p.conv_ksize = 5
    assert lib.kda_fwd(C.byref(p), None) == 2
    p.conv_ksize = 4
    assert lib.kda_workspace_bytes(C.byref(p), C.byref(fb1), C.byref(bb)) == 0
    assert fb1.value == fb0.value + 64 * 128 * 2         # one BF16 [64][dv] record per unit more
    p.workspace_bytes = fb0.value
    assert lib.kda_fwd(C.byref(p), None) == 4            # workspace too small for the fused call
    p.dtype = _lib.DTYPE_F32
    assert lib.kda_fwd(C.byref(p), None) == 10           # FP32 has no fused convolution
    p.dtype, p.flags = _lib.DTYPE_BF16, _lib.FLAG_FORCE_SIMT
    assert lib.kda_fwd(C.byref(p), None) == 10
    assert b"short convolution" in lib.kda_status_string(10)


def _patched(version=1, span=232.0, precision="tf32x3"):
    m = ModuleType("chunk_intra")
    m.OPENKIMI_KDA_GUARDED_DIAGONAL_VERSION = version
    m._OPENKIMI_GUARD_MAX_LOG2_SPAN = span
    m._OPENKIMI_GUARD_DOT_PRECISION = precision
    return m


def test_guard_contract_name_and_rejections():
    from openkimi_b200 import chunk_intra, validated_kda_backend_name

    assert validated_kda_backend_name(_patched()).endswith("(openkimi_guarded_diagonal_v1,tf32x3,span<=232)")
    assert validated_kda_backend_name(chunk_intra).endswith("span<=232)")
    for module, message in ((_patched(version=0), "guarded KDA patch v1"),
                            (_patched(span=240.0), "exceeds the validated maximum 232"),
                            (_patched(precision="tf32"), "is not validated")):
        with pytest.raises(RuntimeError, match=message):
            validated_kda_backend_name(module)


def test_reference_validator_accepts_our_contract_module():
    """The attribute names and types are the ones the reference's own validator reads
    (k3mini/backends.py:68-109): version int 1, span a finite float <= 232, precision str."""
    from openkimi_b200 import chunk_intra

    assert chunk_intra.OPENKIMI_KDA_GUARDED_DIAGONAL_VERSION == 1
    assert isinstance(chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN, float)
    assert chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN <= 232.0
    assert chunk_intra._OPENKIMI_GUARD_DOT_PRECISION == "tf32x3"


def test_no_gpu_means_loud_failure():
    import torch

    from openkimi_b200 import chunk_kda, resolve_kda_backend

    if torch.cuda.is_available():
        pytest.skip("GPU present")
    q = torch.zeros(1, 64, 1, 64)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        chunk_kda(q, q, q, q, torch.zeros(1, 64, 1))
    with pytest.raises(RuntimeError, match="sm_100"):
        resolve_kda_backend()


def test_product_never_imports_the_oracle():
    """No file of the package imports, opens or shells out to anything under oracle/ (citations of
    the reference's own ``*_oracle.py`` file names in comments are fine)."""
    pkg = os.path.join(ROOT, "openkimi_b200")
    bad = re.compile(r"^\s*(from|import)\s+oracle\b|[\"']oracle[/\"']|oracle\.kda_|import_module\(.oracle", re.M)
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not bad.search(text), f
