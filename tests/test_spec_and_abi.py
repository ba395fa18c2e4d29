"""Spec-string grammar, and the C-ABI library: it loads, exports every symbol the header declares, and rejects bad
arguments on the host (no kernel is launched in this file, so it runs without a GPU)."""
import ctypes
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_parse_vit_spec_matches_reference_table():
    import fastbb_b200 as fb
    assert fb.parse_vit_spec("fh-g0") == ("fh", False)
    assert fb.parse_vit_spec("hh-g1") == ("hh", True)
    assert fb.parse_vit_spec("ff-g2") == ("ff", "nofc2")
    assert fb.parse_vit_spec("sdpa-g3") == ("sdpa", "chunk")
    assert fb.parse_vit_spec("hh") == ("hh", False)            # no gemm part -> g0, as in the reference
    assert fb.parse_vit_spec("hh-g1-graph") == ("hh", True)    # suffix accepted everywhere
    assert fb.split_graph_suffix("hh-g1-graph") == ("hh-g1", True)
    assert fb.split_graph_suffix("fh-g0") == ("fh-g0", False)
    with pytest.raises(KeyError):
        fb.parse_vit_spec("hh-g7")
    with pytest.raises(ValueError):
        fb.parse_vit_spec("xx-g1")


def test_default_spec_from_environment(monkeypatch):
    import fastbb_b200 as fb
    monkeypatch.setenv("FASTBB_VIT", "hh-g1")
    assert importlib.reload(fb).DEFAULT_VIT == "hh-g1"
    monkeypatch.delenv("FASTBB_VIT")
    assert importlib.reload(fb).DEFAULT_VIT == "fh-g0"


def test_install_vit_off_leaves_module_alone():
    import torch
    import fastbb_b200 as fb
    m = torch.nn.Linear(2, 2)
    assert fb.install_vit(m, "off") is None
    assert m.weight.dtype == torch.float32 and "get_intermediate_layers" not in m.__dict__


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "fastbb_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fbb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from fastbb_b200 import _lib
    lib = _lib.load()
    names = _declared_functions()
    assert {"fbb_layernorm_f16", "fbb_linear_f16", "fbb_flash64_f16", "fbb_version"} <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/fastbb_b200.h but not exported"
        assert n in _lib.PROTOTYPES, f"{n} has no ctypes prototype in fastbb_b200/_lib.py"
    assert sorted(_lib.PROTOTYPES) == names
    assert lib.fbb_version() == 100


def test_attention_only_library_exports_the_attention_subset():
    """libfastbb_flash64.so (python -m fastbb_b200.build --flash-only) is what a project that vendors only attention.py
    and _lib.py loads: the attention entry points and the status calls, nothing else."""
    from fastbb_b200 import _lib, build
    lib = _lib.load(build.build(flash_only=True))
    assert lib.flash_only and lib.fbb_version() == 100
    for n in _declared_functions():
        assert hasattr(lib, n) == (n in _lib.FLASH_ONLY_SYMBOLS), n
    q = ctypes.c_void_p(256)
    assert lib.fbb_flash64_f16(q, q, q, q, 1, 8, 2, 1024, 128, 64, 1024, 128, 64, 1024, 128, 64, 1024, 128, 64, 0.125, 7, None) == -4


def test_missing_library_fails_loudly(tmp_path):
    from fastbb_b200 import _lib
    with pytest.raises(OSError, match="no fallback"):
        _lib.load(str(tmp_path / "libfastbb_b200.so"))


def test_argument_validation_on_the_host():
    from fastbb_b200 import _lib
    lib = _lib.load()
    A = 0x7F0000000000  # an aligned, never dereferenced address: every case below is rejected before any launch
    assert lib.fbb_linear_f16(None, A, A, None, None, None, 8, 8, 8, 8, 8, 8, 0, 0, 0, None) == -1
    assert lib.fbb_linear_f16(A, A, A, None, None, None, 8, 8, 12, 16, 16, 8, 0, 0, 0, None) == -2       # K % 8
    assert lib.fbb_linear_f16(A, A, A, None, None, None, 8, 12, 8, 8, 8, 16, 0, 0, 0, None) == -2       # N % 8
    assert lib.fbb_linear_f16(A + 2, A, A, None, None, None, 8, 8, 8, 8, 8, 8, 0, 0, 0, None) == -3     # alignment
    assert lib.fbb_linear_f16(A, A, A, None, None, None, 8, 8, 8, 8, 8, 8, 0, 7, 0, None) == -4         # epilogue enum
    assert lib.fbb_linear_f16(A, A, A, None, A, None, 8, 16, 8, 8, 8, 8, 8, 2, 0, None) == -2           # swiglu + res
    assert b"SwiGLU" in lib.fbb_last_error()
    assert lib.fbb_layernorm_f16(A, A, None, None, 4, 12, 12, 12, 1e-6, 0, 0, None) == -2               # C % 8
    assert lib.fbb_layernorm_f16(A, A, None, None, 4, 16, 16, 16, 1e-6, 9, 0, None) == -4
    s = [64 * 3 * 2, 64 * 3 * 2, 64] * 4
    assert lib.fbb_flash64_f16(A, A, A, A, 1, 4, 2, *s, 0.125, 5, None) == -4                           # variant
    assert lib.fbb_flash64_f16(A, A, A, A, 1, 4, 2, *s, -1.0, 0, None) == -2                            # scale <= 0
    bad = list(s); bad[1] = 100
    assert lib.fbb_flash64_f16(A, A, A, A, 1, 4, 2, *bad, 0.125, 0, None) == -3                         # stride % 8
    assert lib.fbb_flash64_f16(A, A, A, A, 0, 4, 2, *s, 0.125, 0, None) == 0                            # empty batch: no-op
    assert lib.fbb_linear_f16(A, A, A, None, None, None, 0, 8, 8, 8, 8, 8, 0, 0, 0, None) == 0          # M == 0: no-op
    assert lib.fbb_status_string(-3).decode().startswith("pointer or stride")


def test_python_wrappers_reject_cpu_tensors():
    import torch
    from fastbb_b200.attention import attention
    from fastbb_b200.gemm import linear
    from fastbb_b200.layernorm import layer_norm
    x = torch.zeros(4, 64, dtype=torch.float16)
    with pytest.raises(ValueError):
        layer_norm(x)
    with pytest.raises(ValueError):
        linear(x, torch.zeros(8, 64, dtype=torch.float16))
    with pytest.raises(ValueError):
        linear(x, torch.zeros(8, 64, dtype=torch.float16), act="relu")
    q = torch.zeros(1, 4, 2, 64, dtype=torch.float16)
    with pytest.raises(ValueError):
        attention(q, q, q)
    with pytest.raises(ValueError):
        attention(q, q, q, out=torch.zeros(1, 4, 2, 32, dtype=torch.float16))
