"""CPU: the C-ABI library loads, exports every declared symbol and rejects bad arguments
before any launch (no GPU needed: validation happens first, and without a device the
entry points report FPT_ERR_NO_DEVICE instead of computing)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols(header_name="fpt_b200.h"):
    names = []
    for header in [ROOT / "include" / header_name]:
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        names += re.findall(r"\b((?:fpt|launch)_\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol(fpt):
    lib = fpt.load()
    names = declared_symbols()
    assert len(names) >= 12
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_compat_header_symbols_are_all_exported():
    lib = ctypes.CDLL(str(ROOT / "fast_polynomial_transcendentals_b200" / "libfpt_b200_compat.so"))
    names = declared_symbols("fpt_b200_compat.h")
    assert len(names) == 223
    assert not [n for n in names if not hasattr(lib, n)]


def test_every_header_is_covered():
    assert sorted(p.name for p in (ROOT / "include").glob("*.h")) == ["fpt_b200.h", "fpt_b200_compat.h"]


def test_every_bound_signature_is_declared(fpt):
    declared = set(declared_symbols())
    assert set(fpt.SIGNATURES) <= declared


def test_program_table_matches_golden(fpt):
    import json
    lib = fpt.load()
    fixture = json.loads((ROOT / "tests/golden/program_table.json").read_text())
    assert lib.fpt_program_count() == len(fixture)
    shapes = ("ODD_HALF", "ODD", "ODD_SAT", "SWISH", "XMUL_HALF", "EVEN", "ALG_SIG", "ALG_TANH")
    for i, want in enumerate(fixture):
        name = ctypes.create_string_buffer(32)
        dt, src, shape, deg = (ctypes.c_int() for _ in range(4))
        clamp = ctypes.c_uint16()
        coeffs = (ctypes.c_uint16 * 7)()
        assert lib.fpt_program_info(i, name, 32, dt, src, shape, deg, ctypes.byref(clamp), coeffs) == 0
        assert name.value.decode() == want["name"]
        assert (dt.value, src.value) == ({"fp16": 0, "bf16": 1}[want["dtype"]], {"current": 0, "sollya": 1}[want["source"]])
        assert shapes[shape.value] == want["shape"] and deg.value == want["degree"] and clamp.value == want["clamp"]
        assert list(coeffs)[:len(want["coeffs"])] == want["coeffs"]


def test_argument_validation_happens_before_launch(fpt):
    lib = fpt.load()
    p = ctypes.c_void_p(256)
    assert lib.fpt_unary(p, p, -1, 0, 0, 3, 0, 0, None) == -2          # negative size
    assert lib.fpt_unary(None, p, 8, 0, 0, 3, 0, 0, None) == -1        # null pointer
    assert lib.fpt_unary(p, p, 8, 0, 0, 3, 7, 0, None) == -5           # bad dtype
    assert lib.fpt_unary(p, p, 8, 0, 0, 3, 0, 9, None) == -5           # bad source
    assert lib.fpt_unary(p, p, 8, 0, 0, 9, 0, 0, None) == -4           # no degree-9 program
    assert lib.fpt_unary(p, p, 8, 0, 0, 3, 0, 1, None) == -4           # fp16 has no sollya source
    assert lib.fpt_swish_mul(p, p, None, 8, 3, 1, 0, None) == -1
    assert lib.fpt_swish_mul_packed(p, p, -3, 8, 3, 1, 0, None) == -2
    assert lib.fpt_bwd_algebraic(p, p, p, 8, 2, 0, None) == -4         # only sigmoid / tanh
    assert lib.fpt_unary(p, p, 0, 0, 0, 3, 0, 0, None) == 0            # empty input is a no-op
    assert b"size" in lib.fpt_status_string(-2)
    assert lib.fpt_set_tuning(b"nonsense", 1) == -5


def test_without_a_gpu_the_library_refuses_instead_of_falling_back(fpt):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = fpt.load()
    p = ctypes.c_void_p(256)
    assert lib.fpt_unary(p, p, 8, 0, 0, 3, 0, 0, None) == -7
    with pytest.raises(fpt.FptError):
        fpt.call("fpt_unary", p, p, 8, 0, 0, 3, 0, 0, None)


def test_op_surface_rejects_cpu_tensors():
    import torch
    from fast_polynomial_transcendentals_b200 import spline_ops
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        spline_ops.sigmoid_fwd_d3(torch.zeros(8, dtype=torch.float16))


def test_compat_library_exports_every_launch_symbol_of_the_reference():
    """libfpt_b200_compat.so carries the reference's launch_* names (fixture written from the reference's C++ by
    tests/golden/make_op_surface.py); the generated header declares each with the same number of parameters."""
    import ctypes
    import json
    import re
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    lib_path = root / "fast_polynomial_transcendentals_b200" / "libfpt_b200_compat.so"
    assert lib_path.exists(), "build the library first: python -m fast_polynomial_transcendentals_b200.build"
    lib = ctypes.CDLL(str(lib_path))
    surface = json.loads((root / "tests" / "golden" / "op_surface.json").read_text())
    header = (root / "include" / "fpt_b200_compat.h").read_text()
    declared = {name: params.count(",") + 1 for name, params in re.findall(r"void (launch_[a-z0-9_]+)\(([^)]*)\);", header)}
    assert len(surface["launch_symbols"]) == 221
    for name, parameter_count in surface["launch_symbols"]:
        assert hasattr(lib, name), name
        assert declared.get(name) == parameter_count, (name, declared.get(name), parameter_count)
    assert lib.fpt_compat_symbol_count() == len(declared) == 221
    assert lib.fpt_compat_last_status() == 0
