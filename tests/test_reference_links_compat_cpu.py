"""CPU: the reference's torch-facing C++ (autonumerics_zero/spline_ops/spline_ops.cpp, which declares 221 `launch_*`
kernels launchers as `extern "C"` and defines none of them) compiles unchanged and links, with no undefined symbol
left, against libfpt_b200_compat.so in place of the reference's three .cu files; the resulting extension module imports
and exposes the reference's operator names.  Needs a checkout of the reference (FPT_REFERENCE_ROOT, or a directory
`reference` beside this repository); skipped elsewhere.  Nothing here runs a kernel."""
import json
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "fast_polynomial_transcendentals_b200"
REFERENCE = Path(os.environ.get("FPT_REFERENCE_ROOT", ROOT.parent / "reference"))
SOURCE = REFERENCE / "autonumerics_zero" / "spline_ops" / "spline_ops.cpp"


@pytest.mark.skipif(not SOURCE.exists(), reason="no checkout of the reference here")
def test_reference_extension_links_against_the_compat_library(tmp_path):
    import torch
    from torch.utils import cpp_extension
    out = tmp_path / ("spline_ops" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
    cuda_home = Path(cpp_extension.CUDA_HOME or "/usr/local/cuda")
    includes = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"], str(cuda_home / "include")]
    libdirs = cpp_extension.library_paths()
    version = f"{sys.version_info.major}.{sys.version_info.minor}"
    cmd = ["g++", "-O1", "-std=c++17", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=spline_ops",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{i}" for i in includes], str(SOURCE), "-o", str(out), *[f"-L{d}" for d in libdirs],
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           f"-L{PKG}", "-lfpt_b200_compat", f"-L{cuda_home / 'lib64'}", "-lcudart",
           f"-L{sysconfig.get_config_var('LIBDIR')}", f"-lpython{version}",
           "-Wl,--no-undefined", f"-Wl,-rpath,{PKG}", *[f"-Wl,-rpath,{d}" for d in libdirs]]
    built = subprocess.run(cmd, capture_output=True, text=True)
    assert built.returncode == 0, built.stderr[-3000:]      # --no-undefined: every launch_* was found in the library

    def symbols(path, flag):
        listing = subprocess.run(["nm", "-D", flag, str(path)], capture_output=True, text=True, check=True).stdout
        return {line.split()[-1] for line in listing.splitlines() if " launch_" in line or line.strip().startswith("U launch_")}
    wanted = symbols(out, "--undefined-only")
    offered = symbols(PKG / "libfpt_b200_compat.so", "--defined-only")
    assert len(wanted) > 200 and wanted <= offered, sorted(wanted - offered)[:5]
    # the module imports in a fresh interpreter and carries the reference's operator names
    code = ("import sys, json, torch; sys.path.insert(0, sys.argv[1]); import spline_ops; "
            "print(json.dumps(sorted(n for n in dir(spline_ops) if not n.startswith('_'))))")
    listed = subprocess.run([sys.executable, "-c", code, str(tmp_path)], capture_output=True, text=True)
    assert listed.returncode == 0, listed.stderr[-2000:]
    names = set(json.loads(listed.stdout.strip().splitlines()[-1]))
    golden = json.loads((ROOT / "tests" / "golden" / "op_surface.json").read_text())
    expected = set(golden["pybind"]) if isinstance(golden, dict) and "pybind" in golden else None
    assert {"sigmoid_fwd", "swish_mul_packed_fwd_variant", "rope_apply_fixed_half_turn_d5_d6_fp16"} <= names
    if expected:
        assert expected <= names, sorted(expected - names)[:5]
