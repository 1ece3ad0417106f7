"""Writes tests/golden/op_surface.json: the names the reference's pybind module and dispatcher library export, and the
`launch_*` C symbols (with their parameter counts) that its torch-facing C++ expects from the CUDA side.

Run where the reference checkout is available:  python tests/golden/make_op_surface.py /path/to/reference
The fixture lets the CPU suite check, without the reference, that the Python operator surface is complete."""
import json
import re
import sys
from pathlib import Path


def main() -> None:
    root = Path(sys.argv[1])
    cpp = (root / "autonumerics_zero/spline_ops/spline_ops.cpp").read_text()
    module = cpp[cpp.index("PYBIND11_MODULE"):]
    pybind = re.findall(r'm\.def\(\s*"([a-z0-9_]+)"', module)
    library = cpp[cpp.index("TORCH_LIBRARY("):cpp.index("PYBIND11_MODULE")]
    schemas = re.findall(r'm\.def\(\s*"([a-z0-9_]+)\(', library)
    declarations = cpp[:cpp.index("PYBIND11_MODULE")]
    launch = [[name, params.count(",") + 1] for name, params in
              re.findall(r"void (launch_[a-z0-9_]+)\(([^)]*)\);", declarations)]
    out = {"source": "autonumerics_zero/spline_ops/spline_ops.cpp", "pybind": pybind, "dispatcher": sorted(set(schemas)),
           "launch_symbols": launch}
    Path(__file__).with_name("op_surface.json").write_text(json.dumps(out, indent=1) + "\n")
    print(len(pybind), "pybind names,", len(out["dispatcher"]), "dispatcher schemas,", len(launch), "launch symbols")


if __name__ == "__main__":
    main()
