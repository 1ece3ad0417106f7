"""Writes tests/golden/attention_numerics.json: the polynomial-vs-native error statistics the reference publishes for
its attention components B2 (tanh soft-cap D4) and B3 (direct sigmoid D3 / coupled D4), forward output and gradients,
at B=1, Hq=32, Hkv=8, S=4096, D=128 on N(0,1) bf16 inputs, and for the element-wise sites B1 (SiLU D3, 58 720 256
elements) and B4 (SwiGLU D3, 24 576 x 1280) against the degree-0 SFU kernels.

    python tests/golden/make_attention_numerics.py /path/to/reference
"""
import json
import sys
from pathlib import Path


def main() -> None:
    source = Path(sys.argv[1]) / "evidence/report-data/b1_b4_100_iteration_phase_probes_gb200.json"
    rows = json.loads(source.read_text())["rows"]
    out = {"source": "evidence/report-data/b1_b4_100_iteration_phase_probes_gb200.json",
           "metric_definitions": "scripts/benchmark_components.py:134-147 (max_abs, mean_abs, relative_mae = mean|a-b| / mean|b|, cosine)"}
    for row in rows:
        if row.get("case") in ("B2", "B3"):
            out[row["case"]] = {"shape": row["shape"], "configuration": row["configuration"], "tensors": row["numerics"]["tensors"]}
        if row.get("case") in ("B1", "B4"):      # element-wise sites: SiLU D3 and SwiGLU D3 against the degree-0 (SFU) kernels
            out[row["case"]] = {"shape": row["shape"], "tensors": row["numerics"]}
    Path(__file__).with_name("attention_numerics.json").write_text(json.dumps(out, indent=1) + "\n")
    print({k: list(v["tensors"]) for k, v in out.items() if isinstance(v, dict) and "tensors" in v})


if __name__ == "__main__":
    main()
