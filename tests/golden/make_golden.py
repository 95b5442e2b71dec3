"""Regenerates tests/golden/corpus_golden.json from the reference implementation.

Run where the reference is importable (it is pure Python, needs only NumPy):

    PYTHONPATH=<reference>/src CORPUS_IMPL=reference python tests/golden/make_golden.py

For every case in mytriton_b200/kernel_cases.py the reference compiles the corpus kernel with
NumPy arguments (its compile-only path) and this script records what it printed:
the traced expression tree (dataclass repr), the typed-SSA text, the CUDA C++ source it would hand to NVRTC, and the CTA size
it would launch with — or, when it refuses the kernel, the exception class and
message.  The JSON is what the parity tests compare against and what the GPU
tests compile and run as "the reference's own generated kernels".
"""

from __future__ import annotations

import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

if os.environ.get("CORPUS_IMPL") != "reference":
    raise SystemExit("set CORPUS_IMPL=reference and put the reference's src/ on PYTHONPATH")

from mytriton_b200 import kernel_cases as cases  # noqa: E402
from mytriton_b200 import kernels as corpus  # noqa: E402
from mytriton.block_shapes import cuda_threads_per_block  # noqa: E402
from mytriton.ssa import SSAPrinter  # noqa: E402


def main() -> None:
    golden = {}
    for case in cases.CASES:
        kernel = getattr(corpus, case.kernel)
        kernel.clear_cache()
        entry: dict[str, object] = {"kernel": case.kernel}
        try:
            ops, ssa_ops, src = kernel[case.grid](*cases.build_args(case), **case.constexprs)
        except Exception as error:  # the reference's verdict, whatever it is
            entry["error"] = {"type": type(error).__name__, "message": str(error)}
        else:
            entry["ops_repr"] = repr(ops)          # the traced expression tree, dataclass repr
            entry["ssa"] = SSAPrinter().print_ops(ssa_ops)
            entry["cuda_src"] = src
            entry["threads_per_block"] = cuda_threads_per_block(ssa_ops)
        golden[case.name] = entry
    path = HERE / "corpus_golden.json"
    path.write_text(json.dumps(golden, indent=1, sort_keys=True) + "\n")
    print(f"wrote {path} ({len(golden)} cases)")


if __name__ == "__main__":
    main()
