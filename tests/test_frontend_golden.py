"""The front end against the reference's own output (CPU only).

tests/golden/corpus_golden.json was produced by compiling the corpus with the
reference package (see tests/golden/make_golden.py).  The typed-SSA text this
package prints must match it character for character, and kernels the reference
rejects must be rejected with the same exception type and message — except
where this backend deliberately lifts a limit (blocks wider than 1024 threads).
"""

import pytest

from mytriton_b200 import kernel_cases as cases
from mytriton_b200 import kernels as corpus
from mytriton_b200.ssa import SSAPrinter

LIFTED_LIMITS = {"softmax_4096"}  # reference: "CUDA threads per block must be between 1 and 1024"


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_case_matches_reference(case, golden):
    kernel = getattr(corpus, case.kernel)
    kernel.clear_cache()
    expected = golden[case.name]
    arguments = cases.build_args(case)

    if "error" in expected and case.name not in LIFTED_LIMITS:
        with pytest.raises(Exception) as caught:
            kernel[case.grid](*arguments, **case.constexprs)
        lineage = [cls.__name__ for cls in type(caught.value).__mro__]
        assert expected["error"]["type"] in lineage
        assert str(caught.value) == expected["error"]["message"]
        return

    ops, ssa_ops, src = kernel[case.grid](*arguments, **case.constexprs)
    assert ops
    assert f"void {case.kernel}(" in src
    if "ssa" in expected:
        assert SSAPrinter().print_ops(ssa_ops) == expected["ssa"]
        # the expression tree itself: same node classes, fields, captures and loop structure
        assert repr(ops) == expected["ops_repr"]


def test_reference_rejects_what_this_backend_lifts(golden):
    assert golden["softmax_4096"]["error"]["type"] == "ValueError"
    assert "between 1 and 1024" in golden["softmax_4096"]["error"]["message"]


def test_kernel_signature_matches_reference(golden):
    """Same symbol, same parameter order and C types as the reference's source."""
    for case in cases.CASES:
        expected = golden[case.name]
        if "cuda_src" not in expected:
            continue
        kernel = getattr(corpus, case.kernel)
        _, _, src = kernel[case.grid](*cases.build_args(case), **case.constexprs)
        theirs = expected["cuda_src"].split("void ", 1)[1].split(")", 1)[0]
        mine = src.split("void ", 1)[1].split(")", 1)[0]
        assert mine == theirs, case.name
