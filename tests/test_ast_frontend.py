"""What the AST front end refuses, and a few things it evaluates at trace time (CPU).
Messages follow the reference's src/mytriton/ast_frontend.py."""

import numpy as np
import pytest

import mytriton_b200 as triton
import mytriton_b200.language as tl
from mytriton_b200.ast_frontend import ASTFrontendError
from mytriton_b200.ssa import SSAForRange

OUT = np.zeros(8, dtype=np.float32)
FACTOR = 3


@triton.jit
def returns_kernel(out):
    return 1


@triton.jit
def tuple_assign_kernel(out):
    a, b = 1, 2
    tl.store(out, a + b)


@triton.jit
def while_kernel(out, n):
    while n:
        tl.store(out, 1.0)


@triton.jit
def symbolic_if_kernel(out, n):
    value = 1.0 if n < 3 else 2.0
    tl.store(out, value)


@triton.jit
def for_over_list_kernel(out):
    for k in [1, 2, 3]:
        tl.store(out + k, 1.0)


@triton.jit
def chained_comparison_kernel(out, n):
    lanes = tl.arange(0, 8)
    tl.store(out + lanes, 1.0, mask=0 < lanes < n)


@triton.jit
def unknown_name_kernel(out):
    tl.store(out, missing_name)  # noqa: F821


@triton.jit
def constexpr_branch_kernel(out, n, DOUBLE: tl.constexpr):
    lanes = tl.arange(0, 8)
    scale = 2.0 if DOUBLE else 1.0
    tl.store(out + lanes, lanes * scale * FACTOR, mask=lanes < n)


@triton.jit
def constexpr_if_statement_kernel(x, out, n, ACTIVATION: tl.constexpr):
    lanes = tl.arange(0, 8)
    mask = lanes < n
    values = tl.load(x + lanes, mask=mask)
    if ACTIVATION == "relu":
        values = tl.maximum(values, 0.0)
    elif ACTIVATION == "neg":
        values = -values
    else:
        pass
    tl.store(out + lanes, values, mask=mask)


@triton.jit
def greater_than_kernel(out, n):
    lanes = tl.arange(0, 8)
    tl.store(out + lanes, 1.0, mask=(lanes > 1) & (0 < lanes) & (n > lanes))


@triton.jit
def symbolic_if_statement_kernel(out, n):
    if n < 3:
        tl.store(out, 1.0)


@triton.jit
def static_loop_kernel(out, REPEAT: tl.constexpr):
    total = 0.0
    for k in tl.static_range(1, REPEAT + 1):
        total += k
    for k in range(2):                      # Python ints: unrolled as well
        total = total * 2.0
    tl.store(out, total)


@triton.jit
def loop_local_name_kernel(out, n):
    acc = 0
    for k in range(n):
        twice = k + k                       # created inside the loop: not carried
        acc = acc + twice
    tl.store(out, acc)


@pytest.mark.parametrize("kernel,args,message", [
    (returns_kernel, (OUT,), "return statements are not supported"),
    (tuple_assign_kernel, (OUT,), "only assignment to a simple name"),
    (while_kernel, (OUT, 3), "a while condition must be a scalar boolean"),
    (symbolic_if_kernel, (OUT, 3), "only constexpr conditions in IfExp"),
    (for_over_list_kernel, (OUT,), r"only for \.\.\. in range"),
    (chained_comparison_kernel, (OUT, 3), "wrap each comparison in parentheses"),
])
def test_rejected_constructs(kernel, args, message):
    with pytest.raises(ASTFrontendError, match=message):
        kernel[(1,)](*args)


def test_unknown_names_are_name_errors():
    with pytest.raises(NameError, match="missing_name"):
        unknown_name_kernel[(1,)](OUT)


def test_symbolic_values_cannot_drive_python_control_flow():
    lanes = tl.arange(0, 4)
    with pytest.raises(TypeError, match="Python control flow over symbolic values"):
        bool(lanes < 2)


def test_constexpr_conditions_globals_and_static_loops_fold_at_trace_time():
    _, ssa_doubled, _ = constexpr_branch_kernel[(1,)](OUT, 8, DOUBLE=True)
    _, ssa_plain, _ = constexpr_branch_kernel[(1,)](OUT, 8, DOUBLE=False)
    assert any(op.opcode == "mul" and op.operands[1].value == 2.0 for op in ssa_doubled)
    assert any(op.opcode == "mul" and op.operands[1].value == 3 for op in ssa_plain)   # FACTOR
    _, ssa_ops, src = static_loop_kernel[(1,)](OUT, REPEAT=3)
    assert not any(isinstance(op, SSAForRange) for op in ssa_ops)
    assert "24.0f" in src                                   # (1 + 2 + 3) * 2 * 2, folded


def test_if_statements_on_constexpr_conditions_pick_a_branch_at_trace_time():
    opcodes = {}
    for choice in ("relu", "neg", "none"):
        _, ssa_ops, _ = constexpr_if_statement_kernel[(1,)](OUT, OUT, 8, ACTIVATION=choice)
        opcodes[choice] = [op.opcode for op in ssa_ops]
    assert "maximum" in opcodes["relu"] and "neg" not in opcodes["relu"]
    assert "neg" in opcodes["neg"] and "maximum" not in opcodes["neg"]
    assert "neg" not in opcodes["none"] and "maximum" not in opcodes["none"]
    # a condition on a run-time scalar is lowered by predication (tests/test_control_flow.py)
    _, ssa_ops, _ = symbolic_if_statement_kernel[(1,)](OUT, 3)
    assert [op.opcode for op in ssa_ops] == ["cmp_lt", "store"]


def test_greater_than_and_reflected_less_than_lower_to_less():
    """a > b is b < a; a Python number on the left of < is a constant operand."""
    _, ssa_ops, _ = greater_than_kernel[(1,)](OUT, 5)
    compares = [op for op in ssa_ops if op.opcode == "cmp_lt"]
    assert len(compares) == 3
    from mytriton_b200.ssa import SSAPrinter
    from oracle import ssa_interp
    out = np.zeros(8, dtype=np.float32)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"out": out, "n": 5}, (1,))
    assert out.tolist() == [0, 0, 1, 1, 1, 0, 0, 0]


def test_only_preexisting_names_are_loop_carried():
    _, ssa_ops, _ = loop_local_name_kernel[(1,)](OUT, 3)
    (loop,) = [op for op in ssa_ops if isinstance(op, SSAForRange)]
    assert len(loop.carried_args) == 1 and len(loop.body) == 2


def test_static_range_wants_python_ints():
    with pytest.raises(ValueError, match="static_range stop must be compile-time int"):
        tl.static_range(0, 2.5)
    assert list(tl.static_range(3)) == [0, 1, 2]
