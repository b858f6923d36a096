"""canonicalize, pattern by pattern: identity operands, idempotent operations, involutions, conversions through a
wider type, division by a power of two, arithmetic on splat constants, no-op broadcasts; and what it must leave alone.
Every case also checks, through the interpreter, that results are bit-identical with direct mode (rtol = atol = 0)."""
import numpy as np
import pytest

from nkipy_b200.nkigen import trace

from ..harness import run_kernel_test

R = np.random.default_rng(8)
X = R.standard_normal((8, 16)).astype(np.float32)
Y = R.standard_normal((8, 16)).astype(np.float32)
SPEC = ((8, 16), "f32")
EXACT = dict(rtol=0, atol=0)


def run(fn, inputs, check, n_inputs=None):
    k = trace(input_specs=[SPEC] * len(inputs))(fn)
    return run_kernel_test(k, inputs, passes=["canonicalize"], check=check, **EXACT)


@pytest.mark.parametrize("fn", [lambda x: 1.0 * x, lambda x: x * 1.0, lambda x: 0.0 + x, lambda x: x - 0.0,
                                lambda x: x / 1.0, lambda x: x ** 1.0, lambda x: ((x * 1.0) / 1.0 - 0.0) ** 1.0],
                         ids=["one_times", "times_one", "zero_plus", "minus_zero", "over_one", "power_one", "chain"])
def test_identity_operands_disappear(fn):
    g = run(lambda x: np.exp(fn(x)), [X], "CHECK-NOT: mul(\nCHECK-NOT: add(\nCHECK-NOT: sub(\nCHECK-NOT: div(\nCHECK-NOT: pow(\nCHECK: exp(")
    assert [n.opcode for n in g.nodes] == ["exp"]


def test_identity_fold_does_not_drop_a_broadcast():
    # (8,16) * ones is the identity, but a [16] vector times a splat of shape [8,16] is a broadcast that must stay
    k = trace(input_specs=[((16,), "f32")])(lambda v: v * np.ones((8, 16), np.float32))
    g = run_kernel_test(k, [X[0]], passes=["canonicalize"], **EXACT)
    assert tuple(g.outputs[0].shape) == (8, 16)


@pytest.mark.parametrize("fn,left", [(lambda x: np.maximum(x, x), "max("), (lambda x: np.minimum(x, x), "min("),
                                     (lambda x: np.where(x > 0, x, x), "select(")], ids=["max", "min", "select"])
def test_idempotent_operations(fn, left):
    run(lambda x: fn(x) + 1.0, [X], f"CHECK-NOT: {left}\nCHECK: add(")


def test_logical_idempotence():
    def k(x, y):
        m = x > y
        return np.where(np.logical_and(m, m), x, y), np.where(np.logical_or(m, m), y, x)

    run(k, [X, Y], "CHECK-NOT: and(\nCHECK-NOT: or(\nCHECK-COUNT-2: select(")


def test_involutions():
    def k(x, y):
        return -(-x), np.abs(np.abs(y)), np.abs(-x), np.where(np.logical_not(np.logical_not(x > y)), x, y)

    g = run(k, [X, Y], "CHECK-NOT: neg(\nCHECK-NOT: not(\nCHECK-COUNT-2: abs(")
    assert g.results[0] is g.params[0]


def test_round_trip_through_a_wider_type_disappears():
    k = trace(input_specs=[((8, 16), "f16")])(lambda h: h.astype(np.float32).astype(np.float16) * np.float16(2))
    run_kernel_test(k, [X.astype(np.float16)], passes=["canonicalize"], check="CHECK-NOT: convert(\nCHECK: mul(", **EXACT)


def test_round_trip_through_a_narrower_type_stays():
    run(lambda x: x.astype(np.float16).astype(np.float32) + 1.0, [X], "CHECK-COUNT-2: convert(")


def test_conversion_chains_collapse_when_the_first_step_is_lossless():
    k = trace(input_specs=[((8, 16), "i8")])(lambda b: b.astype(np.int32).astype(np.float32) * 0.5)
    g = run_kernel_test(k, [R.integers(-100, 100, (8, 16)).astype(np.int8)], passes=["canonicalize"],
                        check="CHECK-COUNT-1: convert(", **EXACT)
    (cv,) = [n for n in g.nodes if n.opcode == "convert"]
    assert np.dtype(cv.inputs[0].dtype) == np.int8 and np.dtype(cv.outputs[0].dtype) == np.float32
    # f32 -> i32 -> f32 truncates: both conversions stay
    run(lambda x: (x * 10).astype(np.int32).astype(np.float32), [X], "CHECK-COUNT-2: convert(")


@pytest.mark.parametrize("divisor", [2.0, 4.0, 0.125, 1024.0, -8.0])
def test_division_by_a_power_of_two_becomes_a_multiplication(divisor):
    run(lambda x: x / divisor, [X], "CHECK-NOT: div(\nCHECK: mul(")


@pytest.mark.parametrize("divisor", [3.0, 10.0, 0.3, 6.0])
def test_other_divisors_stay(divisor):
    run(lambda x: x / divisor, [X], "CHECK-NOT: mul(\nCHECK: div(")


def test_arithmetic_on_splat_constants_is_folded():
    def k(x):
        scale = np.full((8, 16), 3.0, np.float32) * 2.0 - np.sqrt(np.full((8, 16), 16.0, np.float32))      # 2
        bias = np.maximum(np.full((8, 16), -1.0, np.float32), 0.5) + np.abs(-np.ones((8, 16), np.float32))  # 1.5
        return x * scale + bias

    g = run(k, [X], "CHECK-COUNT-1: mul(\nCHECK-COUNT-1: add(\nCHECK-NOT: sqrt(\nCHECK-NOT: max(\nCHECK-NOT: abs(\nCHECK-NOT: sub(")
    consts = sorted(float(np.asarray(n.attrs["value"]).reshape(-1)[0]) for n in g.nodes if n.opcode == "constant")
    assert consts == [1.5, 2.0]


def test_folding_a_splat_expression_can_expose_an_identity():
    # (0.5 + 0.5) is folded to 1, then x * 1 goes away: needs the second round
    g = run(lambda x: np.tanh(x * (np.float32(0.5) + np.full((8, 16), 0.5, np.float32))), [X], "CHECK-NOT: mul(\nCHECK: tanh(")
    assert [n.opcode for n in g.nodes] == ["tanh"]


def test_non_splat_constants_are_not_folded():
    from nkipy_b200.core.tensor_apis import constant

    table = np.arange(128, dtype=np.float32).reshape(8, 16)
    k = trace(input_specs=[SPEC])(lambda x: x + np.abs(constant(table) * 2.0))
    text_kernel = lambda x: x + np.abs(table * 2.0)
    from ..harness import ir_after, filecheck

    filecheck(ir_after(k, passes=["canonicalize"]), "CHECK: mul(\nCHECK: abs(\nCHECK: add(")
    run(text_kernel, [X], "CHECK: add(")


def test_a_broadcast_to_the_same_shape_disappears():
    run(lambda x: np.broadcast_to(x, (8, 16)) + 1.0, [X], "CHECK-NOT: broadcast(%0\nCHECK: add(")


def test_things_that_look_foldable_but_are_not():
    # x - x is NaN for infinities, x * 0 likewise; x / x too: all stay
    run(lambda x: (x - x) + (x * 0.0) + (x / x), [X], "CHECK: sub(\nCHECK: mul(\nCHECK: div(")


def test_a_result_may_become_a_parameter():
    g = run(lambda x, y: (x * 1.0, y + x), [X, Y], "CHECK-NOT: mul(\nCHECK: add(")
    assert g.results[0] is g.params[0]


def test_a_constant_of_equal_elements_is_stored_as_one_scalar():
    from nkipy_b200.core.tensor_apis import constant

    big = np.full((64, 128), 0.25, np.float32)
    k = trace(input_specs=[((64, 128), "f32")])(lambda x: x * constant(big))
    from ..harness import ir_after

    before, after = k.to_ir(), ir_after(k, passes=["canonicalize"])
    assert len(after) < len(before) // 20                      # 32 KiB of base64 became four bytes
    x = R.standard_normal((64, 128)).astype(np.float32)
    g = run_kernel_test(k, [x], passes=["canonicalize"], check="CHECK: constant(\nCHECK: broadcast(\nCHECK: mul(", **EXACT)
    (c,) = [n for n in g.nodes if n.opcode == "constant"]
    assert tuple(c.outputs[0].shape) == ()


def test_constants_with_different_elements_and_integer_splats():
    from nkipy_b200.core.tensor_apis import constant

    table = np.arange(16, dtype=np.float32)
    g = run(lambda x: x + constant(table), [X], "CHECK: constant(")
    (c,) = [n for n in g.nodes if n.opcode == "constant"]
    assert tuple(c.outputs[0].shape) == (16,)
    k = trace(input_specs=[((8, 16), "i32")])(lambda i: i + constant(np.full((8, 16), 7, np.int32)))
    g = run_kernel_test(k, [R.integers(0, 9, (8, 16)).astype(np.int32)], passes=["canonicalize"], **EXACT)
    (c,) = [n for n in g.nodes if n.opcode == "constant"]
    assert tuple(c.outputs[0].shape) == () and int(np.asarray(c.attrs["value"])) == 7
