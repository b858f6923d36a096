"""Python operator protocol of traced tensors: forward, reflected and in-place forms of every arithmetic operator,
NumPy broadcasting of their operands, matmul with batch broadcasting, shape errors raised while tracing, and the
call forms of reshape / transpose / astype.  Each kernel runs in direct mode (NumPy) and as an interpreted trace.
Operator list and shape families follow the reference's tests/unit/test_tensor_api_native_ops.py and test_tensor.py."""
import numpy as np
import pytest

from utils import check, trace_kernel

pytestmark = pytest.mark.filterwarnings("ignore::RuntimeWarning")

R = np.random.default_rng(11)


def pos(*s):
    return (R.random(s) + 0.5).astype(np.float32)          # positive: safe for /, //, %, **


BINARY = {
    "add": lambda a, b: a + b, "radd": lambda a, b: b + a,
    "sub": lambda a, b: a - b, "rsub": lambda a, b: b - a,
    "mul": lambda a, b: a * b, "rmul": lambda a, b: b * a,
    "truediv": lambda a, b: a / b, "rtruediv": lambda a, b: b / a,
    "floordiv": lambda a, b: a // b, "rfloordiv": lambda a, b: b // a,
    "mod": lambda a, b: a % b, "rmod": lambda a, b: b % a,
    "pow": lambda a, b: a ** b, "rpow": lambda a, b: b ** a,
}

SCALAR_LEFT = {
    "radd": lambda a: 2.0 + a, "rsub": lambda a: 2.0 - a, "rmul": lambda a: 2.0 * a, "rtruediv": lambda a: 2.0 / a,
    "rfloordiv": lambda a: 2.0 // a, "rmod": lambda a: 2.0 % a, "rpow": lambda a: 2.0 ** a,
}


def _inplace(op):
    def k(a, b):
        c = a * 1.0                     # a fresh value: parameters are left alone here
        c = op(c, b)
        return c
    return k


def _iadd(c, b): c += b; return c
def _isub(c, b): c -= b; return c
def _imul(c, b): c *= b; return c
def _itruediv(c, b): c /= b; return c
def _ifloordiv(c, b): c //= b; return c
def _imod(c, b): c %= b; return c
def _ipow(c, b): c **= b; return c


INPLACE = {"iadd": _iadd, "isub": _isub, "imul": _imul, "itruediv": _itruediv, "ifloordiv": _ifloordiv, "imod": _imod,
           "ipow": _ipow}

BROADCAST = [((16, 16), (16, 16)), ((16, 1), (16, 16)), ((1, 16), (16, 16)), ((16,), (16, 16)), ((1,), (16, 16)),
             ((2, 1, 16), (1, 8, 16)), ((), (16, 16))]


@pytest.mark.parametrize("name", sorted(BINARY))
def test_binary_operator(name):
    check(BINARY[name], pos(8, 16), pos(8, 16), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("name", sorted(SCALAR_LEFT))
def test_python_scalar_on_the_left(name):
    check(SCALAR_LEFT[name], pos(8, 16))


@pytest.mark.parametrize("name", sorted(BINARY))
def test_numpy_array_on_the_left_is_captured_as_a_constant(name):
    c = pos(8, 16)
    check(lambda a: BINARY[name](c, a), pos(8, 16))
    check(lambda a: BINARY[name](a, c), pos(8, 16))


@pytest.mark.parametrize("shape_a,shape_b", BROADCAST)
@pytest.mark.parametrize("name", ["add", "rsub", "mul", "rtruediv", "pow", "mod"])
def test_operands_broadcast(shape_a, shape_b, name):
    a = pos(*shape_a) if shape_a else np.float32(1.5)
    if shape_a == ():
        check(lambda b: BINARY[name](np.float32(1.5), b), pos(*shape_b))
    else:
        check(BINARY[name], a, pos(*shape_b))


@pytest.mark.parametrize("name", sorted(INPLACE))
def test_in_place_operator_on_a_value(name):
    check(_inplace(INPLACE[name]), pos(8, 16), pos(8, 16))


@pytest.mark.parametrize("name", sorted(INPLACE))
def test_in_place_operator_with_broadcast_right_side(name):
    check(_inplace(INPLACE[name]), pos(8, 16), pos(16))
    check(lambda a: _inplace(INPLACE[name])(a, 1.5), pos(8, 16))


def test_in_place_matmul_rebinds():
    def k(a, b):
        c = a * 1.0
        c @= b
        return c
    check(k, pos(8, 8), pos(8, 8))


def test_unary_operators():
    a = R.standard_normal((8, 16)).astype(np.float32)
    check(lambda x: +x, a)
    check(lambda x: -x, a)
    check(lambda x: abs(x), a)
    check(lambda x: -(-x) + (+x), a)


@pytest.mark.parametrize("shape_a,shape_b", [
    ((8, 16), (16, 12)), ((1, 2, 8, 16), (16, 12)), ((8, 16), (1, 2, 16, 12)), ((1, 2, 8, 16), (1, 2, 16, 12)),
    ((1, 8, 16), (16, 12)), ((8, 16), (1, 16, 12)), ((5, 8, 16), (1, 16, 12)), ((3, 1, 8, 16), (1, 4, 16, 12)),
    ((16,), (16, 12)), ((8, 16), (16,)), ((16,), (16,)),
])
def test_matmul_shapes_and_batch_broadcast(shape_a, shape_b):
    a, b = pos(*shape_a), pos(*shape_b)
    check(lambda x, y: x @ y, a, b, rtol=1e-4, atol=1e-4)
    check(lambda x, y: np.matmul(x, y), a, b, rtol=1e-4, atol=1e-4)


def test_reflected_matmul_with_a_constant():
    c = pos(12, 8)
    check(lambda x: c @ x, pos(8, 16))


@pytest.mark.parametrize("shape_a,shape_b", [((8, 16), (8, 16)), ((16, 8), (16, 8)), ((1, 1), (8, 8)), ((2, 8, 16), (3, 16, 8)),
                                             ((16,), (8,))])
def test_matmul_shape_errors_are_raised_while_tracing(shape_a, shape_b):
    with pytest.raises((ValueError, TypeError)):
        trace_kernel(lambda x, y: x @ y, pos(*shape_a), pos(*shape_b))


@pytest.mark.parametrize("shape_a,shape_b", [((8, 16), (8, 15)), ((3, 8), (4, 8)), ((2, 3, 4), (2, 4, 3))])
def test_broadcast_errors_are_raised_while_tracing(shape_a, shape_b):
    with pytest.raises((ValueError, TypeError)):
        trace_kernel(lambda x, y: x + y, pos(*shape_a), pos(*shape_b))


@pytest.mark.parametrize("shape", [(16, 64), (1024,), (4, 256), (2, 8, 64)])
def test_reshape_call_forms(shape):
    a = pos(*shape)
    check(lambda x: x.reshape((32, 32)), a)
    check(lambda x: x.reshape(32, 32), a)
    check(lambda x: x.reshape(-1, 64), a)
    check(lambda x: x.reshape(-1), a)
    check(lambda x: np.reshape(x, (8, -1, 4)), a)


def test_reshape_to_a_different_size_is_an_error():
    with pytest.raises((ValueError, TypeError)):
        trace_kernel(lambda x: x.reshape(7, 7), pos(8, 8))
    with pytest.raises((ValueError, TypeError)):
        trace_kernel(lambda x: x.reshape(-1, -1), pos(8, 8))


@pytest.mark.parametrize("shape", [(16, 16), (8, 32), (2, 8, 16)])
def test_transpose_call_forms(shape):
    a = pos(*shape)
    check(lambda x: x.transpose(), a)
    check(lambda x: x.T, a)
    perm = tuple(reversed(range(len(shape))))
    check(lambda x: x.transpose(perm), a)
    check(lambda x: x.transpose(*perm), a)
    check(lambda x: np.transpose(x, perm), a)


def test_transpose_of_a_batched_tensor_by_axes():
    a = pos(2, 8, 16)
    for perm in [(0, 2, 1), (1, 0, 2), (2, 0, 1), (1, 2, 0)]:
        check(lambda x: x.transpose(perm), a)
    with pytest.raises((ValueError, TypeError, IndexError)):
        trace_kernel(lambda x: x.transpose(0, 0, 1), a)


@pytest.mark.parametrize("src", [np.float32, np.float16, np.int32, np.int8, np.uint8])
@pytest.mark.parametrize("dst", [np.float32, np.float16, np.int32])
def test_astype(src, dst):
    a = (R.random((8, 16)) * 20).astype(src)
    check(lambda x: x.astype(dst), a)


@pytest.mark.parametrize("shape", [(4,), (4, 6), (2, 3, 4), (2, 1, 3, 4)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.int32])
def test_tensor_attributes_while_tracing(shape, dtype):
    seen = {}

    def k(x):
        seen.update(shape=tuple(x.shape), dtype=np.dtype(x.dtype), ndim=x.ndim, size=x.size, t_shape=tuple(x.T.shape),
                    length=len(x))
        return x

    a = np.ones(shape, dtype)
    trace_kernel(k, a)
    assert seen == dict(shape=shape, dtype=np.dtype(dtype), ndim=len(shape), size=a.size, t_shape=a.T.shape,
                        length=shape[0])


def test_operators_compose():
    def k(a, b, c):
        d = (a @ b + c) * 2.0 - 1.0
        d /= (abs(c) + 1.0)
        return (-d) ** 2 % 3.0 // 0.5

    check(k, pos(8, 16), pos(16, 8), pos(8))
