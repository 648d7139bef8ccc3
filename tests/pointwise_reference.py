"""The reference's own test oracle for POINTWISE, restated in double precision.

test/Compiler/FoundationalMathOpsTest.cpp:440-545 checks every mode of the schema, on one graph with A = [2, 3],
B = [3] and T = [2, 1], against closed-form values in f64 with the tolerance 3e-4 + 3e-4 * |expected|
(NaN must be NaN, an infinity must be that infinity). The CPU oracle and the CUDA kernels are pinned to the same
values on the same inputs, and on wider seeded inputs through the same formulas.
"""
import math

import numpy as np

RELU_LOWER, RELU_UPPER, RELU_SLOPE = 0.25, 1.0, 0.2   # FoundationalMathOpsTest.cpp:26-31
SWISH_BETA, ELU_ALPHA, SOFTPLUS_BETA = 0.5, 2.0, 2.0
A = np.array([0.0, 0.25, 0.5, 0.75, 1.0, 1.5], np.float32)   # FoundationalMathOpsTest.cpp:617-619
B = np.array([0.0, 0.25, -2.0], np.float32)
T = np.array([0.0, 9.0], np.float32)


def _sigmoid(v):
    return 1.0 / (1.0 + math.exp(-v))


def _divide(x, y):
    if y != 0.0:
        return x / y
    if x == 0.0 or math.isnan(x):
        return math.nan
    return math.copysign(math.inf, x) * math.copysign(1.0, y)


def _guard(function, *args):
    """C's libm answers where Python raises: domain errors give NaN, poles and overflow an infinity."""
    try:
        return function(*args)
    except ValueError:
        if function is math.log and args[0] == 0.0:
            return -math.inf
        if function is math.fmod:
            return math.nan
        if function is math.pow and args[0] == 0.0 and args[1] < 0:   # a pole: signed for an odd integer exponent
            odd = float(args[1]).is_integer() and int(args[1]) % 2 == 1
            return math.copysign(math.inf, args[0]) if odd else math.inf
        return math.nan
    except OverflowError:
        return math.inf
    except ZeroDivisionError:
        return math.inf


def value(mode, a, b, c, column):
    """One element: a, b, c are IN_0, IN_1, IN_2 as doubles; `column` is the output index along axis 1."""
    if mode == "ADD": return a + b
    if mode == "MUL": return a * b
    if mode == "SQRT": return math.sqrt(a) if a >= 0 else math.nan
    if mode == "MAX": return max(a, b)
    if mode == "MIN": return min(a, b)
    if mode == "RELU_FWD":
        if a < RELU_LOWER:
            return RELU_LOWER + RELU_SLOPE * (a - RELU_LOWER)
        return RELU_UPPER if a > RELU_UPPER else a
    if mode == "TANH_FWD": return math.tanh(a)
    if mode == "SIGMOID_FWD": return _sigmoid(a)
    if mode == "ELU_FWD": return a if a >= 0.0 else ELU_ALPHA * (math.exp(a) - 1.0)
    if mode == "GELU_FWD": return 0.5 * a * (1.0 + math.erf(a / math.sqrt(2.0)))
    if mode == "SOFTPLUS_FWD": return math.log(1.0 + math.exp(SOFTPLUS_BETA * a)) / SOFTPLUS_BETA
    if mode == "SWISH_FWD": return a * _sigmoid(SWISH_BETA * a)
    if mode == "RELU_BWD": return a * (RELU_SLOPE if b < RELU_LOWER else (0.0 if b > RELU_UPPER else 1.0))
    if mode == "TANH_BWD":
        t = math.tanh(b)
        return a * (1.0 - t * t)
    if mode == "SIGMOID_BWD":
        s = _sigmoid(b)
        return a * s * (1.0 - s)
    if mode == "ELU_BWD": return a * (1.0 if b >= 0.0 else ELU_ALPHA * math.exp(b))
    if mode == "GELU_BWD":
        cdf = 0.5 * (1.0 + math.erf(b / math.sqrt(2.0)))
        density = math.exp(-0.5 * b * b) / math.sqrt(2.0 * math.pi)
        return a * (cdf + b * density)
    if mode == "SOFTPLUS_BWD": return a * _sigmoid(SOFTPLUS_BETA * b)
    if mode == "SWISH_BWD":
        s = _sigmoid(SWISH_BETA * b)
        return a * (s + SWISH_BETA * b * s * (1.0 - s))
    if mode == "ERF": return math.erf(a)
    if mode == "IDENTITY": return a
    if mode == "GELU_APPROX_TANH_FWD":
        inner = math.sqrt(2.0 / math.pi) * (a + 0.044715 * a * a * a)
        return 0.5 * a * (1.0 + math.tanh(inner))
    if mode == "GELU_APPROX_TANH_BWD":
        t = math.tanh(math.sqrt(2.0 / math.pi) * (b + 0.044715 * b * b * b))
        return a * (0.5 * (1.0 + t) + 0.5 * b * (1.0 - t * t) * math.sqrt(2.0 / math.pi) * (1.0 + 3.0 * 0.044715 * b * b))
    if mode == "GEN_INDEX": return float(column)
    if mode == "BINARY_SELECT": return b if c != 0.0 else a
    if mode == "EXP": return _guard(math.exp, a)
    if mode == "LOG": return _guard(math.log, a)
    if mode == "NEG": return -a
    if mode == "MOD": return _guard(math.fmod, a, b)
    if mode == "POW": return _guard(math.pow, a, b)
    if mode == "ABS": return abs(a)
    if mode == "CEIL": return float(math.ceil(a))
    if mode == "COS": return math.cos(a)
    if mode == "FLOOR": return float(math.floor(a))
    if mode == "RSQRT": return _divide(1.0, math.sqrt(a)) if a >= 0 else math.nan
    if mode == "SIN": return math.sin(a)
    if mode == "LOGICAL_NOT": return 1.0 if a == 0.0 else 0.0
    if mode == "TAN": return math.tan(a)
    if mode == "SUB": return a - b
    if mode == "ADD_SQUARE": return a + b * b
    if mode == "DIV": return _divide(a, b)
    if mode == "CMP_EQ": return 1.0 if a == b else 0.0
    if mode == "CMP_NEQ": return 1.0 if a != b else 0.0
    if mode == "CMP_GT": return 1.0 if a > b else 0.0
    if mode == "CMP_GE": return 1.0 if a >= b else 0.0
    if mode == "CMP_LT": return 1.0 if a < b else 0.0
    if mode == "CMP_LE": return 1.0 if a <= b else 0.0
    if mode == "LOGICAL_AND": return 1.0 if a != 0.0 and b != 0.0 else 0.0
    if mode == "LOGICAL_OR": return 1.0 if a != 0.0 or b != 0.0 else 0.0
    if mode == "RECIPROCAL": return _divide(1.0, a)
    raise KeyError(mode)


def expected(mode, a, b, t):
    """The [rows, columns] answers for A [rows, columns], B [columns], T [rows, 1] (f32 values, f64 arithmetic)."""
    rows, columns = a.shape
    out = np.empty((rows, columns), np.float64)
    for r in range(rows):
        for c in range(columns):
            out[r, c] = value(mode, float(a[r, c]), float(b[c]), float(t[r]), c)
    return out


def assert_close(mode, actual, reference, absolute=3.0e-4, relative=3.0e-4):
    """FoundationalMathOpsTest.cpp:547-556."""
    actual = np.asarray(actual, np.float64).reshape(-1)
    reference = np.asarray(reference, np.float64).reshape(-1)
    for index, (got, want) in enumerate(zip(actual, reference)):
        if math.isnan(want):
            assert math.isnan(got), (mode, index, got, want)
        elif math.isinf(want):
            assert got == want, (mode, index, got, want)
        else:
            assert abs(got - want) <= absolute + relative * abs(want), (mode, index, got, want)
