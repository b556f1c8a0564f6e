"""CPU oracle for the matvec / matmul path -- TEST INFRASTRUCTURE ONLY.

ctypes + numpy front-end of ``tb200_oracle.c`` (a plain-C restatement of the
TornadoVM Java kernels).  Only the test-suite, the smoke check and the CPU
baseline leg of the benchmark may import this package; the shipped library and
its host bindings never do.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libtb200_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C restatement with the committed Makefile (gcc, a second or two)."""
    src = os.path.join(_HERE, "tb200_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_jrand_next_float.restype = C.c_float
        _lib.orc_jrand_next_double.restype = C.c_double
        _lib.orc_jrand_next_gaussian.restype = C.c_double
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_dp4a_packed.argtypes = [C.c_int32, C.c_int32, C.c_int32]
        _lib.orc_dp4a_packed.restype = C.c_int32
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


class _JRandState(C.Structure):
    _fields_ = [("seed", C.c_uint64), ("have", C.c_int), ("nextg", C.c_double)]


class JavaRandom:
    """java.util.Random with the JDK's documented algorithm."""

    def __init__(self, seed: int):
        self._s = _JRandState()
        lib().orc_jrand_init(C.byref(self._s), C.c_int64(seed))

    def next_int(self, bound: int | None = None) -> int:
        if bound is None:
            return lib().orc_jrand_next_int(C.byref(self._s))
        return lib().orc_jrand_next_int_bound(C.byref(self._s), C.c_int32(bound))

    def next_float(self) -> float:
        return lib().orc_jrand_next_float(C.byref(self._s))

    def next_double(self) -> float:
        return lib().orc_jrand_next_double(C.byref(self._s))

    def next_gaussian(self) -> float:
        return lib().orc_jrand_next_gaussian(C.byref(self._s))

    # bulk fillers ---------------------------------------------------------
    def uniform_f32(self, n: int, lo: float, hi: float) -> np.ndarray:
        out = np.empty(n, np.float32)
        lib().orc_fill_uniform_f32(C.byref(self._s), _p(out), C.c_int64(n), C.c_float(lo), C.c_float(hi))
        return out

    def uniform_f32_interleaved(self, n: int):
        a = np.empty(n, np.float32)
        b = np.empty(n, np.float32)
        lib().orc_fill_uniform_f32_interleaved(C.byref(self._s), _p(a), _p(b), C.c_int64(n))
        return a, b

    def gaussian_f32(self, n: int, mul: float = 1.0) -> np.ndarray:
        out = np.empty(n, np.float32)
        lib().orc_fill_gaussian_f32(C.byref(self._s), _p(out), C.c_int64(n), C.c_float(mul))
        return out

    def gaussian_f16(self, n: int, mul: float = 1.0) -> np.ndarray:
        out = np.empty(n, np.uint16)
        lib().orc_fill_gaussian_f16(C.byref(self._s), _p(out), C.c_int64(n), C.c_float(mul))
        return out

    def ints(self, n: int, bound: int) -> np.ndarray:
        out = np.empty(n, np.int32)
        lib().orc_fill_int_bound(C.byref(self._s), _p(out), C.c_int64(n), C.c_int32(bound))
        return out


# -- conversions ------------------------------------------------------------
def f32_to_f16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16_n(_p(x), _p(out), C.c_int64(x.size))
    return out


def f16_to_f32(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().orc_f16_to_f32_n(_p(h), _p(out), C.c_int64(h.size))
    return out


# -- FP32 GEMV ---------------------------------------------------------------
def sgemv_seq(w, x, n, d, threads: bool = False):
    out = np.empty(d, np.float32)
    (lib().orc_sgemv_seq_mt if threads else lib().orc_sgemv_seq)(_p(w), _p(x), _p(out), n, d)
    return out


def sgemv_workgroup(w, x, n, d, L=32):
    out = np.empty(d, np.float32)
    lib().orc_sgemv_workgroup(_p(w), _p(x), _p(out), n, d, L)
    return out


def sgemv_f64(w, x, n, d):
    out = np.empty(d, np.float64)
    lib().orc_sgemv_f64(_p(w), _p(x), _p(out), n, d)
    return out


# -- Q8_0 ---------------------------------------------------------------------
def q8_quantize(w, rows, cols):
    q = np.empty(rows * cols, np.int8)
    s = np.empty(rows * cols // 32, np.uint16)
    blocks = np.empty(rows * (cols // 32) * 34, np.uint8)
    lib().orc_q8_quantize(_p(w), _p(q), _p(s), _p(blocks), rows, cols)
    return q, s, blocks


def q8_pack_blocks(q, scales):
    nb = scales.size
    blocks = np.empty(nb * 34, np.uint8)
    lib().orc_q8_pack_blocks(_p(q), _p(scales), _p(blocks), C.c_int64(nb))
    return blocks


def q8_gemv_ref(q, scales, x, n, d, L=32):
    out = np.empty(d, np.float32)
    lib().orc_q8_gemv_ref(_p(q), _p(scales), _p(x), _p(out), n, d, L)
    return out


def q8_gemv_seq(q, scales, x, n, d, threads: bool = False):
    out = np.empty(d, np.float32)
    (lib().orc_q8_gemv_seq_mt if threads else lib().orc_q8_gemv_seq)(_p(q), _p(scales), _p(x), _p(out), n, d)
    return out


def q8_gemv_f64(q, scales, x, n, d):
    out = np.empty(d, np.float64)
    lib().orc_q8_gemv_f64(_p(q), _p(scales), _p(x), _p(out), n, d)
    return out


# -- integer dots ---------------------------------------------------------------
def dp4a_n(a, b):
    out = np.empty(a.size // 4, np.int32)
    lib().orc_dp4a_n(_p(a), _p(b), _p(out), C.c_int64(a.size // 4))
    return out


def dp4a_packed(a: int, b: int, c: int) -> int:
    return lib().orc_dp4a_packed(a, b, c)


def quantize_x_tensor(x):
    xq = np.empty(x.size, np.int8)
    s = C.c_float()
    lib().orc_quantize_x_tensor(_p(x), _p(xq), C.byref(s), x.size)
    return xq, np.float32(s.value)


def quantize_x_block(x):
    xq = np.empty(x.size, np.int8)
    xs = np.empty(x.size // 32, np.float32)
    lib().orc_quantize_x_block(_p(x), _p(xq), _p(xs), x.size)
    return xq, xs


def q8_blockdots_i32(q, xq, n, d):
    out = np.empty(d * (n // 32), np.int32)
    lib().orc_q8_blockdots_i32(_p(q), _p(xq), _p(out), n, d)
    return out


def q4_blockdots_i32(blocks, xq, n, d):
    out = np.empty(d * (n // 32), np.int32)
    lib().orc_q4_blockdots_i32(_p(blocks), _p(xq), _p(out), n, d)
    return out


def blockdots_combine_f64(dots, wscales, xs, bpr, d):
    out = np.empty(d, np.float64)
    lib().orc_blockdots_combine_f64(_p(dots), _p(wscales), _p(xs), _p(out), bpr, d)
    return out


def block_scales(blocks, nblocks, block_bytes):
    s = np.empty(nblocks, np.uint16)
    lib().orc_block_scales(_p(blocks), _p(s), C.c_int64(nblocks), block_bytes)
    return s


# -- Q4_0 ---------------------------------------------------------------------
def q4_pack_blocks(nibbles, scales):
    nb = scales.size
    blocks = np.empty(nb * 18, np.uint8)
    nibbles = np.ascontiguousarray(nibbles, np.uint8)
    lib().orc_q4_pack_blocks(_p(nibbles), _p(scales), _p(blocks), C.c_int64(nb))
    return blocks


def q4_gemv_seq(blocks, x, n, d, threads: bool = False):
    out = np.empty(d, np.float32)
    (lib().orc_q4_gemv_seq_mt if threads else lib().orc_q4_gemv_seq)(_p(blocks), _p(x), _p(out), n, d)
    return out


def q4_gemv_f64(blocks, x, n, d):
    out = np.empty(d, np.float64)
    lib().orc_q4_gemv_f64(_p(blocks), _p(x), _p(out), n, d)
    return out


# -- GEMM ---------------------------------------------------------------------
def sgemm_seq(a, b, m, n, k, row0=0, row1=None, threads: bool = False):
    row1 = m if row1 is None else row1
    c = np.zeros(m * n, np.float32)
    (lib().orc_sgemm_seq_mt if threads else lib().orc_sgemm_seq)(_p(a), _p(b), _p(c), m, n, k, row0, row1)
    return c.reshape(m, n)[row0:row1]


def sgemm_f64(a, b, m, n, k, row0=0, row1=None):
    row1 = m if row1 is None else row1
    c = np.empty((row1 - row0) * n, np.float64)
    lib().orc_sgemm_f64(_p(a), _p(b), _p(c), m, n, k, row0, row1)
    return c.reshape(row1 - row0, n)


def hgemm_ref(a, b, m, n, k, row0=0, row1=None):
    row1 = m if row1 is None else row1
    c = np.empty((row1 - row0) * n, np.float32)
    lib().orc_hgemm_ref(_p(a), _p(b), _p(c), m, n, k, row0, row1)
    return c.reshape(row1 - row0, n)


def hgemm_f64(a, b, m, n, k, row0=0, row1=None):
    row1 = m if row1 is None else row1
    c = np.empty((row1 - row0) * n, np.float64)
    lib().orc_hgemm_f64(_p(a), _p(b), _p(c), m, n, k, row0, row1)
    return c.reshape(row1 - row0, n)


def num_threads() -> int:
    return lib().orc_num_threads()


def rel_l2(got, ref) -> float:
    got = np.asarray(got, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(got - ref) / (den if den > 0 else 1.0))


# -- seeded workloads (java.util.Random(seed)-compatible streams) ----------------
def make_sgemv(rows, cols, seed=42, lo=-1.0, hi=1.0):
    """v first, then m, as MatrixVectorRowMajor.java:907-908 fills input then weights."""
    r = JavaRandom(seed)
    v = r.uniform_f32(cols, lo, hi)
    m = r.uniform_f32(rows * cols, lo, hi)
    return m, v


def make_sgemm(m, n, k, seed=42):
    assert m == n == k, "interleaved fill follows the square benchmark"
    r = JavaRandom(seed)
    return r.uniform_f32_interleaved(m * k)


def make_hgemm(m, n, k, seed=42):
    r = JavaRandom(seed)
    mul = 1.0 / np.sqrt(np.float64(k))
    a = r.gaussian_f16(m * k, mul)
    b = r.gaussian_f16(k * n, mul)
    return a, b


def make_q8(rows, cols, batch=1, seed=42):
    """int8 U[-127,127], fp16 scale |N(0,1)|*0.02, x ~ N(0,1)."""
    r = JavaRandom(seed)
    q = (r.ints(rows * cols, 255) - 127).astype(np.int8)
    g = np.abs(r.gaussian_f32(rows * cols // 32, 0.02))
    scales = f32_to_f16(g)
    x = r.gaussian_f32(batch * cols)
    return q, scales, x


def make_q4(rows, cols, batch=1, seed=42):
    """nibbles U[0,15], fp16 scale |N(0,1)|*0.02, x ~ N(0,1); returns 18-byte blocks."""
    r = JavaRandom(seed)
    nib = r.ints(rows * cols, 16).astype(np.uint8)
    g = np.abs(r.gaussian_f32(rows * cols // 32, 0.02))
    scales = f32_to_f16(g)
    x = r.gaussian_f32(batch * cols)
    return q4_pack_blocks(nib, scales), scales, x


# -- fused GEMM epilogues (restated from the reference's own test oracles) ------------
def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns -> float32 (BFloat16Array keeps the upper 16 bits of a float)."""
    return (np.asarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round to nearest even."""
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def activation_ref(x: np.ndarray, act: str) -> np.ndarray:
    """The activations as TestCutlass.java checks them (tornado-unittests/.../cutlass/TestCutlass.java:302-545):
    relu = max(0, x); gelu = 0.5 x (1 + erf(x / sqrt 2)); silu = x / (1 + exp(-x)); sigmoid; tanh;
    hardswish = x * min(max(x + 3, 0), 6) / 6.  Evaluated in double."""
    from math import erf
    x = np.asarray(x, np.float64)
    if act == "none":
        return x
    if act == "relu":
        return np.maximum(x, 0.0)
    if act == "gelu":
        return 0.5 * x * (1.0 + np.vectorize(erf)(x / np.sqrt(2.0)))
    if act == "silu":
        return x / (1.0 + np.exp(-x))
    if act == "sigmoid":
        return 1.0 / (1.0 + np.exp(-x))
    if act == "tanh":
        return np.tanh(x)
    if act == "hardswish":
        return x * np.minimum(np.maximum(x + 3.0, 0.0), 6.0) / 6.0
    raise ValueError(act)


def gemm_epilogue_ref(prod, act="none", alpha=1.0, beta=0.0, c=None, bias=None):
    """act(alpha * prod + beta * C + bias) in double on an fp32-accumulated product [m][n]
    (hgemmJava + the per-test expression of TestCutlass.java:302-545; alpha / beta as
    Cutlass.cutlassHgemm, Cutlass.java:83-100)."""
    x = alpha * np.asarray(prod, np.float64)
    if beta != 0.0:
        x = x + beta * np.asarray(c, np.float64)
    if bias is not None:
        x = x + np.asarray(bias, np.float64)[None, :]
    return activation_ref(x, act)


# -- fp8 (OCP E4M3 / E5M2), restated from tornado-api/.../types/FP8.java:44-80 and the OCP 8-bit float specification ----
def fp8_decode_table(fmt: str) -> np.ndarray:
    """float32 value of every byte.  E4M3: bias 7, subnormals m * 2^-9, no infinity, S.1111.111 = NaN, max 448
    (FP8.java:41, :52-76).  E5M2: bias 15, IEEE-like (the upper byte of an fp16), max 57344 (FP8.java:43)."""
    out = np.empty(256, np.float32)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        if fmt == "e4m3":
            e, m = (b >> 3) & 15, b & 7
            if e == 0:
                v = m * 2.0 ** -9
            elif e == 15 and m == 7:
                v = float("nan")
            else:
                v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        elif fmt == "e5m2":
            e, m = (b >> 2) & 31, b & 3
            if e == 0:
                v = m * 2.0 ** -16
            elif e == 31:
                v = float("inf") if m == 0 else float("nan")
            else:
                v = (1.0 + m / 4.0) * 2.0 ** (e - 15)
        else:
            raise ValueError(fmt)
        out[b] = sign * v
    return out


def fp8_encode_exact(values: np.ndarray, fmt: str) -> np.ndarray:
    """Bytes of values that the format represents exactly (the reference's test inputs, multiples of 0.25 in
    [-2, 2): TestMatrixMultiplicationMMAFP8.java:433-439); raises on any other value."""
    table = fp8_decode_table(fmt)
    lookup = {}
    for b in range(256):
        v = float(table[b])
        if v == v and abs(v) != float("inf") and v not in lookup:  # +0 before -0, finite only
            lookup[v] = b
    return np.array([lookup[float(v)] for v in np.asarray(values, np.float32).ravel()], np.uint8)


def fp8_gemm_ref(a: np.ndarray, b: np.ndarray, m: int, n: int, k: int, fmt: str) -> np.ndarray:
    """gemmReferenceE4M3 / gemmReferenceE5M2 (TestMatrixMultiplicationMMAFP8.java:226-248): decode, multiply,
    accumulate.  Accumulated in float64 here; for the reference's exactly representable inputs every partial sum is
    exact in fp32 as well, so the order and the width of the accumulator do not matter (:420-423)."""
    t = fp8_decode_table(fmt).astype(np.float64)
    return (t[np.asarray(a, np.uint8).reshape(m, k)] @ t[np.asarray(b, np.uint8).reshape(k, n)])
