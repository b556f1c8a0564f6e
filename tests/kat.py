"""Builders for the closed-form GEMM cases of tests/golden/reference_kats.json."""
import numpy as np


def build(case):
    m, n, k = case["m"], case["n"], case["k"]
    i = np.arange(m)[:, None]
    kk = np.arange(k)[None, :]
    a = {"k+1": np.broadcast_to(kk + 1.0, (m, k)), "one": np.ones((m, k)), "16i+k": i * 16.0 + kk}[case["a"]]
    kr = np.arange(k)[:, None]
    j = np.arange(n)[None, :]
    b = {
        "one": np.ones((k, n)),
        "k+1": np.broadcast_to(kr + 1.0, (k, n)),
        "identity": (kr == j).astype(np.float64),
        "select_j_mod_16": (kr == (j % 16)).astype(np.float64),
    }[case["b"]]
    ii = np.arange(m)[:, None]
    exp = {
        "const": lambda: np.full((m, n), case.get("value", 0.0)),
        "16i+j": lambda: ii * 16.0 + j,
        "16i+j%16": lambda: ii * 16.0 + (j % 16),
    }[case["expect"]]()
    a16 = np.ascontiguousarray(a, np.float32).astype(np.float16).view(np.uint16)
    b16 = np.ascontiguousarray(b, np.float32).astype(np.float16).view(np.uint16)
    return a16, b16, exp.astype(np.float32)
