"""Writes tests/golden/reference_kats.json.

The reference is Java and cannot run where this repository is built, so the
golden vectors are the closed-form known answers its own unit tests assert and
the documented outputs of the JDK classes it relies on.  Each entry names the
reference file:line it comes from.  Run: python tests/golden/make_golden.py
"""
import json
import os

KATS = {
    "java_util_random": {
        "source": "JDK java.util.Random Javadoc algorithm (48-bit LCG); values printed by any JDK",
        "seed": 42,
        "next_int": [-1170105035, 234785527],
        "next_int_10": [0, 3, 8],
        "next_gaussian_first": 1.1419053154730547,
    },
    "mma_gemm": [
        {"source": "TestMatrixMultiplicationMMA.java:381-432 testGemmDistinctK",
         "m": 16, "n": 16, "k": 16, "a": "k+1", "b": "one", "expect": "const", "value": 136.0, "tol": 0.01},
        {"source": "TestMatrixMultiplicationMMA.java:434-484 testGemmDistinctKInB",
         "m": 16, "n": 16, "k": 16, "a": "one", "b": "k+1", "expect": "const", "value": 136.0, "tol": 0.01},
        {"source": "TestMatrixMultiplicationMMA.java:486-537 testGemmIdentityB",
         "m": 16, "n": 16, "k": 16, "a": "16i+k", "b": "identity", "expect": "16i+j", "tol": 0.01},
        {"source": "TestMatrixMultiplicationMMA.java:539-592 testGemmDistinctAB",
         "m": 16, "n": 16, "k": 16, "a": "k+1", "b": "k+1", "expect": "const", "value": 1496.0, "tol": 0.01},
        {"source": "TestMatrixMultiplicationMMA.java:983-1030 testSingleWarpManyFragments",
         "m": 32, "n": 64, "k": 16, "a": "16i+k", "b": "select_j_mod_16", "expect": "16i+j%16", "tol": 0.01},
    ],
    "mma_random_shapes": {
        "source": "TestMatrixMultiplicationMMA.java:289-329, tolerance :370",
        "shapes": [[16, 16, 16], [16, 16, 64], [32, 32, 64], [16, 64, 64], [64, 64, 64]],
        "abs_tol": 0.01,
    },
    "tolerances": {
        "sgemv_abs": {"value": 1e-4, "source": "MatrixVectorRowMajor.java:54 (8192 -> 2048)"},
        "q8_gemv_abs": {"value": 1e-1, "source": "MatrixVectorRowMajor.java:55; QuantizationTests.java:838-884"},
        "sgemm_abs": {"value": 0.1, "source": "MatrixMultiplication2D.java:195-205"},
        "sgemm_rel_cutlass": {"value": 1e-4, "source": "TestCutlass.java:105-125"},
        "hgemm_rel_example": {"value": 2e-2, "source": "MatrixMultiplicationMMA.java:59, :662-677 (denominator max(|ref|,1))"},
        "x_quant_roundtrip_abs": {"value": 0.01, "source": "QuantizationTests.java:551-590"},
    },
}

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kats.json")
    with open(out, "w") as f:
        json.dump(KATS, f, indent=1)
    print(out)
