"""Known-answer tests the reference itself holds for this path, run on the oracle."""
import numpy as np


def test_all_ones_matmul_equals_k(orc):
    # lib/gpu_benching.dart:34-37,60: A = B = ones(1024x1024) => c[0] "should be k".
    # 256 keeps the CPU suite short; the full 1024 case runs on the GPU path.
    n = 256
    ops = orc.Ops()
    Cm = ops.matmul_fwd(np.ones((n, n)), np.ones((n, n)))
    assert np.all(Cm == float(n))


def test_matvec_demo(orc):
    # lib/autogradEngine/tensor.dart:1359-1376: M=[[1,2],[3,4]], v=[10,20], loss=sum(M.v).
    ops = orc.Ops()
    M = np.array([[1.0, 2.0], [3.0, 4.0]])
    v = np.array([10.0, 20.0])
    y = ops.matvec_fwd(M, v)
    assert y.tolist() == [50.0, 110.0] and y.sum() == 160.0
    dM, dv = np.zeros_like(M), np.zeros_like(v)
    ops.matvec_bwd(M, v, np.ones(2), dM, dv)
    assert dM.tolist() == [[10.0, 20.0], [10.0, 20.0]] and dv.tolist() == [4.0, 6.0]


def test_grads_accumulate(orc):
    # every backward closure uses += (e.g. tensor.dart:918-924)
    ops = orc.Ops()
    rng = np.random.default_rng(0)
    A, B, dC = rng.normal(size=(3, 4)), rng.normal(size=(4, 5)), rng.normal(size=(3, 5))
    dA, dB = np.ones_like(A), np.ones_like(B)
    ops.matmul_bwd(A, B, dC, dA, dB)
    assert np.allclose(dA, 1 + dC @ B.T) and np.allclose(dB, 1 + A.T @ dC)


def test_tanh_overflow_guard(orc):
    # tensor.dart:582-586: exp(2x) overflow returns exactly 1.0
    ops = orc.Ops()
    y = ops.unary_fwd("tanh", np.array([400.0, -400.0, 0.0]))
    assert y.tolist() == [1.0, -1.0, 0.0]


def test_positional_table_formula(orc):
    # positionalEncodingLayer.dart:41: exponent 2*i/dModel for every column i
    pe = orc.Ops().positional_table(4, 6)
    assert pe[0].tolist() == [0.0, 1.0, 0.0, 1.0, 0.0, 1.0]
    assert abs(pe[3, 1] - np.cos(3 / 10000 ** (2 / 6))) < 1e-15
    assert abs(pe[2, 4] - np.sin(2 / 10000 ** (8 / 6))) < 1e-15


def test_omp_build_is_bit_identical(orc):
    rng = np.random.default_rng(1)
    A, B = rng.normal(size=(37, 53)), rng.normal(size=(53, 29))
    assert np.array_equal(orc.Ops(False).matmul_fwd(A, B), orc.Ops(True).matmul_fwd(A, B))
    x = rng.normal(size=(17, 33))
    assert np.array_equal(orc.Ops(False).softmax_fwd(x, 17), orc.Ops(True).softmax_fwd(x, 17))
