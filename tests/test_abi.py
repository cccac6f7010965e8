"""The shared library loads on a machine without a GPU and exports every symbol fml.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib_path():
    from flutter_ml_b200 import _build
    return _build.build()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fml.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(?:int32_t|void|const char\*)\s+(\w+)\s*\(", text)
    return sorted(set(names))


def test_header_symbols_are_exported(lib_path):
    lib = ctypes.CDLL(lib_path)
    names = declared_symbols()
    assert "fml_gemm" in names and "multiplyMatrices" in names and "benchtest" in names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_python_prototypes_cover_the_header(lib_path):
    from flutter_ml_b200 import _lib
    assert set(declared_symbols()) == set(_lib.PROTOTYPES)


def test_init_fails_loudly_without_a_device(lib_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from flutter_ml_b200 import _lib
    with pytest.raises(_lib.FmlError, match="no CUDA device"):
        _lib.Context()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "flutter_ml_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(".py"):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle", src, flags=re.M) and "oracle." not in src, f


def test_tape_kind_knows_the_reference_op_names():
    """fml_tape_kind is host-only: every opName string of the reference's hot path
    (lib/autogradEngine/tensor.dart:410-1232, softmax.dart:113, layerNormalization.dart:200,
    embeddingLayer.dart:65) maps to a kind, vector and matrix spellings to the same one."""
    from flutter_ml_b200 import _lib
    lib = _lib.load()
    names = ["matMul", "matVecMul", "addMatrixAndVector", "add_matrix", "add_vector", "relu_matrix", "relu_vector",
             "sigmoid_vector", "sigmoid_matrix", "tanh_vector", "tanh_matrix", "multiply_vector", "multiply_matrix",
             "concat_vector", "concat_matrix_col", "scale_matrix", "transpose", "softmax_matrix", "layer_norm",
             "embedding_lookup", "mse_vector", "mse_matrix", "sum_vector", "sum_matrix", "leaky_relu", "elu", "swish",
             "gelu", "softmax_xent", "dense", "conv2d", "addScalarToMatrix", "attention"]
    kinds = {n: lib.fml_tape_kind(n.encode()) for n in names}
    assert all(k > 0 for k in kinds.values()), kinds
    assert kinds["relu_matrix"] == kinds["relu_vector"] and kinds["add_matrix"] == kinds["add_vector"]
    assert kinds["matMul"] == 1 and kinds["dense"] == 23
    assert lib.fml_tape_kind(b"max_pool_2d") == 0 and lib.fml_tape_kind(None) == 0
    from flutter_ml_b200 import tape
    assert tape.KIND["matMul"] == kinds["matMul"] and tape.KIND["layer_norm"] == kinds["layer_norm"]


def test_stage_rows_gathers_and_narrows_on_host_threads():
    """fml_stage_rows is host-only work (no context state, no device): rows picked by index or by range, float64 and
    int64 sources narrowed to 4-byte elements, any thread count gives the same bytes."""
    import ctypes as C
    import numpy as np
    from flutter_ml_b200 import _lib
    L = _lib.load()
    rng = np.random.default_rng(0)
    n, row = 5000, 257
    for kind, src in ((0, rng.standard_normal((n, row)).astype(np.float32)), (1, rng.standard_normal((n, row))),
                      (2, rng.integers(-9, 9, (n, row)).astype(np.int32)), (3, rng.integers(-9, 9, (n, row)))):
        out_dt = np.float32 if kind < 2 else np.int32
        idx = rng.permutation(n)[:3000].astype(np.int64)
        for threads in (1, 4, 0):
            dst = np.zeros((3000, row), out_dt)
            assert L.fml_stage_rows(None, dst.ctypes.data, src.ctypes.data, kind, row, idx.ctypes.data, 0, 3000, threads) == 0
            assert np.array_equal(dst, src[idx].astype(out_dt))
            dst = np.zeros((1234, row), out_dt)
            assert L.fml_stage_rows(None, dst.ctypes.data, src.ctypes.data, kind, row, None, 77, 1234, threads) == 0
            assert np.array_equal(dst, src[77:77 + 1234].astype(out_dt))
    # background form: two gathers outstanding at once, complete after fml_stage_wait
    a64, i64_ = rng.standard_normal((n, row)), rng.integers(0, 99, (n,))
    idx = rng.permutation(n).astype(np.int64)
    d1, d2 = np.zeros((n, row), np.float32), np.zeros((n,), np.int32)
    assert L.fml_stage_rows_async(None, d1.ctypes.data, a64.ctypes.data, 1, row, idx.ctypes.data, 0, n, 3) == 0
    assert L.fml_stage_rows_async(None, d2.ctypes.data, i64_.ctypes.data, 3, 1, idx.ctypes.data, 0, n, 3) == 0
    assert L.fml_stage_wait(None) == 0
    assert np.array_equal(d1, a64[idx].astype(np.float32)) and np.array_equal(d2, i64_[idx].astype(np.int32))
    assert L.fml_stage_wait(None) == 0                                         # nothing outstanding: returns at once
    assert L.fml_stage_rows(None, None, None, 0, 1, None, 0, 1, 0) != 0      # rejected, not a crash
    assert L.fml_stage_rows(None, dst.ctypes.data, src.ctypes.data, 9, row, None, 0, 1, 0) != 0


def test_per_device_once_bookkeeping():
    """One-time kernel set-up (the shared-memory opt-in of cudaFuncSetAttribute) is per DEVICE: the guard around it
    must run its body once for every device ordinal, not once per process.  Host-only self test of that guard."""
    import ctypes as C
    from flutter_ml_b200 import _lib
    L = _lib.load()
    runs = C.c_int32(0)
    for device in (0, 1, 5, 63):
        for _ in range(3):
            assert L.fml_selftest_per_device_once(device, C.byref(runs)) == 0
            assert runs.value == 1, (device, runs.value)          # once per ordinal, however often it is asked
    before = runs.value
    assert L.fml_selftest_per_device_once(64, C.byref(runs)) == 0 and L.fml_selftest_per_device_once(64, C.byref(runs)) == 0
    assert runs.value >= 2                                        # no slot for this ordinal: the body runs every time
    assert L.fml_selftest_per_device_once(0, None) == -1


def test_host_mirror_defaults_match_the_reference_constructors():
    """Default hyper-parameters and argument order of the host mirror against the reference's constructors (values read
    from lib/optimizers/{adam.dart:17-19, adamw.dart:41-44, amsgrad.dart:32-34, rmsprop.dart:28-29, adagrad.dart:26,
    nag.dart:30, sgdmomentum.dart:28} and lib/transformer/multiHeadAttentionLayer.dart:33): a ported call with default
    arguments must mean the same thing."""
    import inspect
    from flutter_ml_b200 import layers, optimizers as O
    d = lambda cls: {k: v.default for k, v in inspect.signature(cls.__init__).parameters.items() if v.default is not inspect.Parameter.empty}  # noqa: E731
    assert (d(O.Adam)["beta1"], d(O.Adam)["beta2"], d(O.Adam)["epsilon"]) == (0.9, 0.999, 1e-8)
    aw = d(O.AdamW)
    assert (aw["beta1"], aw["beta2"], aw["epsilon"], aw["weightDecay"]) == (0.9, 0.999, 1e-8, 0.01)
    am = d(O.AMSGrad)
    assert (am["beta1"], am["beta2"], am["epsilon"]) == (0.9, 0.999, 1e-8)
    assert (d(O.RMSprop)["beta"], d(O.RMSprop)["epsilon"]) == (0.99, 1e-8)
    assert d(O.Adagrad)["epsilon"] == 1e-8
    assert d(O.NAG)["momentum"] == 0.9 and d(O.SGDMomentum)["momentum"] == 0.9
    assert list(inspect.signature(layers.MultiHeadAttention.__init__).parameters)[1:3] == ["dModel", "numHeads"]
    import pytest as _pytest
    with _pytest.raises(ValueError):
        layers.MultiHeadAttention(8, 64)          # (numHeads, dModel) order of a mis-ported call: 8 is not a multiple of 64
