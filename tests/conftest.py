import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def qx():
    """The product: ctypes binding of libqx_b200.so (built on demand)."""
    lib_path = os.path.join(entry.PKG_DIR, "libqx_b200.so")
    if not os.path.exists(lib_path):
        entry._load_file("_qx_b200_build", os.path.join(entry.PKG_DIR, "build.py")).build()
    return entry.load_package()


@pytest.fixture(scope="session")
def wl():
    return entry._load_file(entry.PKG_NAME + ".workloads",
                            os.path.join(entry.PKG_DIR, "workloads.py"))


@pytest.fixture(scope="session")
def oracle_mod():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def orc(oracle_mod):
    """CPU oracle (plain-C restatement): the checker, never the thing under test."""
    return oracle_mod.Oracle()


@pytest.fixture(scope="session")
def ref(oracle_mod):
    """The unmodified reference library, when it was built on this machine."""
    if not oracle_mod.Reference.available():
        pytest.skip("oracle/_ref/libqx_ref.so not built here")
    return oracle_mod.Reference()


@pytest.fixture(scope="session")
def golden():
    here = os.path.join(ROOT, "tests", "golden")
    return {
        "default": np.load(os.path.join(here, "golden_default.npz")),
        "forced_ref": np.load(os.path.join(here, "golden_forced_ref.npz")),
    }


@pytest.fixture(scope="session")
def gold_inputs():
    return entry._load_file("_qx_make_golden", os.path.join(ROOT, "tests", "golden", "make_golden.py"))


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def assert_bit_equal(a, b, what=""):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    bad = np.nonzero(bits(a).reshape(-1) != bits(b).reshape(-1))[0]
    assert bad.size == 0, f"{what}: {bad.size} of {a.size} elements differ, first at {bad[:4]}: " \
                          f"{a.reshape(-1)[bad[:4]]} vs {b.reshape(-1)[bad[:4]]}"


# f32 outputs of the dequantising paths: |got - ref| <= 1e-4 + 1e-5 * |ref| per element,
# against the reference's own f32 path (the stated tolerance of this path).
def assert_close_f32_path(got, ref, what="", atol=1e-4, rtol=1e-5):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    err = np.abs(got - ref)
    tol = atol + rtol * np.abs(ref)
    worst = np.argmax(err / tol)
    assert np.all(err <= tol), f"{what}: max err/tol {np.max(err / tol):.3f} at {worst}: " \
                               f"{got.reshape(-1)[worst]} vs {ref.reshape(-1)[worst]}"


# the bound of the reference's own GEMV test against its float64 oracle
# (tests/correctness/test_qgemv.cpp:46-56, :297): atol 1e-5 + rtol 1e-4
def assert_close_ref_test(got, ref64, what=""):
    assert_close_f32_path(got, ref64, what, atol=1e-5, rtol=1e-4)
