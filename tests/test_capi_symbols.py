"""The shared library loads and exports every function include/checkers_b200.h declares
(no GPU needed: nothing is called that touches a device)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "checkers_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(chk_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    import checkers_b200  # noqa: F401  builds nothing; fails loudly if the library is missing
    from checkers_b200.build import LIB
    lib = ctypes.CDLL(LIB)
    names = declared_functions()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_host_only_entry_points():
    """Calls that involve no device: table normalisation and argument checking."""
    import numpy as np

    import checkers_b200 as chk
    hist = np.zeros(256, np.uint32)
    hist[[0, 60, 61, 188]] = [500000, 300000, 150000, 50000]
    nf, cf, xm, s = chk.normalize_histogram(hist)
    assert s == 4096 and cf[256] == 4096 and (nf[[0, 60, 61, 188]] > 0).all() and nf.sum() == 4096
    assert np.array_equal(xm, nf << 19)
    nf2, _, _, s2 = chk.normalize_histogram(hist, ensure_full_alphabet=True)
    assert s2 > 4096 and (nf2 >= 1).all()          # the reference's single decrement pass
    _, _, _, s3 = chk.normalize_histogram(hist, ensure_full_alphabet=True, repair=True)
    assert s3 == 4096
    from checkers_b200._lib import lib
    assert lib.chk_tensor_count(None, None) != 0 and b"NULL" in lib.chk_last_error()


def test_package_has_no_cpu_path():
    """Nothing shipped may reach for the oracle or the emulator."""
    pkg = os.path.join(ROOT, "checkers_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                for needle in ("oracle_lib", "liboracle", "checkers_oracle", "oracle/", "emu_lib", "cuda_emu",
                               "libemu_kernels"):
                    assert needle not in text, (f, needle)
