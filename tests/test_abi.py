"""CPU: the C-ABI library loads, exports what include/ks_b200.h declares, and fails loudly without a GPU."""
import ctypes
import os
import re
import subprocess
import tempfile

import numpy as np
import pytest

from kernel_scheduling_b200 import _lib
from kernel_scheduling_b200.records import KEY_ROW_DTYPE, PAIR_ROW_DTYPE, RECORD_DTYPE

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ks_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ks_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 53
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in ks_b200.h but not exported"
    assert sorted(n for n, _, _ in _lib.KS_API) == names, "the ctypes table and the header disagree"
    assert lib.ks_version() == 1


def test_struct_sizes_match_the_header():
    src = '#include <stdio.h>\n#include "ks_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu\\n", sizeof(ks_record), sizeof(ks_pair_row), sizeof(ks_key_row), sizeof(ks_config), sizeof(ks_table_info));return 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        c, exe = os.path.join(d, "s.c"), os.path.join(d, "s")
        open(c, "w").write(src)
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        sizes = [int(x) for x in subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [RECORD_DTYPE.itemsize, PAIR_ROW_DTYPE.itemsize, KEY_ROW_DTYPE.itemsize, ctypes.sizeof(_lib.KsConfig), ctypes.sizeof(_lib.KsTableInfo)]


def test_function_base_matches_reference_golden():
    rows = [line.rstrip("\n").split("\t") for line in open(os.path.join(ROOT, "tests", "golden", "function_base.tsv"))]
    assert len(rows) >= 25
    for sym, want in rows:
        assert _lib.function_base(sym) == want, sym
    # the two examples in the reference header's own comment (scheduler/kernel_key.hpp:3-4)
    assert _lib.function_base("_apply_write_kernel") == "_apply_write_kernel"
    assert any(s.startswith("_ZN2at6native29vectorized_elementwise_kernel") and w == "vectorized_elementwise_kernel" for s, w in rows)


def test_function_base_small_buffer():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4)
    assert lib.ks_function_base(b"sleep_kernel", buf, 4) == -_lib.ERR_CAPACITY
    assert lib.ks_function_base(b"abc", buf, 4) == 3 and buf.value == b"abc"


def test_no_cpu_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from kernel_scheduling_b200.pair_table import PairTableBuilder

    with pytest.raises(_lib.KsError):
        PairTableBuilder()


def test_missing_library_is_an_error(tmp_path):
    with pytest.raises(RuntimeError):
        _lib.load(str(tmp_path / "nope.so"))


def test_status_strings():
    lib = _lib.load()
    assert lib.ks_status_string(0) == b"ok"
    assert b"start_ns" in lib.ks_status_string(-_lib.ERR_NOT_ORDERED)
    assert len({lib.ks_status_string(i) for i in range(0, 11)}) == 11
