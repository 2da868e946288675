"""CPU: the C-ABI library loads, exports every symbol the header declares, refuses to compute
without a GPU, and the host-side mirror covers the reference's operator table."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "camel_tensor_b200.h"


@pytest.fixture(scope="module")
def built():
    from camel_b200.build import build

    return build()


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ct_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "ct_matmul" in syms and "ct_binary" in syms and "ct_conv2d" in syms
    assert len(syms) >= 35


def test_library_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(str(built))
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_binding_covers_header(built):
    from camel_b200 import _lib

    assert sorted(_lib.PROTOTYPES) == declared_symbols()


def test_no_cpu_fallback(built):
    """Without a CUDA device every compute entry point must fail loudly."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import numpy as np

    import camel_b200
    from camel_b200 import tensor as T

    with pytest.raises(camel_b200.CamelTensorError) as e:
        T.from_numpy(np.ones(4, np.float32))
    assert e.value.status == camel_b200._lib.ERR_NO_DEVICE
    out = np.zeros(4, np.float32)
    a = np.ones(4, np.float32)
    rc = camel_b200.lib.ct_matmul_host(a.ctypes.data, a.ctypes.data, 2, 2, 2, out.ctypes.data)
    assert rc == camel_b200._lib.ERR_NO_DEVICE
    assert not out.any()


def test_library_links_no_vendor_math(built):
    """The measured path must not pull cuBLAS / cuDNN / torch into the library."""
    import subprocess

    deps = subprocess.run(["ldd", str(built)], capture_output=True, text=True).stdout
    for banned in ("cublas", "cudnn", "torch", "nccl", "cutlass"):
        assert banned not in deps.lower()


def test_mirror_covers_reference_operator_table():
    """Every URI the reference registers (operators.cpp:160-194; fixture written from the compiled
    reference) has a same-named function in camel_b200.tensor."""
    from camel_b200 import tensor as T

    rows = [l.split("\t") for l in (ROOT / "tests/golden/operator_table.tsv").read_text().splitlines()]
    uris = sorted({r[1] for r in rows})
    assert len(uris) == 31
    alias = {"sum_axis": "sum", "max_axis": "max", "argmax_axis": "argmax"}
    host_only = {"random", "show"}  # unseedable RNG and printing stay on the host side of the plugin
    for uri in uris:
        name = uri.split(":", 1)[1]
        if name in host_only:
            continue
        assert hasattr(T, alias.get(name, name)), f"no mirror for {uri}"
