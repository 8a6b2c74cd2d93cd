"""The C-ABI library loads on a machine without a GPU and exports every symbol the header
declares; compute entry points fail loudly (no CPU fallback) when no device exists."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def header_symbols():
    text = (ROOT / "include" / "tenferro_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tfb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_symbols():
    syms = header_symbols()
    assert "tfb_execute" in syms and "tfb_einsum_with_plan_into" in syms and len(syms) > 40


def test_library_exports_every_declared_symbol(tb):
    from tenferro_b200 import _lib

    lib = C.CDLL(str(_lib.LIB_PATH))
    missing = [s for s in header_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_binding_table_matches_header(tb):
    from tenferro_b200 import _lib

    assert sorted(_lib.PROTOTYPES) == header_symbols()


def header_arity():
    """{symbol: number of parameters} from the header's prototypes."""
    text = (ROOT / "include" / "tenferro_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for name, params in re.findall(r"\b(tfb_[a-z0-9_]+)\s*\(([^()]*)\)\s*;", text):
        params = params.strip()
        out[name] = 0 if params in ("", "void") else len(params.split(","))
    return out


def test_rust_sys_crate_matches_the_header():
    """The Rust `extern "C"` block is generated from the header and must agree with it: same
    symbols, same number of parameters, and the committed file is what the generator writes now."""
    import subprocess
    import sys

    sys_dir = ROOT / "rust" / "tenferro-b200-sys"
    r = subprocess.run([sys.executable, str(sys_dir / "gen_sys.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    rs = (sys_dir / "src" / "lib.rs").read_text()
    block = rs[rs.index('extern "C" {'):]
    rust = {}
    for name, params in re.findall(r"pub fn (tfb_[a-z0-9_]+)\(([^)]*)\)", block):
        rust[name] = len([p for p in params.split(",") if p.strip()])
    assert rust == header_arity()
    # every enum constant and struct of the header is there too
    text = (ROOT / "include" / "tenferro_b200.h").read_text()
    for const in set(re.findall(r"\b(TFB_[A-Z0-9_]+)\b\s*(?:=|,|\})", re.sub(r"/\*.*?\*/", "", text, flags=re.S))):
        assert f"pub const {const}:" in rs, const
    for struct in ("tfb_desc", "tfb_view", "tfb_compute_device", "tfb_gemm_problem"):
        assert f"pub struct {struct} {{" in rs
    # field order and count of the view struct (the one every call passes)
    view = rs[rs.index("pub struct tfb_view {"):]
    fields = re.findall(r"pub (\w+):", view[:view.index("}")])
    assert fields == ["base", "rank", "dims", "strides", "offset", "flags"]


def test_rust_safe_crate_uses_only_declared_items():
    """Every `sys::` item the safe crate names exists in the generated sys crate."""
    rs = (ROOT / "rust" / "tenferro-b200-sys" / "src" / "lib.rs").read_text()
    declared = set(re.findall(r"pub (?:fn|const|type|struct) (\w+)", rs))
    used = set()
    for path in (ROOT / "rust" / "tenferro-b200" / "src").glob("*.rs"):
        used |= set(re.findall(r"\bsys::(\w+)", path.read_text()))
    assert used and not (used - declared), sorted(used - declared)
    # the four pieces the binding consists of
    backend = (ROOT / "rust" / "tenferro-b200" / "src" / "backend.rs").read_text()
    assert "impl TensorPrims<Standard> for CudaBackend" in backend
    assert "impl<T: ScalarBase> Drop for CudaBuffer<T>" in (ROOT / "rust" / "tenferro-b200" / "src" / "buffer.rs").read_text()


def test_version_and_device_format(tb):
    from tenferro_b200._lib import lib

    assert b"sm_100a" in lib.tfb_version()
    # Display of ComputeDevice (tenferro-device/src/lib.rs:12-18, 62-72).
    assert str(tb.ComputeDevice.Cpu(0)) == "cpu:0"
    assert str(tb.ComputeDevice.Cuda(3)) == "cuda:3"
    assert str(tb.ComputeDevice.Hip(1)) == "hip:1"


def test_no_cpu_fallback_without_device(tb):
    """Without a GPU the context cannot be created and says why; nothing computes on the CPU."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the failure path is exercised on CPU-only machines")
    with pytest.raises(tb.DeviceError, match="no CPU path"):
        tb.Context(0)
    with pytest.raises(tb.NoCompatibleComputeDevice):
        tb.preferred_compute_devices(tb.LogicalMemorySpace.MainMemory(), tb.OpKind.Contract)
    with pytest.raises(tb.NoCompatibleComputeDevice):
        tb.preferred_compute_devices(tb.LogicalMemorySpace.GpuMemory(0), tb.OpKind.Contract)


def test_product_does_not_import_oracle():
    """The oracle is test infrastructure: no product source may name it."""
    pkg = ROOT / "tenferro-rs_b200"
    for path in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.h")) + list(pkg.rglob("*.cuh")):
        assert "oracle" not in path.read_text().lower(), path
