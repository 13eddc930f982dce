"""CPU-side checks of the boundary: the shared library loads without a GPU, exports every symbol that
include/edge_infer_b200.h declares, and the Python prototypes cover the same set. No compute calls."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "edge_infer_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ei_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(package):
    lib = package.abi.load_library()
    names = declared_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_prototypes_match_header(package):
    assert sorted(package.abi.PROTOTYPES) == declared_symbols()


def test_view_layouts_match_reference_aggregates(package):
    abi = package.abi
    word = ctypes.sizeof(ctypes.c_size_t)
    assert ctypes.sizeof(abi.View1) == 3 * word      # TensorView<T,1>{T*, size_t[1], size_t[1]}
    assert ctypes.sizeof(abi.View2) == 5 * word
    assert ctypes.sizeof(abi.View3) == 7 * word
    assert ctypes.sizeof(abi.Array) == 2 * word      # ArrayView<T>{T*, size_t}
    assert ctypes.sizeof(abi.VerifyResult) == 8 + 64


def test_version_and_error_string(package):
    lib = package.abi.load_library()
    assert b"sm_100a" in lib.ei_version()
    assert isinstance(lib.ei_last_error(), bytes)


def test_rope_table_matches_oracle_table(package, oracle):
    import numpy as np
    table = package.operators.build_rope_table(64, 128, 1e6)
    expected = oracle.op_rope_table(128, 1e6, 64)
    assert np.array_equal(table.view(np.uint32), expected.view(np.uint32))


def test_invalid_arguments_are_rejected_without_a_gpu(package):
    import pytest
    abi = package.abi
    lib = abi.load_library()
    out = abi.AwqWeight()
    empty2 = abi.View2(None, (0, 0), (0, 0))
    with pytest.raises(ValueError):
        abi.check(lib.ei_prepare_awq_bf16(empty2, empty2, empty2, 128, 256, abi.View1(None, (0,), (0,)), ctypes.byref(out)))
    with pytest.raises(ValueError):
        abi.check(lib.ei_build_rope_table(None, 4, 128, 1e6))


def test_synthetic_awq_packing_roundtrip(package):
    import numpy as np
    syn = package.synthetic
    q, s, z = syn.awq_triple(1, "wq0", 16, 256, 128, padded_groups=5)
    assert q.shape == (16, 32) and s.shape == (16, 5) and z.shape == (16, 1)
    dense = syn.awq_dequantize(q, s, z, 256, 128, round_bf16=False)
    k = 133
    w = (q.view(np.uint32)[3, k // 8] >> ((k % 8) * 4)) & 15
    zero = (z.view(np.uint32)[3, 0] >> 4) & 15
    assert dense[3, k] == (np.float32(w) - np.float32(zero)) * syn.bf16_to_float(s[3:4, 1:2])[0, 0]


SHIM_PROGRAM = r"""
#include <cstdio>
#include "edge_infer_b200.hpp"
using namespace edge_infer_b200;
int main() {
  // Argument validation happens before any CUDA call, so these paths run without a GPU: a null weight must
  // surface as std::invalid_argument, the exception the reference's operator throws for the same mistake.
  op::cuda::ExecutionContext ctx{};
  TensorView<const std::uint16_t, 2> x{};
  TensorView<std::uint16_t, 2> y{};
  op::cuda::AwqLinearWeight<std::uint16_t> weight{};
  int caught = 0;
  try {
    op::cuda::awq_linear<std::uint16_t>(ctx, x, weight, y);
  } catch (const std::invalid_argument&) {
    caught = 1;
  } catch (const std::exception&) {
    caught = 2;
  }
  std::printf("%d %s\n", caught, ei_version());
  return caught == 1 ? 0 : 1;
}
"""


def test_cpp_shim_compiles_links_and_maps_errors(package, tmp_path):
    """include/edge_infer_b200.hpp: the op::cuda names over the C ABI, exceptions as in the reference."""
    import shutil
    import subprocess

    if shutil.which("g++") is None:
        import pytest
        pytest.skip("no g++")
    library = Path(package.abi.LIB_PATH)
    source = tmp_path / "shim.cpp"
    source.write_text(SHIM_PROGRAM)
    binary = tmp_path / "shim"
    subprocess.run(["g++", "-std=c++17", "-I", str(ROOT / "include"), str(source), "-o", str(binary),
                    f"-L{library.parent}", "-ledge_infer_b200", f"-Wl,-rpath,{library.parent}"], check=True)
    result = subprocess.run([str(binary)], capture_output=True, text=True)
    assert result.returncode == 0, result.stdout + result.stderr
    assert result.stdout.startswith("1 ")
