"""The C-ABI library loads on a host without a GPU, exports every entry point the
header declares, and refuses to compute without a device.  No compute calls here."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT
from rstorch_b200 import _lib


def declared_in_header():
    text = open(os.path.join(ROOT, "include", "rstorch_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rst_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_in_tree():
    assert os.path.exists(_lib.LIB_PATH), "run `python -m rstorch_b200.build`"
    assert os.path.dirname(_lib.LIB_PATH) == os.path.join(ROOT, "rstorch_b200")


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    names = declared_in_header()
    assert len(names) >= 50
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.exported_symbols()) == names, "ctypes table and header disagree"


def _split_args(arglist: str) -> list[str]:
    arglist = arglist.strip()
    return [] if arglist in ("", "void") else [a for a in arglist.split(",") if a.strip()]


def test_rust_bindings_declare_the_same_entry_points():
    """`bindings/rust/src/ffi.rs` cannot be compiled here (no Rust toolchain); this keeps its
    `extern "C"` block in step with the header by name, argument count and, for the
    value arguments, width (int / int64_t / uint64_t / double / size_t)."""
    header = open(os.path.join(ROOT, "include", "rstorch_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    c_decls = {m.group(1): _split_args(m.group(2))
               for m in re.finditer(r"\b(rst_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", header)}
    rust = open(os.path.join(ROOT, "bindings", "rust", "src", "ffi.rs")).read()
    rust = re.sub(r"//[^\n]*", "", rust)
    block = rust[rust.index('extern "C" {'):]
    block = block[:block.index("\n}\n")]
    rs_decls = {m.group(1): _split_args(m.group(2))
                for m in re.finditer(r"pub fn (rst_[a-z0-9_]+)\s*\(([^)]*)\)", block)}
    assert sorted(rs_decls) == sorted(c_decls)
    scalar = {"int": "c_int", "int64_t": "i64", "uint64_t": "u64", "double": "c_double", "size_t": "usize"}
    for name, c_args in c_decls.items():
        r_args = rs_decls[name]
        assert len(r_args) == len(c_args), f"{name}: {len(c_args)} arguments in C, {len(r_args)} in Rust"
        for c_arg, r_arg in zip(c_args, r_args):
            r_type = r_arg.split(":", 1)[1].strip()
            is_ptr = "*" in c_arg or "[" in c_arg
            assert is_ptr == r_type.startswith("*"), f"{name}: `{c_arg.strip()}` against `{r_arg.strip()}`"
            if not is_ptr:
                c_type = c_arg.strip().rsplit(" ", 1)[0].replace("const ", "").strip()
                assert scalar[c_type] == r_type, f"{name}: `{c_arg.strip()}` against `{r_arg.strip()}`"
    # constants the façade relies on
    for const in ("RST_BIAS_GRAD_NOALLOC_MAX_COLS", "RST_COMM_ID_BYTES"):
        c_val = re.search(rf"#define {const} (\d+)", header).group(1)
        assert re.search(rf"pub const {const}: \w+ = {c_val};", rust), const
    for m in re.finditer(r"\b(RST_(?:OK|ERR_[A-Z_]+)) = (\d+)", header):
        assert re.search(rf"pub const {m.group(1)}: c_int = {m.group(2)};", rust), m.group(1)


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.rst_version() >> 16 == 0
    assert lib.rst_status_string(0) == b"ok"
    for code in range(1, 11):
        assert lib.rst_status_string(code) not in (b"ok", b"unknown status")
    assert lib.rst_status_string(99) == b"unknown status"
    assert lib.rst_xent_slots() >= 2


def test_null_handles_are_rejected_not_dereferenced():
    lib = _lib.load()
    assert lib.rst_ctx_synchronize(None) == _lib.RST_ERR_INVALID_ARG
    assert lib.rst_tensor_free(None) == _lib.RST_OK           # free(NULL) is a no-op
    out = C.c_void_p()
    assert lib.rst_tensor_alloc(None, 2, 2, C.byref(out)) == _lib.RST_ERR_INVALID_ARG
    assert lib.rst_linear_forward(None, None, None, None, 0, None) == _lib.RST_ERR_INVALID_ARG
    assert lib.rst_sgd_plan_step(None, 0.1) == _lib.RST_ERR_INVALID_ARG
    assert lib.rst_graph_launch(None) == _lib.RST_ERR_INVALID_ARG
    assert lib.rst_last_error(None) == b"bad graph"          # message of the last context-less failure


def test_no_device_means_a_loud_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import rstorch_b200 as rt
    with pytest.raises(rt.RstError) as e:
        rt.Context(0)
    assert e.value.status == _lib.RST_ERR_CUDA
    assert "no CPU path" in str(e.value)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "rstorch_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
