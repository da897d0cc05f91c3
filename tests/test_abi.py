"""The C-ABI library loads without a GPU, exports every declared symbol, and fails loudly."""
import ctypes as C
import os
import re

import pytest

from dyninfer_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "dyninfer_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(dyninfer_cuda_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound(native_lib):
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(native_lib, n), f"{n} declared in include/dyninfer_cuda.h but not exported"
    assert set(names) == set(_lib.PROTOTYPES), set(names) ^ set(_lib.PROTOTYPES)
    assert native_lib.dyninfer_cuda_abi_version() == 1


def test_row_bytes_table(native_lib):
    rb = native_lib.dyninfer_cuda_row_bytes
    assert rb(_lib.ENC["gguf.q4_0"], 1024) == 576 and rb(_lib.ENC["gguf.q4_1"], 1024) == 640
    assert rb(_lib.ENC["gguf.q8_0"], 1024) == 1088 and rb(_lib.ENC["gguf.q6_k"], 1024) == 840
    assert rb(_lib.ENC["mlx.affine.u4"], 1024) == 512 and rb(_lib.ENC["plain.bf16"], 1024) == 2048
    assert rb(_lib.ENC["gguf.q6_k"], 128) == 0 and rb(99, 1024) == 0


def test_argument_validation_precedes_any_launch(native_lib):
    """Host-side checks answer before the device is touched, so they can be tested anywhere."""
    w = _lib.Weight(_lib.ENC["gguf.q4_0"], 0, 0, 0, 4, 48, None, None, None)   # cols not a block multiple
    assert native_lib.dyninfer_cuda_dequant(C.byref(w), None, None) != 0
    assert "multiple" in _lib.last_error()
    w = _lib.Weight(42, 0, 0, 0, 4, 64, None, None, None)
    assert native_lib.dyninfer_cuda_linear(C.byref(w), None, 0, 1, None, None) != 0
    assert "unknown encoding" in _lib.last_error()
    h = C.c_void_p()
    rc = native_lib.dyninfer_cuda_session_create_with_file_params(b"hip", b"{}", None, 0, None, 0, C.byref(h))
    assert rc != 0 and "no CPU fallback" in _lib.last_error() and not h.value
    rc = native_lib.dyninfer_cuda_session_create_with_file_params(b"cuda", b"{not json", None, 0, None, 0, C.byref(h))
    assert rc != 0 and "model descriptor" in _lib.last_error()
    rc = native_lib.dyninfer_cuda_session_create_with_file_params(
        b"cuda", b'{"layers":1,"hidden":64,"intermediate":128,"heads":4,"head_dim":16,"vocab":32,'
        b'"params":{"token_embd.weight":{"encoding":"gguf.q3_k","shape":[32,64]}}}', None, 0, None, 0, C.byref(h))
    assert rc != 0 and "E_KERNEL_COVERAGE" in _lib.last_error()
    assert native_lib.dyninfer_cuda_session_invoke_paged_chunk(None, None, 0, 0, 0, None, None, None, 0) != 0
    assert native_lib.dyninfer_cuda_session_kv_page_count(None) == 0


def test_no_gpu_means_error_not_fallback(native_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    n = C.c_int(-1)
    assert native_lib.dyninfer_cuda_device_count(C.byref(n)) != 0 and n.value == 0
    assert "no CPU fallback" in _lib.last_error()


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "dyninfer_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


def _header_enums():
    src = open(os.path.join(ROOT, "include", "dyninfer_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return {k: int(v) for k, v in re.findall(r"\b(DYNINFER_ENC_[A-Z0-9_]+)\s*=\s*(\d+)", src)}


def test_rust_ffi_crate_follows_the_header():
    """The crate is source only (no Rust toolchain here), so its text is held to the header: every export
    declared once in the extern block, every encoding constant with the header's value."""
    rs = open(os.path.join(ROOT, "crates", "dyninfer-cuda-sys", "src", "lib.rs")).read()
    rs = re.sub(r"//[^\n]*", "", rs)
    fns = re.findall(r"\bpub fn (dyninfer_cuda_[a-z0-9_]+)\s*\(", rs)
    assert sorted(fns) == _declared(), set(fns) ^ set(_declared())
    consts = {k: int(v) for k, v in re.findall(r"pub const (DYNINFER_ENC_[A-Z0-9_]+): i32 = (\d+);", rs)}
    assert consts == _header_enums()


def test_python_encoding_ids_follow_the_header():
    enums = _header_enums()
    names = {"plain.f32": "F32", "plain.f16": "F16", "plain.bf16": "BF16", "gguf.q4_0": "Q4_0",
             "gguf.q4_1": "Q4_1", "gguf.q8_0": "Q8_0", "gguf.q6_k": "Q6_K", "mlx.affine.u4": "MLX_U4",
             "gguf.q4_k": "Q4_K", "gguf.q5_k": "Q5_K", "gguf.iq4_xs": "IQ4_XS"}
    assert set(_lib.ENC) == set(names)
    for enc, short in names.items():
        assert _lib.ENC[enc] == enums["DYNINFER_ENC_" + short], enc
    assert sorted(enums.values()) == list(range(len(enums)))


def test_struct_fields_agree_in_header_rust_and_ctypes():
    """Field names and their order, struct by struct, in the three places that spell them out."""
    hdr = open(os.path.join(ROOT, "include", "dyninfer_cuda.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    rs = open(os.path.join(ROOT, "crates", "dyninfer-cuda-sys", "src", "lib.rs")).read()
    twins = {"dyninfer_cuda_weight_t": _lib.Weight, "dyninfer_cuda_parameter_file_t": _lib.ParameterFile,
             "dyninfer_cuda_file_param_t": _lib.FileParam,
             "dyninfer_cuda_allocator_statistics_t": _lib.AllocatorStatistics}
    found = re.findall(r"typedef struct (\w+) \{(.*?)\}", hdr, flags=re.S)
    assert {n for n, _ in found} == set(twins)
    for name, body in found:
        c_fields = [re.search(r"(\w+)\s*$", f.strip()).group(1) for f in body.split(";") if f.strip()]
        rust_body = re.search(r"pub struct %s \{(.*?)\}" % name, rs, flags=re.S).group(1)
        assert re.findall(r"pub (\w+):", rust_body) == c_fields, name
        assert [f[0] for f in twins[name]._fields_] == c_fields, name


def test_safe_rust_crate_calls_only_declared_exports():
    rs = open(os.path.join(ROOT, "crates", "dyninfer-cuda-sys", "src", "lib.rs")).read()
    declared = set(re.findall(r"\bpub (?:fn|const|struct) (\w+)", rs))
    src_dir = os.path.join(ROOT, "crates", "dyninfer-cuda", "src")
    used = set()
    for f in sorted(os.listdir(src_dir)):
        used |= set(re.findall(r"\bsys::(\w+)", open(os.path.join(src_dir, f)).read()))
    assert used and used <= declared, used - declared
