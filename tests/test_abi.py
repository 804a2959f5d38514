"""The C ABI without a GPU: the library builds, loads and exports what the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from neura_b200 import _lib, build

    build.build()
    return _lib.load()


def declared_symbols():
    with open(os.path.join(ROOT, "include", "neura_cuda.h")) as fh:
        text = fh.read()
    return sorted(set(re.findall(r"\b(neura_cuda_\w+)\s*\(", text)))


def test_every_declared_entry_point_is_exported(lib):
    from neura_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in neura_cuda.h but not exported"
    assert sorted(_lib.SYMBOLS) == names, "the ctypes table and the header disagree"


def test_geometry_entry_points_need_no_device(lib):
    assert lib.neura_cuda_payload_bytes(8, 32) == 34
    assert lib.neura_cuda_payload_bytes(9, 256) == 144
    assert lib.neura_cuda_payload_bytes(9, 18944 * 3584) == 38191104
    assert lib.neura_cuda_payload_bytes(0, 10) == 40
    assert lib.neura_cuda_payload_bytes(11, 256) == 210        # Q6_K: heads and embeddings of common GGUF mixes
    # the other formats a GGUF may hold (crates/neura-abi/tests/layout.rs pins the same sizes)
    assert lib.neura_cuda_payload_bytes(10, 256) == 176 and lib.neura_cuda_payload_bytes(12, 512) == 220
    assert lib.neura_cuda_payload_bytes(1, 7) == 14 and lib.neura_cuda_payload_bytes(2, 7) == 14
    assert lib.neura_cuda_sealed_bytes(10, 32, 256) == 0       # sealed layouts exist for Q8_0 and Q4_K only
    assert lib.neura_cuda_payload_bytes(3, 256) == 0           # the int8 element (element.rs:7) is not on this path
    # sealing pads rows to tiles of 32 and keeps the block bytes
    assert lib.neura_cuda_sealed_bytes(9, 18944, 3584) == 38191104
    assert lib.neura_cuda_sealed_bytes(9, 33, 256) == 64 * 144
    assert lib.neura_cuda_sealed_bytes(8, 4864, 896) == 4630528
    assert lib.neura_cuda_sealed_bytes(9, 16, 200) == 0


def test_open_without_a_gpu_is_an_error_not_a_fallback(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    handle = ctypes.c_void_p()
    code = lib.neura_cuda_open(0, ctypes.byref(handle))
    assert code != 0 and not handle.value
    assert lib.neura_cuda_last_error()


def test_the_package_has_no_cpu_path():
    import neura_b200

    with pytest.raises(neura_b200.NeuraCudaError):
        import torch

        if torch.cuda.is_available():
            raise neura_b200.NeuraCudaError(0, "skipped: a GPU is present")
        neura_b200.Runtime(0)


def test_model_shapes_count_the_bytes_the_baseline_names():
    from neura_b200 import qwen

    assert qwen.QWEN25_32B_Q4K.weight_elements() == 31984189440
    assert qwen.QWEN25_32B_Q4K.weight_bytes() == 17991106560
    assert qwen.QWEN25_05B_Q8.weight_elements() == 493961216
    assert qwen.QWEN25_05B_Q8.weight_bytes() == 524833792


def header_signatures():
    """name -> number of parameters, for every entry point the header declares."""
    with open(os.path.join(ROOT, "include", "neura_cuda.h")) as fh:
        text = re.sub(r"/\*.*?\*/", "", fh.read(), flags=re.S)
    found = {}
    for name, args in re.findall(r"\b(neura_cuda_\w+)\s*\(([^;{]*?)\)\s*;", text):
        args = args.strip()
        found[name] = 0 if args == "void" else args.count(",") + 1
    return found


def test_the_rust_binding_declares_every_entry_point_with_the_headers_arity():
    # crates/neura-cuda/src/sys.rs is what a Rust host links against; no Rust toolchain is here to compile it, so its
    # declarations are checked against the header: the same names, the same number of parameters, nothing extra
    with open(os.path.join(ROOT, "crates", "neura-cuda", "src", "sys.rs")) as fh:
        text = fh.read()
    declared = {}
    for name, args in re.findall(r"pub fn (neura_cuda_\w+)\(([^)]*)\)", text):
        args = args.strip()
        declared[name] = 0 if not args else args.count(",") + 1
    header = header_signatures()
    assert len(header) >= 50
    assert declared == header
    # the structs that cross the boundary by value or by pointer keep the header's fields, in order
    with open(os.path.join(ROOT, "include", "neura_cuda.h")) as fh:
        c_text = re.sub(r"/\*.*?\*/", "", fh.read(), flags=re.S)
    for c_name, rust_name in (("nc_weight", "NcWeight"), ("nc_step", "NcStep"), ("nc_then", "NcThen"),
                              ("nc_decoder_layer", "NcDecoderLayer"), ("nc_decoder_desc", "NcDecoderDesc")):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (c_name, c_name), c_text, flags=re.S).group(1)
        c_fields = []
        for statement in body.split(";"):
            statement = statement.strip()
            if statement:
                c_fields += [re.sub(r"[\s\*]", "", part).split(" ")[-1] for part in
                             re.sub(r"^(const\s+)?\w+\s+", "", statement).split(",")]
        rust_body = re.search(r"pub struct %s \{(.*?)\n\}" % rust_name, text, flags=re.S).group(1)
        rust_fields = re.findall(r"pub (\w+):", rust_body)
        assert rust_fields == c_fields, f"{rust_name} and {c_name} disagree"
    # and the safe wrapper uses nothing the binding does not declare
    with open(os.path.join(ROOT, "crates", "neura-cuda", "src", "lib.rs")) as fh:
        used = set(re.findall(r"sys::(neura_cuda_\w+)", fh.read()))
    assert used and used <= set(declared)
