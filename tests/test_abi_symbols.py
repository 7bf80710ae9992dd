"""No GPU: the C-ABI library loads and exports every symbol include/b200_kquant.h declares, the
descriptor has the wire size of the reference's rpc_tensor, and the product package refuses to
work without its CUDA library (there is no CPU fallback to fall into)."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_kquant.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"B200_API[^;(]*?\b(b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mesh_llm_b200 import build, capi

    build.build()
    lib = C.CDLL(capi.SO_PATH)
    names = declared_symbols()
    assert len(names) >= 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    unbound = [n for n in names if n not in capi.SIGNATURES]
    assert not unbound, unbound


def test_tensor_descriptor_matches_rpc_tensor_wire_size():
    from mesh_llm_b200 import capi

    # third_party/llama.cpp/patches/0002 lines 1070-1085: 296 bytes packed
    assert C.sizeof(capi.Tensor) == 296
    assert capi.Tensor.name.offset == 296 - 68 and capi.Tensor.data.offset == 296 - 76
    assert C.sizeof(capi.StageConfig) == 25 * 4


def test_host_calls_need_no_gpu_and_report_errors():
    from mesh_llm_b200 import capi

    L = capi.lib()
    assert L.b200_reg_name() == b"B200"
    assert L.b200_status_string(-4) == b"unsupported"
    assert L.b200_row_bytes(12, 5120) == 2880 and L.b200_row_bytes(14, 5120) == 4200
    # KV-cache rows: q8_0 / q4_0 codes + f16 scales, padded to 16 bytes
    assert L.b200_kv_row_bytes(8, 128) == 144 and L.b200_kv_row_bytes(2, 128) == 80 and L.b200_kv_row_bytes(1, 128) == 256
    assert L.b200_device_row_bytes(14, 5120) == 4208 and L.b200_device_row_bytes(12, 5120) == 2880
    assert L.b200_mul_mat_scratch_bytes(1, 256) == 768
    assert L.b200_dev_supports_op(1, 12, 0) == 1 and L.b200_dev_supports_op(1, 8, 0) == 0


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "mesh_llm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("the CPU oracle", "").replace("CPU oracle", ""), f
