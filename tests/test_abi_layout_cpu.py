"""No GPU: the layout of the structs that cross the C ABI, as three parties state it.

The C header is the definition.  A C compiler is asked for sizeof and offsetof of every field of
b200_stage_config and b200_tensor; the ctypes mirrors used by the tests and the bench must agree
field by field, and so must the Rust `#[repr(C)]` structs printed in INTEGRATION.md, which a
maintainer of the reference would paste into its host code: a struct that is short by a field
makes b200_stage_create read past its end.
"""
import ctypes as C
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200_kquant.h")

RUST_SIZES = {"i32": 4, "u32": 4, "f32": 4, "u64": 8, "i64": 8}


def header_struct_fields(name):
    """[(field, c type, array length or 0)] of `typedef struct <name> { ... }` in the header"""
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    body = re.search(r"typedef struct %s\s*\{(.*?)\}\s*%s;" % (name, name), text, flags=re.S).group(1)
    out = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        ctype, rest = decl.split(None, 1)
        for f in rest.split(","):
            f = f.strip()
            m = re.match(r"(\w+)\[(\d+)\]$", f)
            out.append((m.group(1), ctype, int(m.group(2))) if m else (f, ctype, 0))
    return out


def compiler_layout(struct, fields, tmp_path):
    src = tmp_path / f"layout_{struct}.c"
    lines = ['#include <stddef.h>', '#include <stdio.h>', f'#include "{HEADER}"', "int main(void) {",
             f'  printf("sizeof %zu\\n", sizeof({struct}));']
    for f, _, _ in fields:
        lines.append(f'  printf("{f} %zu\\n", offsetof({struct}, {f}));')
    lines += ["  return 0;", "}"]
    src.write_text("\n".join(lines))
    exe = tmp_path / f"layout_{struct}"
    subprocess.check_call(["gcc", "-o", str(exe), str(src)])
    out = subprocess.check_output([str(exe)], text=True).split()
    vals = dict(zip(out[0::2], map(int, out[1::2])))
    return vals.pop("sizeof"), vals


def rust_struct_fields(name):
    """[(field, rust type, array length or 0)] of `pub struct <name> { ... }` in INTEGRATION.md"""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    body = re.search(r"pub struct %s\s*\{(.*?)\}" % name, text, flags=re.S).group(1)
    out = []
    for f, ty in re.findall(r"pub (\w+):\s*(\[[^\]]+\]|\w+)", body):
        m = re.match(r"\[(\w+);\s*(\d+)\]", ty)
        out.append((f, m.group(1), int(m.group(2))) if m else (f, ty, 0))
    return out


def test_stage_config_layout_agrees_between_header_ctypes_and_the_rust_binding(tmp_path):
    from mesh_llm_b200 import capi

    fields = header_struct_fields("b200_stage_config")
    size, offs = compiler_layout("b200_stage_config", fields, tmp_path)
    assert C.sizeof(capi.StageConfig) == size
    assert [f for f, _, _ in fields] == [f for f, _ in capi.StageConfig._fields_]
    for f, _, _ in fields:
        assert getattr(capi.StageConfig, f).offset == offs[f], f
    rust = rust_struct_fields("B200StageConfig")
    assert [f for f, _, _ in rust] == [f for f, _, _ in fields]
    pos = 0
    for (f, rty, n), (_, cty, _) in zip(rust, fields):
        assert pos == offs[f], (f, pos, offs[f])
        assert (rty == "f32") == (cty == "float"), f
        pos += RUST_SIZES[rty] * max(n, 1)
    assert pos == size


def test_tensor_descriptor_layout_agrees_between_header_ctypes_and_the_rust_binding(tmp_path):
    from mesh_llm_b200 import capi

    fields = header_struct_fields("b200_tensor")
    size, offs = compiler_layout("b200_tensor", fields, tmp_path)
    assert size == 296 == C.sizeof(capi.Tensor)
    for f, _, _ in fields:
        assert getattr(capi.Tensor, f).offset == offs[f], f
    rust = [("type" if f == "ty" else f, t, n) for f, t, n in rust_struct_fields("B200Tensor")]  # `type` is a Rust keyword
    assert [f for f, _, _ in rust] == [f for f, _, _ in fields]
    pos = 0  # #[repr(C, packed)]: fields follow one another without padding
    for f, rty, n in rust:
        assert pos == offs[f], (f, pos, offs[f])
        pos += (1 if rty == "u8" else RUST_SIZES[rty]) * max(n, 1)
    assert pos == size
