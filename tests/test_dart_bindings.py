"""The documented and generated dart:ffi bindings agree with include/fml.h and with the ctypes mirror (CPU only).

No Dart SDK exists where these tests run, so the Dart files cannot be executed; what CAN be checked is what breaks a
binding silently: a struct whose field order, types or size differ from the C struct (C then reads past the Dart
allocation), a missing or mistyped entry point, a stale generated file, a stale snippet in the integration guide.
"""
import ctypes
import importlib.util
import os
import re
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GEN = os.path.join(ROOT, "dart", "lib", "cuda", "gen_fml_bindings.py")


@pytest.fixture(scope="module")
def gen():
    spec = importlib.util.spec_from_file_location("gen_fml_bindings", GEN)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["gen_fml_bindings"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def hdr(gen):
    return gen.parse_header(open(os.path.join(ROOT, "include", "fml.h")).read())


CTYPES_OF = {"fml_config": "Config", "fml_gemm_desc": "GemmDesc", "fml_lstm_desc": "LstmDesc",
             "fml_attention_desc": "AttentionDesc", "fml_op": "Op"}


def _canon(t):
    """(kind, bytes) of a C type as far as the ABI sees it: every pointer is 8 opaque bytes."""
    if t.array:
        return ("array", t.array) + _canon(type(t)(t.base, t.ptr, 0))
    if t.ptr:
        return ("ptr", 8)
    return {"int32_t": ("i", 4), "int64_t": ("i", 8), "uint8_t": ("u", 1), "float": ("f", 4), "double": ("f", 8)}[t.base]


def _canon_ctypes(ct):
    if hasattr(ct, "_length_"):
        return ("array", ct._length_) + _canon_ctypes(ct._type_)
    if ct in (ctypes.c_void_p, ctypes.c_char_p) or hasattr(ct, "contents"):
        return ("ptr", 8)
    return {ctypes.c_int32: ("i", 4), ctypes.c_int64: ("i", 8), ctypes.c_uint8: ("u", 1), ctypes.c_float: ("f", 4),
            ctypes.c_double: ("f", 8)}[ct]


def test_header_structs_match_the_ctypes_mirror(gen, hdr):
    """Field order, kinds, offsets and sizeof of every struct in fml.h against flutter_ml_b200/_lib.py, the binding all
    GPU tests run through; the header layout is computed with the LP64 rules and cross-checked by the C compiler."""
    from flutter_ml_b200 import _lib
    assert set(hdr.structs) == set(CTYPES_OF)
    for cname, pyname in CTYPES_OF.items():
        st, cls = hdr.structs[cname], getattr(_lib, pyname)
        layout, size, _ = gen.struct_layout(st, hdr.structs)
        assert size == ctypes.sizeof(cls), cname
        assert len(layout) == len(cls._fields_), cname
        for (fname, off, fsize), f, (pname, ptype) in zip(layout, st.fields, cls._fields_):
            member = getattr(cls, pname)
            assert (off, fsize) == (member.offset, member.size), (cname, fname)
            assert _canon(f.type) == _canon_ctypes(ptype), (cname, fname)
            assert pname == fname or (fname, pname) == ("in", "inp"), (cname, fname, pname)


def test_header_layout_rules_agree_with_the_c_compiler(gen, hdr, tmp_path):
    """sizeof / offsetof as gcc computes them for the real header equal the LP64 arithmetic used above."""
    import subprocess
    lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "fml.h"', "int main(void) {"]
    for st in hdr.structs.values():
        lines.append(f'  printf("{st.name} %zu\\n", sizeof({st.name}));')
        for f in st.fields:
            lines.append(f'  printf("{st.name}.{f.name} %zu\\n", offsetof({st.name}, {f.name}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for st in hdr.structs.values():
        layout, size, _ = gen.struct_layout(st, hdr.structs)
        assert int(got[st.name]) == size
        for fname, off, _ in layout:
            assert int(got[f"{st.name}.{fname}"]) == off, (st.name, fname)


def _assert_dart_struct_matches(gen, hdr, dart_struct, cname):
    st = hdr.structs[cname]
    assert [gen.camel(f.name) for f in st.fields] == [f.name for f in dart_struct.fields], cname
    for cf, df in zip(st.fields, dart_struct.fields):
        assert _canon(cf.type) == _canon(df.type), (cname, cf.name)
        if cf.type.ptr and not cf.type.array and cf.type.base in ("float", "int32_t"):
            assert cf.type.key() == df.type.key(), (cname, cf.name)      # pointee type too
    assert gen.struct_layout(dart_struct, {})[1] == gen.struct_layout(st, hdr.structs)[1], cname


def test_generated_dart_file_is_current_and_complete(gen, hdr):
    path = os.path.join(ROOT, "dart", "lib", "cuda", "fml_bindings.dart")
    text = open(path).read()
    assert text == gen.generate(hdr), "stale: run python dart/lib/cuda/gen_fml_bindings.py"
    structs = gen.parse_dart_structs(text)
    assert {gen.dart_class(n) for n in hdr.structs} == set(structs)
    for cname in hdr.structs:
        _assert_dart_struct_matches(gen, hdr, structs[gen.dart_class(cname)], cname)
    # one lookupFunction per declared entry point, bound to the symbol name the library exports
    looked_up = re.findall(r"\)>\('(\w+)'\);", text)
    assert sorted(looked_up) == sorted(f.name for f in hdr.functions)
    from flutter_ml_b200 import _lib
    assert set(looked_up) == set(_lib.PROTOTYPES)
    # native signatures: argument count and integer widths of a few calls a drifted binding would get wrong
    sig = {m.group(2): m.group(1) for m in re.finditer(r"lookupFunction<\s*(.+?),\s*\n.+?\)>\('(\w+)'\);", text)}
    assert sig["fml_alloc"] == "Int32 Function(Pointer<FmlCtx>, Int64, Pointer<Pointer<Float>>)"
    assert sig["multiplyMatrices"] == "Void Function(Pointer<Float>, Pointer<Float>, Pointer<Float>, Int32, Int32, Int32)"
    assert sig["fml_last_error"] == "Pointer<Utf8> Function(Pointer<FmlCtx>)"
    assert sig["fml_adam_step"].count("Double") == 5 and sig["fml_adam_step"].count("Pointer<Float>") == 4
    for fn in hdr.functions:
        assert sig[fn.name].count(",") + 1 == max(len(fn.params), 1), fn.name


def test_enum_constants_match_the_python_binding(hdr):
    from flutter_ml_b200 import _lib, tape
    prec = dict(hdr.enums["fml_precision"])
    assert (prec["FML_PREC_TF32"], prec["FML_PREC_3XTF32"], prec["FML_PREC_FP32"]) == (_lib.PREC_TF32, _lib.PREC_3XTF32, _lib.PREC_FP32)
    act = dict(hdr.enums["fml_act"])
    assert act["FML_ACT_GELU"] == _lib.ACT_GELU and act["FML_ACT_RELU"] == _lib.ACT_RELU
    kinds = dict(hdr.enums["fml_op_kind"])
    assert kinds["FML_OP_MATMUL"] == tape.KIND["matMul"] and kinds["FML_OP_ATTENTION"] == tape.KIND["attention"]
    assert len(kinds) == len(tape.KIND)


def test_integration_guide_structs_match_the_header(gen, hdr):
    """Every `final class ... extends Struct` quoted in INTEGRATION.md has the fields of the C struct it binds, in order,
    with the same types (a guide that stops short of the last fields hands C a struct smaller than it reads)."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = "\n".join(re.findall(r"```dart\n(.*?)```", text, flags=re.S))
    quoted = gen.parse_dart_structs(blocks)
    by_class = {gen.dart_class(n): n for n in hdr.structs}
    assert "FmlGemmDesc" in quoted, "the guide no longer shows the product descriptor"
    for cls, st in quoted.items():
        assert cls in by_class, f"{cls} is not a struct of fml.h"
        _assert_dart_struct_matches(gen, hdr, st, by_class[cls])
