#!/usr/bin/env python
"""Generates fml_bindings.dart (dart:ffi structs, constants and one lookupFunction per entry point) from
include/fml.h, and exposes the header parser so that a test can compare struct layouts between the header,
the generated Dart file and the ctypes mirror.

    python dart/lib/cuda/gen_fml_bindings.py            # rewrites dart/lib/cuda/fml_bindings.dart
    python dart/lib/cuda/gen_fml_bindings.py --check    # exit 1 if the committed file is stale

The pattern replaced is the reference's hand-written binding (lib/cuda/cudacaller.dart:6-19: two typedefs and one
DynamicLibrary lookup).  A hand-copied struct that drifts from the header makes C read past the Dart allocation, so
the structs are never written by hand.
"""
from __future__ import annotations

import os
import re
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(HERE)))
HEADER = os.path.join(ROOT, "include", "fml.h")
OUTPUT = os.path.join(HERE, "fml_bindings.dart")

SCALARS = {"int32_t": ("Int32", "int", 4), "int64_t": ("Int64", "int", 8), "uint8_t": ("Uint8", "int", 1),
           "float": ("Float", "double", 4), "double": ("Double", "double", 8)}


@dataclass
class CType:
    base: str          # int32_t, float, char, void, fml_ctx, fml_gemm_desc ...
    ptr: int = 0       # levels of indirection
    array: int = 0     # > 0: fixed-size array of `base` + `ptr` elements

    def key(self) -> Tuple[str, int, int]:
        return (self.base, self.ptr, self.array)


@dataclass
class Field:
    name: str
    type: CType


@dataclass
class Struct:
    name: str
    fields: List[Field] = field(default_factory=list)


@dataclass
class Function:
    name: str
    ret: CType
    params: List[Field] = field(default_factory=list)


@dataclass
class Header:
    structs: Dict[str, Struct]
    enums: Dict[str, List[Tuple[str, int]]]
    defines: Dict[str, int]
    functions: List[Function]
    opaque: List[str]


def _strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def _parse_type(decl: str) -> Tuple[CType, str]:
    """'const float* const* bufs' -> (CType(float, 2), 'bufs'); 'uint8_t out[128]' -> (CType(uint8_t, 0, 128), 'out')."""
    decl = decl.strip()
    arr = 0
    m = re.search(r"\[(\d+)\]\s*$", decl)
    if m:
        arr = int(m.group(1))
        decl = decl[:m.start()].strip()
    ptr = decl.count("*")
    toks = [t for t in re.sub(r"[*]", " ", decl).split() if t not in ("const", "struct")]
    if len(toks) == 1:       # unnamed parameter (e.g. `void`)
        return CType(toks[0], ptr, arr), ""
    return CType(" ".join(toks[:-1]), ptr, arr), toks[-1]


def parse_header(text: str) -> Header:
    text = _strip_comments(text)
    defines = {m.group(1): int(m.group(2), 0) for m in re.finditer(r"#define\s+(FML_\w+)\s+(-?\w+)\s*$", text, flags=re.M)
               if re.fullmatch(r"-?(0x)?[0-9a-fA-F]+", m.group(2))}
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    text = re.sub(r'extern\s+"C"\s*\{', "", text)
    enums: Dict[str, List[Tuple[str, int]]] = {}
    for m in re.finditer(r"typedef\s+enum\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        items, nxt = [], 0
        for part in m.group(1).split(","):
            part = part.strip()
            if not part:
                continue
            if "=" in part:
                n, v = part.split("=")
                nxt = int(v.strip(), 0)
                items.append((n.strip(), nxt))
            else:
                items.append((part, nxt))
            nxt += 1
        enums[m.group(2)] = items
    text = re.sub(r"typedef\s+enum\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    structs: Dict[str, Struct] = {}
    for m in re.finditer(r"typedef\s+struct\s*(\w*)\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        st = Struct(m.group(3))
        for stmt in m.group(2).split(";"):
            stmt = stmt.strip()
            if not stmt:
                continue
            # `int32_t M, N, K` and `const float* q` forms; a '*' binds to the first declarator only in this header
            first, *rest = [s.strip() for s in stmt.split(",")]
            t, name = _parse_type(first)
            st.fields.append(Field(name, t))
            for r in rest:
                arr = 0
                am = re.search(r"\[(\d+)\]\s*$", r)
                if am:
                    arr, r = int(am.group(1)), r[:am.start()].strip()
                st.fields.append(Field(r.replace("*", "").strip(), CType(t.base, r.count("*"), arr)))
        structs[st.name] = st
    text = re.sub(r"typedef\s+struct\s*\w*\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    opaque = [m.group(2) for m in re.finditer(r"typedef\s+struct\s+(\w+)\s+(\w+)\s*;", text)]
    text = re.sub(r"typedef\s+struct\s+\w+\s+\w+\s*;", "", text)
    functions = []
    for m in re.finditer(r"([\w\s\*]+?)\b(\w+)\s*\(([^()]*)\)\s*;", text):
        ret, _ = _parse_type(m.group(1).strip() + " _")
        params = []
        body = m.group(3).strip()
        if body and body != "void":
            for i, p in enumerate(body.split(",")):
                t, name = _parse_type(p)
                params.append(Field(name or f"arg{i}", t))
        functions.append(Function(m.group(2), ret, params))
    return Header(structs, enums, defines, functions, opaque)


# ---------------------------------------------------------------------------------------- C layout (LP64)
def c_size_align(t: CType, structs: Dict[str, Struct]) -> Tuple[int, int]:
    if t.ptr:
        s, a = 8, 8
    elif t.base in SCALARS:
        s = a = SCALARS[t.base][2]
    elif t.base in structs:
        s, a = struct_layout(structs[t.base], structs)[1:]
    else:
        raise ValueError(f"no size for {t}")
    return (s * t.array, a) if t.array else (s, a)


def struct_layout(st: Struct, structs: Dict[str, Struct]):
    """([(field name, offset, size)], sizeof, alignment) under the System V x86-64 / AArch64 LP64 rules."""
    off, align, out = 0, 1, []
    for f in st.fields:
        s, a = c_size_align(f.type, structs)
        off = (off + a - 1) // a * a
        out.append((f.name, off, s))
        off += s
        align = max(align, a)
    return out, (off + align - 1) // align * align, align


# ---------------------------------------------------------------------------------------- Dart emission
DART_RESERVED = {"in": "inp", "is": "is_", "new": "new_", "var": "var_", "final": "final_", "class": "class_"}


def camel(name: str, upper_first: bool = False) -> str:
    if name in DART_RESERVED:
        return DART_RESERVED[name]
    parts = [p for p in name.split("_") if p]
    if not parts:
        return name
    head = parts[0] if not upper_first else parts[0][:1].upper() + parts[0][1:]
    return head + "".join(p[:1].upper() + p[1:] for p in parts[1:])


def dart_class(cname: str) -> str:
    return camel(cname, upper_first=True)     # fml_gemm_desc -> FmlGemmDesc


def native_type(t: CType, hdr: Header) -> str:
    """dart:ffi native type of a C type (arrays decay to pointers in parameter position)."""
    ptr = t.ptr + (1 if t.array else 0)
    if t.base == "char" and ptr >= 1:
        inner = "Utf8"
        ptr -= 1
    elif t.base == "void":
        if ptr == 0:
            return "Void"
        inner = "Void"
        ptr -= 1
    elif t.base in SCALARS:
        inner = SCALARS[t.base][0]
        if ptr == 0:
            return inner
        ptr -= 1
    elif t.base in hdr.structs or t.base in hdr.opaque:
        inner = dart_class(t.base)
        if ptr == 0:
            return inner
        ptr -= 1
    else:
        raise ValueError(f"unmapped C type {t}")
    out = f"Pointer<{inner}>"
    for _ in range(ptr):
        out = f"Pointer<{out}>"
    return out


def dart_type(t: CType, hdr: Header) -> str:
    if t.ptr or t.array:
        return native_type(t, hdr)
    if t.base == "void":
        return "void"
    if t.base in SCALARS:
        return SCALARS[t.base][1]
    return native_type(t, hdr)


def emit_struct(st: Struct, hdr: Header) -> str:
    lines = [f"/// `{st.name}` of include/fml.h ({struct_layout(st, hdr.structs)[1]} bytes).",
             f"final class {dart_class(st.name)} extends Struct {{"]
    for f in st.fields:
        name = camel(f.name)
        t = f.type
        if t.array:
            elem = native_type(CType(t.base, t.ptr), hdr)
            lines.append(f"  @Array({t.array}) external Array<{elem}> {name};")
        elif t.ptr:
            lines.append(f"  external {native_type(t, hdr)} {name};")
        elif t.base in SCALARS:
            n, d, _ = SCALARS[t.base]
            lines.append(f"  @{n}() external {d} {name};")
        else:
            lines.append(f"  external {dart_class(t.base)} {name};")
    lines.append("}")
    return "\n".join(lines)


def generate(hdr: Header) -> str:
    out = ["// GENERATED by dart/lib/cuda/gen_fml_bindings.py from include/fml.h -- do not edit by hand.",
           "// dart:ffi binding of libflutter_ml_b200.so: every struct, constant and entry point of the C ABI.",
           "// Replaces the two typedefs and the single lookup of the original lib/cuda/cudacaller.dart.",
           "// ignore_for_file: non_constant_identifier_names, constant_identifier_names",
           "import 'dart:ffi';", "", "import 'package:ffi/ffi.dart';", ""]
    for name in hdr.opaque:
        out += [f"/// Opaque `{name}` handle.", f"final class {dart_class(name)} extends Opaque {{}}", ""]
    for ename, items in hdr.enums.items():
        out.append(f"/// `{ename}`.")
        out.append(f"abstract final class {dart_class(ename)} {{")
        for n, v in items:
            out.append(f"  static const int {n} = {v};")
        out += ["}", ""]
    if hdr.defines:
        out.append("abstract final class FmlLimits {")
        for n, v in hdr.defines.items():
            out.append(f"  static const int {n} = {v};")
        out += ["}", ""]
    for st in hdr.structs.values():
        out += [emit_struct(st, hdr), ""]
    out += ["/// One field per entry point; `FmlBindings(DynamicLibrary.open('cuda_lib/libflutter_ml_b200.so'))`.",
            "class FmlBindings {", "  final DynamicLibrary lib;", "  FmlBindings(this.lib);", ""]
    for fn in hdr.functions:
        nat = ", ".join(native_type(p.type, hdr) for p in fn.params)
        drt = ", ".join(dart_type(p.type, hdr) for p in fn.params)
        out.append(f"  late final {camel(fn.name)} = lib.lookupFunction<")
        out.append(f"      {native_type(fn.ret, hdr)} Function({nat}),")
        out.append(f"      {dart_type(fn.ret, hdr)} Function({drt})>('{fn.name}');")
    out += ["}", ""]
    return "\n".join(out)


# ---------------------------------------------------------------------------------------- Dart parsing (for the layout test)
DART_NATIVE = {"Int32": ("int32_t", 0), "Int64": ("int64_t", 0), "Uint8": ("uint8_t", 0), "Float": ("float", 0),
               "Double": ("double", 0)}


def _dart_pointer(t: str, class_to_c: Dict[str, str]) -> CType:
    depth = 0
    while t.startswith("Pointer<") and t.endswith(">"):
        t = t[len("Pointer<"):-1]
        depth += 1
    if t == "Utf8":
        return CType("char", depth)
    if t == "Void":
        return CType("void", depth)
    if t in DART_NATIVE:
        return CType(DART_NATIVE[t][0], depth)
    return CType(class_to_c.get(t, t), depth)


def parse_dart_structs(text: str, class_to_c: Optional[Dict[str, str]] = None) -> Dict[str, Struct]:
    """`final class X extends Struct { ... }` blocks of a Dart source (or of Dart snippets in a document)."""
    class_to_c = class_to_c or {}
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for m in re.finditer(r"final\s+class\s+(\w+)\s+extends\s+Struct\s*\{(.*?)\}", text, flags=re.S):
        st = Struct(m.group(1))
        for stmt in m.group(2).split(";"):
            stmt = " ".join(stmt.split())
            if not stmt:
                continue
            am = re.match(r"@Array\((\d+)\) external Array<(.+)> (\w+)$", stmt)
            if am:
                t = _dart_pointer(am.group(2), class_to_c)
                st.fields.append(Field(am.group(3), CType(t.base, t.ptr, int(am.group(1)))))
                continue
            sm = re.match(r"@(\w+)\(\) external (?:int|double) (\w+)$", stmt)
            if sm:
                st.fields.append(Field(sm.group(2), CType(DART_NATIVE[sm.group(1)][0])))
                continue
            pm = re.match(r"external (Pointer<.+>) (\w+)$", stmt)
            if pm:
                st.fields.append(Field(pm.group(2), _dart_pointer(pm.group(1), class_to_c)))
                continue
            raise ValueError(f"unparsed Dart struct member in {st.name}: {stmt!r}")
        out[st.name] = st
    return out


def main(argv):
    hdr = parse_header(open(HEADER).read())
    text = generate(hdr)
    if "--check" in argv:
        ok = os.path.exists(OUTPUT) and open(OUTPUT).read() == text
        print("up to date" if ok else "stale: run dart/lib/cuda/gen_fml_bindings.py")
        return 0 if ok else 1
    with open(OUTPUT, "w") as f:
        f.write(text)
    print(OUTPUT, f"{len(hdr.structs)} structs, {len(hdr.functions)} functions")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
