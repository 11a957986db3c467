"""Foreign-function declarations generated from the public C headers.

The kernel and host libraries have a plain C ABI (``csrc/include/*.h``); this module parses those headers and renders
the matching declarations for another language.  ``render_rust()`` produces the ``extern "C"`` block and the
``#[repr(C)]`` structs of the ``incin-b200-sys`` crate (the reference framework is a Rust library: crates/incin is the
facade its users link; this is the equivalent entry for Rust callers of the B200 kernels).  The test-suite renders the
block again and compares it with the committed crate source, so a header change that is not mirrored in the crate fails.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from pathlib import Path

HEADERS = ("incin_b200.h", "incin_comm.h", "incin_b200_noalloc.h", "incin_host.h")
INCLUDE_DIR = Path(__file__).resolve().parent.parent / "csrc" / "include"

_SCALARS = {"int": "c_int", "unsigned": "c_uint", "unsigned int": "c_uint", "long long": "c_longlong", "float": "f32",
            "double": "f64", "int64_t": "i64", "uint64_t": "u64", "uint32_t": "u32", "uint8_t": "u8", "int32_t": "i32",
            "void": "c_void", "char": "c_char", "size_t": "usize"}


@dataclass
class Param:
    name: str
    ctype: str


@dataclass
class Function:
    name: str
    ret: str
    params: list[Param]


@dataclass
class Struct:
    name: str
    fields: list[tuple[str, str, int]]      # (name, ctype, array length or 0)


def _strip_comments(src: str) -> str:
    src = re.sub(r"/\*.*?\*/", " ", src, flags=re.S)
    return re.sub(r"//[^\n]*", " ", src)


def _norm(t: str) -> str:
    return re.sub(r"\s+", " ", t.replace("*", " * ")).strip().replace(" *", "*")


def parse_headers(include_dir: Path = INCLUDE_DIR) -> tuple[list[Struct], list[Function]]:
    structs, funcs, seen = [], [], set()
    for h in HEADERS:
        path = include_dir / h
        if not path.exists():
            continue
        src = _strip_comments(path.read_text())
        src = re.sub(r"^\s*#.*$", "", src, flags=re.M)
        for m in re.finditer(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*(\w+)\s*;", src, re.S):
            fields = []
            for decl in m.group(2).split(";"):
                decl = decl.strip()
                if not decl:
                    continue
                mm = re.match(r"^((?:const\s+)?(?:unsigned\s+int|unsigned|long\s+long|\w+)(?:\s*\*+)?)\s*(.*)$", decl)
                base, names = mm.group(1).strip(), mm.group(2)
                # pointer stars bind to the type for every declarator in our headers
                for nm in names.split(","):
                    nm = nm.strip()
                    this_base = base
                    while nm.startswith("*"):          # `const void *q, *k, *v;`
                        nm, this_base = nm[1:].strip(), (base if base.endswith("*") else base + "*")
                    arr = re.match(r"(\w+)\[(\w+)\]", nm)
                    if arr:
                        n = arr.group(2)
                        fields.append((arr.group(1), _norm(this_base), int(n) if n.isdigit() else 64))
                    else:
                        fields.append((nm, _norm(this_base), 0))
            structs.append(Struct(m.group(3), fields))
        body = re.sub(r"typedef\s+struct\s+\w+\s*\{.*?\}\s*\w+\s*;", " ", src, flags=re.S)
        for m in re.finditer(r"([\w\s\*]+?)\b(incin_\w+)\s*\(([^;{]*?)\)\s*;", body, re.S):
            name = m.group(2)
            if name in seen:
                continue
            seen.add(name)
            params = []
            plist = m.group(3).strip()
            if plist and plist != "void":
                for p in plist.split(","):
                    p = p.strip()
                    arr = re.match(r"(.+?)(\w+)\[(\w*)\]$", p)
                    if arr:
                        params.append(Param(arr.group(2), _norm(arr.group(1)) + "*"))
                        continue
                    mm = re.match(r"^((?:const\s+)?(?:unsigned\s+int|unsigned|long\s+long|\w+)(?:\s*\*+\s*(?:const\s*\*+)?)?)\s*(\w+)$", p)
                    if not mm:
                        raise ValueError(f"cannot parse parameter {p!r} of {name}")
                    params.append(Param(mm.group(2), _norm(mm.group(1))))
            funcs.append(Function(name, _norm(m.group(1).replace("extern", "").replace('"C"', "")), params))
    return structs, funcs


def _rust_type(ctype: str, structs: set[str]) -> str:
    """``const T* const*`` -> ``*const *const T``: the const before the base qualifies the pointee, a const after a
    star qualifies that pointer level."""
    toks = re.findall(r"\*|\w+", ctype.replace("struct ", ""))
    base_const, base_words, levels = False, [], []
    for t in toks:
        if t == "*":
            levels.append(False)
        elif t == "const":
            if levels:
                levels[-1] = True
            else:
                base_const = True
        else:
            base_words.append(t)
    base = " ".join(base_words)
    if base in structs:
        out = base
    elif base in _SCALARS:
        out = _SCALARS[base]
    else:
        raise ValueError(f"no Rust mapping for C type {ctype!r}")
    pointee_const = base_const
    for lvl_const in levels:
        out = ("*const " if pointee_const else "*mut ") + out
        pointee_const = lvl_const
    return out


_KEYWORDS = {"type", "ref", "in", "box", "move", "loop", "match", "fn", "mod", "use", "impl", "self"}


def _ident(n: str) -> str:
    return f"r#{n}" if n in _KEYWORDS else n


def parse_constants(include_dir: Path = INCLUDE_DIR) -> list[tuple[str, int]]:
    """Enumerators of every (named or anonymous) enum in the headers, in declaration order, with their values."""
    consts, seen = [], set()
    for h in HEADERS:
        path = include_dir / h
        if not path.exists():
            continue
        src = _strip_comments(path.read_text())
        for m in re.finditer(r"\benum\b\s*\w*\s*\{(.*?)\}", src, re.S):
            nxt = 0
            for item in m.group(1).split(","):
                item = item.strip()
                if not item:
                    continue
                name, _, val = (t.strip() for t in item.partition("="))
                value = int(val, 0) if val else nxt
                nxt = value + 1
                if name not in seen:
                    seen.add(name)
                    consts.append((name, value))
    return consts


def render_rust(include_dir: Path = INCLUDE_DIR) -> str:
    structs, funcs = parse_headers(include_dir)
    names = {s.name for s in structs}
    out = ["// Generated from csrc/include/*.h by `python -m incin_b200 ffi`; do not edit by hand.",
           "#![allow(non_camel_case_types, non_snake_case)]", "",
           "use core::ffi::{c_char, c_int, c_longlong, c_uint, c_void};", ""]
    for cname, cval in parse_constants(include_dir):
        out.append(f"pub const {cname}: c_int = {cval};")
    out.append("")
    for s in structs:
        out += ["#[repr(C)]", "#[derive(Clone, Copy)]", f"pub struct {s.name} {{"]
        for name, ct, n in s.fields:
            rt = _rust_type(ct, names)
            out.append(f"    pub {_ident(name)}: {'[' + rt + '; ' + str(n) + ']' if n else rt},")
        out += ["}", ""]
    out.append('extern "C" {')
    for f in sorted(funcs, key=lambda f: f.name):
        ps = ", ".join(f"{_ident(p.name)}: {_rust_type(p.ctype, names)}" for p in f.params)
        ret = "" if f.ret == "void" else f" -> {_rust_type(f.ret, names)}"
        out.append(f"    pub fn {f.name}({ps}){ret};")
    out += ["}", ""]
    return "\n".join(out)
