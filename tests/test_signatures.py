"""The ctypes signatures in ``ops/library.py`` against the ``extern "C"`` definitions in the
CUDA sources: same names, same number of arguments, pointers where pointers are, floats where
floats are.  A drift between the two corrupts arguments silently, so it is checked without a
GPU, from the source text."""

import ctypes
import os
import re

from servelab_b200.ops import library as L

CSRC = os.path.join(os.path.dirname(os.path.abspath(L.__file__)), "..", "csrc")


def _definitions():
    """name -> list of parameter declarations, for every ``int|long long|const char* slb_*(...) {``."""
    out = {}
    for fn in sorted(os.listdir(CSRC)):
        if not fn.endswith(".cu"):
            continue
        text = open(os.path.join(CSRC, fn)).read()
        text = re.sub(r"//[^\n]*", "", text)
        for m in re.finditer(r"\b(?:int|long long|const char\*)\s+(slb_\w+)\s*\(", text):
            depth, i = 1, m.end()
            while depth:
                depth += {"(": 1, ")": -1}.get(text[i], 0)
                i += 1
            rest = text[i:i + 40].lstrip()
            if not rest.startswith("{"):
                continue                                    # a declaration or a call
            params = text[m.end():i - 1].strip()
            plist = [] if params in ("", "void") else [p.strip() for p in params.split(",")]
            named = [p for p in plist if re.search(r"\w+\s*$", p) and not p.endswith("*")]
            if len(named) != len(plist):
                continue                                    # the stub of a head size that has no kernel
            out.setdefault(m.group(1), plist)
        # a status word with its accessor `int fn(int reset)`, defined through the macro of common.cuh
        for m in re.finditer(r"^SLB_DEFINE_STATUS_WORD\(\s*\w+\s*,\s*(slb_\w+)\s*\)", text, re.M):
            out.setdefault(m.group(1), ["int reset"])
    return out


def _kind(param: str) -> str:
    if "*" in param or "cudaStream_t" in param:
        return "pointer"
    if re.match(r"(const\s+)?float\b", param):
        return "float"
    if re.match(r"(const\s+)?long long\b", param):
        return "longlong"
    return "int"


_CTYPES = {ctypes.c_void_p: "pointer", ctypes.c_float: "float", ctypes.c_longlong: "longlong",
           ctypes.c_int: "int"}


def test_every_declared_signature_matches_its_definition():
    defs = _definitions()
    tables = dict(L._CORE_SIGNATURES)
    tables.update(L._OPTIONAL_SIGNATURES)
    tables.update(L._ATTN_SIGNATURES)
    assert len(tables) > 30
    problems = []
    for name, sig in tables.items():
        if name not in defs:
            problems.append(f"{name}: no definition found in the sources")
            continue
        kinds = [_kind(p) for p in defs[name]]
        want = [_CTYPES[t] for t in sig]
        if kinds != want:
            problems.append(f"{name}: sources {kinds} != library.py {want}")
    assert not problems, "\n".join(problems)
