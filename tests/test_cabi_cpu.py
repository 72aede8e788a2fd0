"""The C-ABI library builds for sm_100a, loads without a GPU, and exports exactly what the header declares."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "toner_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(toner_[a-z0-9_]+)\s*\(", text))


def test_library_builds_and_exports_every_declared_symbol():
    from toner_b200.csrc import build
    from toner_b200 import _lib
    path = build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    declared = declared_symbols()
    assert declared, "no declarations found in include/toner_b200.h"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))


def test_binding_structs_match_the_header_layout():
    """Field order of the ctypes structs follows the C structs (checked by name against the header)."""
    from toner_b200 import _lib
    text = open(os.path.join(ROOT, "include", "toner_b200.h")).read()
    for struct, cls in (("toner_operand", _lib.Operand), ("toner_gemm_desc", _lib.GemmDesc)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                ident = re.findall(r"([A-Za-z_][A-Za-z0-9_]*)\s*(?:\[\d+\])?\s*$", part.strip())
                if ident:
                    names.append(ident[0])
        assert names == [f[0] for f in cls._fields_], (struct, names, [f[0] for f in cls._fields_])


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from toner_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    try:
        _lib.load()
    except _lib.TonerError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")
