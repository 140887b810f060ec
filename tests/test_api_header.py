"""The C header against the sources and against the Python signatures (no GPU, no compiler)."""
import ctypes
import glob
import os
import re

from herbert_rs_b200 import ops

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "herbert_rs_b200", "csrc")
CTYPE = {"int": ctypes.c_int, "float": ctypes.c_float, "long long": ctypes.c_longlong,
         "unsigned long long": ctypes.c_ulonglong}


def _declarations(text, definition):
    pat = r'extern "C"\s+([^{;]*?\))\s*\{' if definition else r'^([a-z][^;{}#/]*?\))\s*;'
    return [" ".join(m.group(1).split()) for m in re.finditer(pat, text, flags=re.S | re.M)]


def _header_decls():
    out = {}
    for h in ("api.h", "no_alloc.h"):
        for d in _declarations(open(os.path.join(CSRC, h)).read(), False):
            out[re.search(r"(hb_\w+)\(", d).group(1)] = d
    return out


def test_every_exported_launcher_is_declared_as_it_is_defined():
    decls = _header_decls()
    defined = {}
    for f in glob.glob(os.path.join(CSRC, "*.cu")):
        for d in _declarations(open(f).read(), True):
            defined[re.search(r"(hb_\w+)\(", d).group(1)] = d
    assert set(defined) == set(decls), (sorted(set(defined) - set(decls)), sorted(set(decls) - set(defined)))
    for name, d in defined.items():
        assert decls[name] == d, name


def test_the_python_signatures_are_the_headers():
    decls = _header_decls()
    for name, sig in ops._SIGS.items():
        args = decls[name][decls[name].index("(") + 1:-1]
        want = []
        for a in args.split(","):
            a = a.strip()
            if "*" in a:
                want.append(ctypes.c_void_p)
            else:
                want.append(CTYPE[a.rsplit(" ", 1)[0].replace("const ", "")])
        assert want == list(sig), (name, [w.__name__ for w in want], [s.__name__ for s in sig])
