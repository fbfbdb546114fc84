"""The C-ABI library loads without a GPU and exports every function include/*.h declares;
the Python prototype table covers the same set. No compute calls here."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(tfb_[a-z0-9_]+)\s*\(", text))
    return names


def test_header_declares_something():
    assert len(declared_symbols()) >= 7


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(os.path.join(ROOT, "tensors_b200", "libtfb.so"))
    missing = [n for n in sorted(declared_symbols()) if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_python_prototypes_match_header():
    import tensors_b200.capi as capi
    assert set(capi.PROTOTYPES) == declared_symbols()


def test_error_string_is_callable_without_gpu():
    import tensors_b200.capi as capi
    assert isinstance(capi.last_error(), str)
