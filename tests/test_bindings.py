"""The ctypes signatures in esp_b200/csrc/ops.py against the C entry points they bind.

A launcher's parameter list is read from its source text and every parameter is
mapped to the ctypes type that carries it; a drift between the two (a parameter
added on one side only, an int where a pointer goes) would otherwise show only
as a wrong result or a fault on the device.
"""
import ctypes
import re
from pathlib import Path

from esp_b200.csrc import ops
from esp_b200.csrc.build import LIBRARIES

CSRC = Path(ops.__file__).parent


def c_kind(param: str):
    """The ctypes type of one C parameter declaration."""
    p = param.strip()
    if "*" in p or p.startswith("cudaStream_t"):
        return ctypes.c_void_p
    words = p.split()[:-1]                      # the declaration without the parameter's name
    text = " ".join(w for w in words if w != "const")
    return {"int": ctypes.c_int, "long long": ctypes.c_longlong, "unsigned long long": ctypes.c_ulonglong,
            "float": ctypes.c_float}[text]


def entry_points():
    found = {}
    for src in sorted(CSRC.glob("*.cu")):
        text = src.read_text()
        for m in re.finditer(r"ESP_API\s+int\s+(\w+)\s*\(([^)]*)\)", text):
            params = [p for p in m.group(2).replace("\n", " ").split(",") if p.strip()]
            found[m.group(1)] = (src.name, [c_kind(p) for p in params])
    return found


def test_every_bound_entry_point_has_the_parameters_its_signature_says():
    found = entry_points()
    for name, sig in ops._SIGNATURES.items():
        assert name in found, f"{name} is bound in ops.py but no source file exports it"
        src, kinds = found[name]
        assert len(kinds) == len(sig), f"{name} ({src}): {len(kinds)} parameters in C, {len(sig)} in ops.py"
        for i, (a, b) in enumerate(zip(kinds, sig)):
            assert a is b, f"{name} ({src}): parameter {i} is {a.__name__} in C and {b.__name__} in ops.py"


def test_every_exported_entry_point_is_bound_or_is_the_plain_c_interface():
    found = entry_points()
    unbound = sorted(set(found) - set(ops._SIGNATURES))
    # the allocation-free decode entry point is for C callers (its header is attn_decode_noalloc.h)
    assert [n for n in unbound if not n.endswith("_noalloc")] == []


def test_every_source_file_belongs_to_one_library():
    listed = [f for files in LIBRARIES.values() for f in files]
    assert sorted(listed) == sorted(p.name for p in CSRC.glob("*.cu"))
    assert len(listed) == len(set(listed))
