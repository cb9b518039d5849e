"""The C-ABI library builds for sm_100a, loads, and exports what include/mlora.h declares."""
import os
import re

from conftest import ROOT, load


def _declared():
    src = open(os.path.join(ROOT, "include", "mlora.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(mlora_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported_and_bound():
    load("build").build()
    lib = load("_lib")
    handle = lib.lib()
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(handle, n), f"{n} declared in mlora.h but not exported"
        assert n in lib.PROTOTYPES, f"{n} has no ctypes prototype"
    assert sorted(lib.PROTOTYPES) == names
    assert handle.mlora_version() >= 100


def test_host_side_argument_checks_need_no_gpu():
    lib = load("_lib")
    h = lib.lib()
    # size / alignment validation happens before any CUDA call
    rc = h.mlora_linear(None, 0, None, None, 0, 4, 12, 8, None, None, None, None, None, 0, 0, 1, None, 0, None, 0, None)
    assert rc == -1 and b"multiples of 8" in h.mlora_last_error()
    rc = h.mlora_paged_attention(None, 0, None, None, None, 0, None, None, 1, 4, 4, 80, 16, 1e4, 1, None, 0, 1,
                                 None, 0, None)
    assert rc == -1 and b"head_dim" in h.mlora_last_error()
    assert h.mlora_bucket_sort_workspace(1024, 4, 64) == 0
    assert h.mlora_bucket_sort_workspace(5000, 1, 16) == 5 * 17 * 4


def test_every_entry_point_rejects_nonsense_on_the_host():
    """Negative sizes and null pointers come back as a negative status with a message, from every launching entry
    point, on a machine without a GPU: nothing is launched and nothing is dereferenced."""
    import ctypes as C

    lib = load("_lib")
    h = lib.lib()
    seen = 0
    for name, (res, args) in sorted(lib.PROTOTYPES.items()):
        if res is not C.c_int or name == "mlora_version":
            continue
        vals = []
        for a in args:
            if a is C.c_void_p or hasattr(a, "contents") or (hasattr(a, "_type_") and not isinstance(a._type_, str)):
                vals.append(None)
            elif a in (C.c_float, C.c_double):
                vals.append(0.0)
            else:
                vals.append(-1)
        rc = getattr(h, name)(*vals)
        assert rc < 0, f"{name} accepted negative sizes / null pointers"
        assert len(h.mlora_last_error()) > 0
        seen += 1
    assert seen >= 12
