"""The Python side of the C ABI declares every exported launcher's arguments; a count that
differs from the C declaration would make ctypes pass the extra pointers as 32-bit ints."""
import os
import re

from microllm_rocm_b200.kernels import attention, gemm_bf16, ops, replay  # noqa: F401  (they register their signatures)

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "microllm_rocm_b200", "csrc")
EXPORT = re.compile(r"MLB_EXPORT\s+int\s+(\w+)\s*\(([^)]*)\)", re.S)


def declared_arguments():
    found = {}
    for name in sorted(os.listdir(CSRC)):
        if not name.endswith((".cu", ".cuh", ".h")):
            continue
        text = open(os.path.join(CSRC, name)).read()
        for fn, params in EXPORT.findall(text):
            params = params.strip()
            found[(name, fn)] = 0 if params in ("", "void") else params.count(",") + 1
    return found


def test_every_registered_signature_has_the_launchers_argument_count():
    declared = declared_arguments()
    checked = 0
    for source, functions in ops._SIGNATURES.items():
        for fn, argtypes in functions.items():
            assert (source, fn) in declared, f"{fn} is registered for {source} but not exported there"
            assert len(argtypes) == declared[(source, fn)], \
                f"{source}: {fn} takes {declared[(source, fn)]} arguments, the binding declares {len(argtypes)}"
            checked += 1
    assert checked >= 20


def test_every_launcher_with_arguments_is_registered():
    registered = {(s, f) for s, fns in ops._SIGNATURES.items() for f in fns}
    for (source, fn), count in declared_arguments().items():
        if count == 0 or not source.endswith(".cu") or source == "gemv_noalloc.cu":
            continue                      # getters without arguments; the no-alloc entry point is called by raw symbol
        assert (source, fn) in registered, f"{source}: {fn} has no ctypes signature"
