"""The CUDA libraries as files: they build for sm_100a without a GPU and export what the engine
switches at run time (no GPU needed: nothing is launched)."""
import ctypes

from vllm_lite_b200.csrc import build, ops


def kernel_libraries():
    for name in build.SOURCES:
        yield name, None
    for name, variants in build.VARIANTS.items():
        for defines in variants:
            yield name, defines


def test_every_kernel_library_builds_and_exports_the_launch_switch():
    """Steps of many tokens are launched without programmatic dependent launch; the switch lives in
    every library (csrc/common.cuh), so a library without it would keep the attribute on."""
    for name, defines in kernel_libraries():
        handle = build.load(name, defines)
        assert isinstance(handle, ctypes.CDLL)
        assert hasattr(handle, "vl_set_pdl"), f"{name} {defines} exports no vl_set_pdl"


def test_the_paired_product_has_no_path_to_dependent_launch():
    """The product on clusters of two blocks stood still on the device now and then when it was started
    as a programmatic dependent.  Its launcher therefore builds its own launch with the cluster attribute
    alone: it neither names the other attribute nor goes through the shared launcher that adds it."""
    import re
    text = (build.CSRC / "gemm_tc5_pair.cu").read_text()
    code = re.sub(r"//[^\n]*", "", text)
    assert "ProgrammaticStreamSerialization" not in code
    assert "vl_launch(" not in code and "vl_pdl_enabled" not in code
    assert re.search(r"cfg\.numAttrs\s*=\s*1\s*;", code) and code.count("numAttrs") == 1
    assert code.count("cudaLaunchKernelEx") == 1
    # the kernels that allocate tensor memory do so behind their wait for the kernels before them
    for name in ("gemm_tc5_pair.cu", "gemm_tc5.cu", "flash_tc5.cu"):
        body = re.sub(r"//[^\n]*", "", (build.CSRC / name).read_text())
        body = body[body.index("__global__"):]
        assert 0 < body.index("pdl_wait();") < body.index("alloc"), name


def test_dependent_launch_is_off_until_switched_on():
    assert ops._pdl is False or ops._pdl_libs            # the module's default; a test before may have stepped
    for name, defines in kernel_libraries():
        handle = build.load(name, defines)
        if (name, build._variant(defines)) not in ops._pdl_libs:
            assert handle.vl_get_pdl() == 0, name


def test_digest_covers_every_header():
    """A library is rebuilt when any header beside the sources changes, plain C headers included."""
    import hashlib
    before = build._digest("attention")
    h = build.CSRC / "zz_probe_header.h"
    try:
        h.write_text("// probe\n")
        assert build._digest("attention") != before
    finally:
        h.unlink()
    assert build._digest("attention") == before


def test_set_pdl_reaches_the_libraries_that_are_loaded():
    calls = []
    saved, saved_flag = dict(ops._pdl_libs), ops._pdl
    try:
        ops._pdl_libs.clear()
        ops._pdl_libs[("fake", "")] = calls.append
        ops.set_pdl(not saved_flag)
        ops.set_pdl(not saved_flag)              # no change: nothing is called again
        ops.set_pdl(saved_flag)
        assert calls == [int(not saved_flag), int(saved_flag)]
    finally:
        ops._pdl_libs.clear()
        ops._pdl_libs.update(saved)
        ops._pdl = saved_flag


def test_ctypes_signatures_match_the_c_declarations():
    """The engine calls its libraries through ctypes, where nothing checks an argument list: a float
    passed where the C side reads an int goes wrong silently.  So the declarations are read from the
    sources and compared, kind by kind (pointer, int, 64-bit int, float), with what ops.py binds."""
    import re
    declared = {}
    for path in build.CSRC.glob("*.cu"):
        for m in re.finditer(r'extern "C" int (\w+)\(([^)]*)\)\s*\{', path.read_text(), re.S):
            declared[(path.stem, m.group(1))] = [a.strip() for a in m.group(2).replace("\n", " ").split(",") if a.strip()]

    def c_kind(arg):
        if "*" in arg:
            return "pointer"
        type_words = " ".join(arg.split()[:-1])
        if "float" in type_words:
            return "float"
        if "long long" in type_words or "size_t" in type_words or "int64" in type_words:
            return "int64"
        return "int"

    py_kind = {ctypes.c_void_p: "pointer", ctypes.c_float: "float", ctypes.c_int: "int",
               ctypes.c_longlong: "int64", ctypes.c_size_t: "int64"}
    assert ops._SIGNATURES
    for key, bound in ops._SIGNATURES.items():
        assert key in declared, f"{key} is bound but not declared extern C in its source"
        assert [c_kind(a) for a in declared[key]] == [py_kind[t] for t in bound], key


def test_host_core_bindings_match_the_c_declarations():
    """The same check for the C++ core of cache manager and scheduler (cache/native.py)."""
    import re
    from ctypes import c_int, c_longlong
    from vllm_lite_b200.cache import native
    lib = native._core()
    text = (build.CSRC / "host" / "cache_core.cpp").read_text()
    found = 0
    for m in re.finditer(r"^\s*([\w \*]+?)\s*\b(v[cs]_\w+)\(([^)]*)\)\s*\{", text, re.S | re.M):
        ret, name, args = m.group(1).strip(), m.group(2), [a.strip() for a in m.group(3).replace("\n", " ").split(",") if a.strip()]
        fn = getattr(lib, name)
        assert fn.argtypes is not None, f"{name} is exported but not bound"

        def c_kind(text_type):
            if "*" in text_type:
                return "pointer"
            return "int64" if "long long" in text_type else "int"

        def py_kind(t):
            return {c_int: "int", c_longlong: "int64"}.get(t, "pointer")

        assert [c_kind(" ".join(a.split()[:-1]) if "*" not in a else a) for a in args] == [py_kind(t) for t in fn.argtypes], name
        want = "void" if ret == "void" else c_kind(ret)
        assert want == ("void" if fn.restype is None else py_kind(fn.restype)), name
        found += 1
    assert found >= 19
