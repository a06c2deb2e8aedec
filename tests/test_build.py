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
