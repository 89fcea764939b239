"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, and rejects bad
arguments on the host before touching a device (no compute call needs a GPU here)."""
import os
import re

from conftest import ROOT, load_package


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "elleci_int2.h")).read()
    return sorted(set(re.findall(r"EL_API\s+[\w\s\*]+?\b(el_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    pkg = load_package()
    handle = pkg._lib.lib()
    names = _declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(handle, name), name
        assert name in pkg._lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(pkg._lib.SIGNATURES) == names
    assert handle.el_version() >= 100


def test_status_strings_and_host_side_argument_checks():
    pkg = load_package()
    lib = pkg._lib
    handle = lib.lib()
    assert handle.el_status_string(lib.EL_OK) == b"ok"
    for code in (lib.EL_ERR_INVALID_ARG, lib.EL_ERR_NULL_PTR, lib.EL_ERR_ALIGNMENT, lib.EL_ERR_UNSUPPORTED_SHAPE,
                 lib.EL_ERR_CUDA, lib.EL_ERR_DEVICE, lib.EL_ERR_DRIVER, lib.EL_ERR_TOO_LARGE):
        assert handle.el_status_string(code) not in (b"ok", b"unknown status")
    # argument validation happens before any CUDA call
    assert handle.el_pack_ternary(None, None, -1, 4, 0, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_pack_ternary(None, None, 4, 4, 7, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_pack_ternary(None, None, 4, 4, 0, None) == lib.EL_ERR_NULL_PTR
    assert handle.el_pack_ternary(None, None, 0, 4, 0, None) == lib.EL_OK            # empty input: nothing to do
    assert handle.el_quantize_rows(None, 9, 8, None, None, 1, 8, 1e-5, 0, None, None, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_quantize_rows(None, lib.EL_BF16, 4, None, None, 1, 8, 1e-5, 0, None, None, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_gemm_fwd(None, None, None, lib.EL_BF16, None, 2, 1.0, 4, 4, 4, 0, None, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_gemm_fwd(None, None, None, lib.EL_BF16, None, 1, 1.0, 4, 4, 4, 0, None, None) == lib.EL_ERR_NULL_PTR
    assert handle.el_hysteresis_from_dw(None, None, None, 1e-3, 5.0, 2, 0.0, 1, 70000, 70000, 0, 1, None) == lib.EL_ERR_UNSUPPORTED_SHAPE
    assert handle.el_linear_decode_static(None, lib.EL_BF16, None, None, lib.EL_BF16, 1.0, 65, 8, 64, None, None) == lib.EL_ERR_TOO_LARGE
    assert handle.el_decode_workspace_bytes(11008) == (64 * 11008 + 4 * 86) * 4
    assert handle.el_rmsnorm_quantize_rows(None, 9, 8, None, 1e-6, None, None, None, 1, 8, 1e-5, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_rmsnorm_quantize_rows(None, lib.EL_BF16, 4, None, 1e-6, None, None, None, 1, 8, 1e-5, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_rmsnorm_backward(None, None, 9, None, None, None, None, None, 0, 1, 8, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_swiglu_quantize_rows(None, None, 9, 8, None, 1e-6, None, None, None, 1, 8, 1e-5, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_swiglu_quantize_rows(None, None, lib.EL_BF16, 4, None, 1e-6, None, None, None, 1, 8, 1e-5, None) == lib.EL_ERR_INVALID_ARG
    assert handle.el_swiglu_backward(None, None, None, lib.EL_F16, 8, None, None, None, None, 4, None, None, 0, 1, 8, None) == lib.EL_ERR_INVALID_ARG
    # tuning knobs: range-checked, process-wide
    assert handle.el_set_decode_gemv_max_tokens(9) == lib.EL_ERR_INVALID_ARG
    assert handle.el_set_decode_mma_max_tokens(65) == lib.EL_ERR_INVALID_ARG
    assert handle.el_set_decode_gemv_max_tokens(2) == lib.EL_OK and handle.el_set_decode_mma_max_tokens(64) == lib.EL_OK
    assert handle.el_set_decode_overlap(0) == lib.EL_OK
    assert handle.el_set_peer_barrier_limit_us(-5) == lib.EL_ERR_INVALID_ARG
    assert handle.el_set_peer_barrier_limit_us(1000) == lib.EL_OK and handle.el_set_peer_barrier_limit_us(0) == lib.EL_OK
    try:
        lib.check("el_gemm_fwd", lib.EL_ERR_ALIGNMENT)
    except pkg.ElleciError as e:
        assert e.status == lib.EL_ERR_ALIGNMENT and "alignment" in str(e)
    else:
        raise AssertionError("check() must raise")


def test_tuning_setters_from_several_threads_leave_a_valid_value():
    """The knobs are process-wide atomics: setters racing on several host threads must each succeed and leave one of
    the values that was set (checked through the range check of a follow-up call, since there is no getter)."""
    import threading
    pkg = load_package()
    handle = pkg._lib.lib()
    rcs = []

    def hammer(v):
        for _ in range(2000):
            rcs.append(handle.el_set_decode_gemv_max_tokens(v))
            rcs.append(handle.el_set_decode_mma_max_tokens(8 * v))
            rcs.append(handle.el_set_decode_overlap(v & 1))

    threads = [threading.Thread(target=hammer, args=(v,)) for v in (1, 2, 3, 4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert set(rcs) == {0}
    assert handle.el_set_decode_gemv_max_tokens(2) == 0 and handle.el_set_decode_mma_max_tokens(64) == 0
    assert handle.el_set_decode_overlap(0) == 0
