"""The self-checking build of the library (FLUXB_DEBUG=1): the same kernels with device-side
checks of tile coordinates, push ranges, gather indices, flag call numbers and store bounds
compiled in. The checks must stay silent on correct runs, and the results must not change."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_debug_build_runs_the_dense_and_moe_checks_clean():
    env = dict(os.environ, FLUXB_DEBUG="1")
    code = (
        "import tempname_new_b200._native as n; assert n.lib()._name.endswith('libfluxb_debug.so'); "
        "import pytest, sys; sys.exit(pytest.main(['-q', '-x', '-m', 'gpu', "
        "'tests/test_dense_gpu.py', 'tests/test_moe_gpu.py', '-k', "
        "'bf16 or fused_ops or ulysses or int8 or moe or grouped']))"
    )
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


@pytest.mark.gpu
def test_debug_build_reports_a_flag_from_a_far_future_call():
    """The call-number check is a comparison of two values the kernel already holds: a flag that is
    2^26 calls ahead of the expected one is reported through the status word (site 105), and the
    same wait in the normal build passes silently."""
    code = (
        "import ctypes, torch; from tempname_new_b200 import _native; dev = torch.device('cuda', 0); "
        "flag = torch.full((1,), 1 << 26, dtype=torch.int32, device=dev); "
        "status = torch.zeros(4, dtype=torch.int32, device=dev); "
        "rc = _native.lib().fluxb_wait_flag(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint32(1), "
        "ctypes.c_uint64(200000000), ctypes.c_void_p(status.data_ptr()), "
        "ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)); "
        "torch.cuda.synchronize(); print('STATUS', rc, status.tolist()[0])"
    )
    for debug, expect in (("1", "STATUS 0 105"), ("0", "STATUS 0 0")):
        r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=dict(os.environ, FLUXB_DEBUG=debug),
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0 and expect in r.stdout, r.stdout[-1000:] + r.stderr[-2000:]


def test_debug_switch_selects_the_library(monkeypatch):
    from tempname_new_b200 import _native
    monkeypatch.setenv("FLUXB_DEBUG", "1")
    assert _native.debug_enabled()
    monkeypatch.setenv("FLUXB_DEBUG", "0")
    assert not _native.debug_enabled()
    assert _native._LIB_DEBUG.name == "libfluxb_debug.so" and _native._LIB.name == "libfluxb.so"
