"""The allocation-free gradient-norm entry point (csrc/grad_norm_static.h), called through its exported C symbol and
compared against the caller-buffer entry point ``sb_grad_norm_clip``.  Collected last by name so that it also runs after
every other GPU test has used the library."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "speech_b200", "ops", "libspeech_b200.so")


def _lib():
    lib = ctypes.CDLL(LIB_PATH)
    lib.sb_grad_norm_clip_static.restype = ctypes.c_int
    lib.sb_grad_norm_clip_static.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_float,
                                             ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    lib.sb_grad_norm_clip.restype = ctypes.c_int
    lib.sb_grad_norm_clip.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                      ctypes.c_float, ctypes.c_void_p]
    lib.sb_grad_norm_partials.restype = ctypes.c_int
    lib.sb_grad_norm_static_max_parts.restype = ctypes.c_int
    return lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_static_grad_norm_matches_buffer_variant_twice():
    lib = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    torch.manual_seed(3)
    n = 40_000_003  # 160 MB of fp32: larger than L2, and not a multiple of 4
    partial = torch.empty(lib.sb_grad_norm_partials(), dtype=torch.float32, device=dev)
    for call in range(2):  # two calls in a row share the static scratch
        g = torch.randn(n, device=dev, dtype=torch.float32) * (0.5 + call)
        max_norm, scale = 1.0, 0.25 * (call + 1)
        ref_scalars = torch.zeros(3, device=dev)
        new_scalars = torch.zeros(3, device=dev)
        assert lib.sb_grad_norm_clip(g.data_ptr(), n, partial.data_ptr(), ref_scalars.data_ptr(), max_norm, scale, _stream()) == 0
        assert lib.sb_grad_norm_clip_static(g.data_ptr(), n, new_scalars.data_ptr(), max_norm, scale, 0, _stream()) == 0
        torch.cuda.synchronize()
        oracle = float(g.double().pow(2).sum().sqrt()) * scale
        assert abs(float(new_scalars[0]) - oracle) <= 1e-4 * oracle
        torch.testing.assert_close(new_scalars, ref_scalars, rtol=1e-5, atol=1e-6)
        assert float(new_scalars[2]) == 0.0


def test_static_grad_norm_other_part_counts_and_flag():
    lib = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.randn(1_000_001, device=dev)
    for parts in (1, 37, lib.sb_grad_norm_static_max_parts()):
        s = torch.zeros(3, device=dev)
        assert lib.sb_grad_norm_clip_static(g.data_ptr(), g.numel(), s.data_ptr(), 2.0, 1.0, parts, _stream()) == 0
        torch.cuda.synchronize()
        want = float(g.double().norm())
        assert abs(float(s[0]) - want) <= 1e-4 * want
        assert abs(float(s[1]) - min(1.0, 2.0 / (want + 1e-6))) <= 1e-5
    g[17] = float("inf")
    s = torch.zeros(3, device=dev)
    assert lib.sb_grad_norm_clip_static(g.data_ptr(), g.numel(), s.data_ptr(), 2.0, 1.0, 0, _stream()) == 0
    torch.cuda.synchronize()
    assert float(s[2]) == 1.0


def test_static_grad_norm_rejects_oversize(capfd):
    lib = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.ones(1024, device=dev)
    s = torch.full((3,), -7.0, device=dev)
    too_many = lib.sb_grad_norm_static_max_parts() + 1
    rc = lib.sb_grad_norm_clip_static(g.data_ptr(), g.numel(), s.data_ptr(), 1.0, 1.0, too_many, _stream())
    torch.cuda.synchronize()
    assert rc == -2
    assert "static scratch holds" in capfd.readouterr().err
    assert s.tolist() == [-7.0, -7.0, -7.0]  # nothing was launched
    assert lib.sb_grad_norm_clip_static(None, 4, s.data_ptr(), 1.0, 1.0, 0, _stream()) == -1
