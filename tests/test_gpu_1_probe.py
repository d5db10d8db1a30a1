"""Pins the tcgen05 operand-layout conventions the prefill kernel relies on, one MMA tile at a time, through the
test-only probe library (tests/probe).  Every case is a shape and layout the kernels use; the probe refuses anything else
on the host, which is checked too (no launch happens for a refused request)."""
import ctypes

import numpy as np
import pytest
import torch

import layouts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def probe():
    from probe import build_probe
    return build_probe.load()


def idesc(cfmt, afmt, bfmt, m, n):
    return (cfmt << 4) | (afmt << 7) | (bfmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24)


def core_image(mat):
    """[R, Kbytes] uint8 -> no-swizzle K-major image [R/8][Kbytes/16][R%8][16]."""
    r, kb = mat.shape
    return np.ascontiguousarray(mat.reshape(r // 8, 8, kb // 16, 16).transpose(0, 2, 1, 3)).reshape(-1)


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def run(probe, a_img, b_img, a_desc, b_desc, desc, f16_kind, ksteps, ncols, expect_ok=True):
    """a_desc / b_desc = (lbo bytes, sbo bytes, layout type, byte advance per K step)."""
    out = torch.zeros((128, ncols), dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    a, b = dev(a_img), dev(b_img)
    status = probe.tri_umma_probe(a.data_ptr(), a.numel(), b.data_ptr(), b.numel(), *a_desc, *b_desc, desc, int(f16_kind),
                                  ksteps, ncols, out.data_ptr(), err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    if not expect_ok:
        return status
    assert status == 0, probe.tri_probe_last_error().decode()
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    return out.cpu().numpy()


def test_qk_swizzled_a_core_b(probe):
    rng = np.random.default_rng(0)
    a = rng.integers(-127, 128, (128, 128), dtype=np.int8)
    b = rng.integers(-127, 128, (64, 128), dtype=np.int8)
    a_img = layouts.swizzle128(a.view(np.uint8)).reshape(-1)
    got = run(probe, a_img, layouts.pack_k8(b), (0, 1024, 2, 32), (128, 1024, 0, 256), idesc(2, 1, 1, 128, 64), False, 4, 64)
    assert (got == a.astype(np.int32) @ b.astype(np.int32).T).all()


def test_pv_u8_s8_core(probe):
    rng = np.random.default_rng(1)
    p = rng.integers(0, 256, (128, 64), dtype=np.uint8)
    v = rng.integers(-127, 128, (128, 64), dtype=np.int8)      # [channel][key position]
    got = run(probe, core_image(p), core_image(v.view(np.uint8)), (128, 512, 0, 256), (128, 512, 0, 256),
              idesc(2, 0, 1, 128, 128), False, 2, 128)
    assert (got == p.astype(np.int32) @ v.astype(np.int32).T).all()


def test_pv_f16_core(probe):
    rng = np.random.default_rng(2)
    p = rng.random((128, 64), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((128, 64), dtype=np.float32).astype(np.float16)   # [channel][key]
    want = p.astype(np.float32) @ v.astype(np.float32).T
    got = run(probe, core_image(p.view(np.uint8).reshape(128, 128)), core_image(v.view(np.uint8).reshape(128, 128)),
              (128, 1024, 0, 256), (128, 1024, 0, 256), idesc(1, 0, 0, 128, 128), True, 4, 128).view(np.float32)
    assert np.abs(got - want).max() < 1e-3, np.abs(got - want).max()


def test_requests_outside_the_kernels_shapes_are_refused_on_the_host(probe):
    img = np.zeros(8192, np.uint8)
    ok_a, ok_b = (128, 512, 0, 256), (128, 512, 0, 256)
    good = idesc(2, 0, 1, 128, 128)
    # an instruction descriptor the kernels never build; a descriptor that reaches past its image; a bad layout type
    assert run(probe, img, img, ok_a, ok_b, idesc(2, 0, 1, 128, 256), False, 2, 128, expect_ok=False) < 0
    assert run(probe, img, img, (128, 1024, 0, 256), ok_b, good, False, 2, 128, expect_ok=False) < 0
    assert run(probe, img, img, (128, 512, 1, 256), ok_b, good, False, 2, 128, expect_ok=False) < 0
    assert b"umma_probe" in probe.tri_probe_last_error()


def test_qk_bf16_rows_both_swizzled(probe):
    """Scores of un-quantised heads: bf16 Q rows (A) and bf16 K rows (B), both as 128-byte-swizzled boxes of 64 features,
    the image a TMA tensor copy of the caller's [T,128] rows leaves; one box = 4 MMAs of 16 features."""
    rng = np.random.default_rng(3)
    bf16 = lambda x: (x.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)       # truncation: exact inputs below
    qf = np.round(rng.standard_normal((128, 64)) * 8).astype(np.float32) / 8               # few mantissa bits: exact in bf16
    kf = np.round(rng.standard_normal((64, 64)) * 8).astype(np.float32) / 8
    a_img = layouts.swizzle128(bf16(qf).view(np.uint8).reshape(128, 128)).reshape(-1)
    b_img = layouts.swizzle128(bf16(kf).view(np.uint8).reshape(64, 128)).reshape(-1)
    got = run(probe, a_img, b_img, (0, 1024, 2, 32), (0, 1024, 2, 32), idesc(1, 1, 1, 128, 64), True, 4, 64).view(np.float32)
    assert np.abs(got - qf @ kf.T).max() < 1e-4
