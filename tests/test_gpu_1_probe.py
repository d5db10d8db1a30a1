"""Pins the tcgen05 operand-layout conventions the prefill kernel relies on, one MMA tile at a time."""
import numpy as np
import pytest
import torch

from triattention_b200.kernels import layouts

pytestmark = pytest.mark.gpu


def idesc(cfmt, afmt, bfmt, m, n):
    return (cfmt << 4) | (afmt << 7) | (bfmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24)


def core_image(mat, chunk_bytes=16):
    """[R, Kbytes] uint8 -> no-swizzle K-major image [R/8][Kbytes/16][R%8][16]."""
    r, kb = mat.shape
    return np.ascontiguousarray(mat.reshape(r // 8, 8, kb // 16, 16).transpose(0, 2, 1, 3)).reshape(-1)


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def test_qk_swizzled_a_core_b(module):
    rng = np.random.default_rng(0)
    a = rng.integers(-127, 128, (128, 128), dtype=np.int8)
    b = rng.integers(-127, 128, (64, 128), dtype=np.int8)
    a_img = layouts.swizzle128(a.view(np.uint8)).reshape(-1)
    b_img = layouts.pack_k8(b)
    want = a.astype(np.int32) @ b.astype(np.int32).T
    tried = {}
    for name, bd in (("lbo128_sbo1024", (128, 1024, 0, 256)), ("lbo1024_sbo128", (1024, 128, 0, 256))):
        got = module.umma_probe(dev(a_img), dev(b_img), (0, 1024, 2, 32), bd, idesc(2, 1, 1, 128, 64), False, 4, 64)
        module.check_device_error()
        tried[name] = bool((got.cpu().numpy() == want).all())
    assert tried["lbo128_sbo1024"], f"QK descriptor convention: {tried}"


def test_pv_u8_s8_core(module):
    rng = np.random.default_rng(1)
    p = rng.integers(0, 256, (128, 64), dtype=np.uint8)
    v = rng.integers(-127, 128, (128, 64), dtype=np.int8)      # [channel][key position]
    want = p.astype(np.int32) @ v.astype(np.int32).T
    got = module.umma_probe(dev(core_image(p)), dev(core_image(v.view(np.uint8))), (128, 512, 0, 256), (128, 512, 0, 256),
                            idesc(2, 0, 1, 128, 128), False, 2, 128)
    module.check_device_error()
    assert (got.cpu().numpy() == want).all()


def test_pv_f16_core(module):
    rng = np.random.default_rng(2)
    p = rng.random((128, 64), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((128, 64), dtype=np.float32).astype(np.float16)   # [channel][key]
    want = p.astype(np.float32) @ v.astype(np.float32).T
    got = module.umma_probe(dev(core_image(p.view(np.uint8).reshape(128, 128))), dev(core_image(v.view(np.uint8).reshape(128, 128))),
                            (128, 1024, 0, 256), (128, 1024, 0, 256), idesc(1, 0, 0, 128, 128), True, 4, 128)
    module.check_device_error()
    got = got.cpu().numpy().view(np.float32)
    assert np.abs(got - want).max() < 1e-3, np.abs(got - want).max()
