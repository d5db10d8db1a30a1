"""Banded causal prefill (tcgen05) against exact integers, the CPU oracle and the reference extension."""
import numpy as np
import pytest
import torch

import triattention_oracle as orc
from ref_harness import RefRunner
import layouts
from triattention_b200.kernels.prefill import Prefill
from triattention_b200.maps import INF, from_bands, per_kv_head
from util import assert_fp_close, bf16_cuda, make_inputs

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def bands_fn_of(bands):
    return from_bands({"0": np.asarray(bands).tolist()}, None)


def test_qk_accumulators_exact(module):
    """TMEM accumulators of the production operand path equal the integer product of the codes."""
    hq, hk, t = 4, 2, 300
    q, k, v = make_inputs(hq, hk, t, seed=3, batch=2)
    pre = Prefill(module, bands_fn_of([[2, 4]] * hq))
    table, ops = pre.write(0, bf16_cuda(q), bf16_cuda(k), bf16_cuda(v))
    reqs = np.array([[0, 0, 0, 0], [1, 1, 2, 0], [5, 2, 4, 0], [7, 0, 1, 1], [2, 2, 3, 1], [6, 1, 0, 1]], np.int32)
    acc = module.qk_accumulators(torch.from_numpy(reqs).cuda(), ops["q8"], ops["q4x"], ops["k8"], ops["k4x"], 2, hq, hk, t)
    module.check_device_error()
    acc = acc.cpu().numpy()
    tiles = (t + 63) // 64
    q8 = ops["q8"].cpu().numpy().astype(np.int32)
    q4 = ops["q4x"].cpu().numpy().astype(np.int32)
    k8 = layouts.unpack_k8(ops["k8"].cpu().numpy().reshape(2 * hk, tiles, 8192)).astype(np.int32)
    k4 = layouts.unpack_k8(ops["k4x"].cpu().numpy().reshape(2 * hk, tiles, 8192)).astype(np.int32)
    for i, (qu, pair, tile, four) in enumerate(reqs):
        rows = np.zeros((128, 128), np.int32)
        lo, hi = pair * 128, min(t, pair * 128 + 128)
        rows[:hi - lo] = (q4 if four else q8)[qu, lo:hi]
        ku = (qu // hq) * hk + (qu % hq) // (hq // hk)
        want = rows @ (k4 if four else k8)[ku, tile].T
        assert (acc[i] == want).all(), (i, np.abs(acc[i] - want).max())


CASES = [
    (4, 2, 200, [[INF, INF], [INF, INF], [2, 3], [2, 3]]),
    (8, 2, 512, [[INF, INF]] * 4 + [[1, INF]] * 4),
    (2, 1, 64, [[INF, INF]] * 2),
    (2, 1, 65, [[1, INF]] * 2),
    (3, 1, 129, [[1, 2], [2, 2], [3, INF]]),
    (4, 1, 1100, [[4, 8], [1, INF], [INF, INF], [16, 17]]),
]


def product_prefill(module, q, k, v, bands, out_dtype=torch.bfloat16):
    pre = Prefill(module, bands_fn_of(bands))
    out = pre(0, bf16_cuda(q), bf16_cuda(k), bf16_cuda(v), SCALE, out_dtype=out_dtype)
    assert out.dtype == out_dtype
    module.check_device_error()
    return out.float().cpu().numpy()


@pytest.mark.parametrize("hq,hk,t,bands", CASES)
def test_prefill_vs_oracle(module, hq, hk, t, bands):
    bands = np.asarray(bands, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=13, batch=2)
    got = product_prefill(module, q, k, v, bands)
    for b in range(2):
        want = orc.prefill(q[b], k[b], v[b], bands, SCALE)
        assert_fp_close(got[b], orc.to_bf16(want), f"prefill b={b}")


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16], ids=["bf16-out", "fp16-out"])
@pytest.mark.parametrize("hq,hk,t,bands", CASES)
def test_prefill_vs_reference(module, ref_ext, hq, hk, t, bands, out_dtype):
    """Both output types of the reference's kernel (prefill_sm80.cu:533-539).  With fp16 outputs the one-ulp allowance
    for the final rounding is 8 times smaller than with bf16 (10 instead of 7 explicit significand bits)."""
    bands = np.asarray(bands, np.int64)
    q, k, v = make_inputs(hq, hk, t, seed=17, batch=1)
    got = product_prefill(module, q, k, v, bands, out_dtype)
    run = RefRunner(ref_ext)
    ref = run.prefill(bf16_cuda(q[0])[None], bf16_cuda(k[0])[None], bf16_cuda(v[0])[None], bands, SCALE, with_decode=False,
                      out_dtype=out_dtype)
    assert_fp_close(got[0], ref["out"].float().cpu().numpy()[0], "prefill vs reference kernel",
                    ulp_digits=7 if out_dtype == torch.bfloat16 else 10)


def test_prefill_c1_config(module, ref_ext):
    """benchmark configuration 1: 8 Q / 2 KV heads, T=512, outlier dims x16, map [INT8, INT4]."""
    q = orc.synth((8, 512, 128), 0, outlier_dims=(7, 42, 77, 113), outlier_scale=16.0)[None]
    k = orc.synth((2, 512, 128), 1, outlier_dims=(7, 42, 77, 113), outlier_scale=16.0)[None]
    v = orc.synth((2, 512, 128), 2)[None]
    fn = per_kv_head(["int8", "int4"], 4)
    pre = Prefill(module, fn)
    got = pre(0, bf16_cuda(q), bf16_cuda(k), bf16_cuda(v), SCALE).float().cpu().numpy()
    module.check_device_error()
    bands = fn(0, 8).numpy().astype(np.int64)
    ref = RefRunner(ref_ext).prefill(bf16_cuda(q), bf16_cuda(k), bf16_cuda(v), bands, SCALE, with_decode=False)
    assert_fp_close(got[0], ref["out"].float().cpu().numpy()[0], "C1 vs reference kernel")


def test_prefill_bf16_heads(module):
    hq, hk, t = 4, 2, 200
    q, k, v = make_inputs(hq, hk, t, seed=19, batch=1)
    pre = Prefill(module, per_kv_head(["int8", "bf16"], 2))
    got = pre(0, bf16_cuda(q), bf16_cuda(k), bf16_cuda(v), SCALE).float().cpu().numpy()
    module.check_device_error()
    want = orc.exact_attention(q[0], k[0], v[0], SCALE)
    assert_fp_close(got[0, 2:], orc.to_bf16(want[2:]), "bf16 heads vs exact attention")
    quant = orc.prefill(q[0], k[0], v[0], np.asarray([[INF, INF]] * 4), SCALE)
    assert_fp_close(got[0, :2], orc.to_bf16(quant[:2]), "quantised heads beside bf16 heads")


SWEEP = [(1, 2), (2, 2), (1, INF), (2, 8), (4, 4), (INF, INF), (8, 2048), (1, 1)]


@pytest.mark.parametrize("rows", [None, 300, 64, 5000], ids=["all-rows", "last-300", "last-64", "more-than-T"])
@pytest.mark.parametrize("batch,hq,hk,t", [(1, 4, 2, 1100), (2, 2, 1, 333)])
def test_sweep_of_configurations_equals_one_run_per_configuration(module, batch, hq, hk, t, rows):
    """One launch over a grid of uniform maps (the calibration's inner loop, calibrate.py:46-63 of the reference) gives,
    for each configuration, bit for bit what a separate prefill with that map gives on the rows it returns."""
    q, k, v = (bf16_cuda(x) for x in make_inputs(hq, hk, t, seed=21, batch=batch))
    out, row0 = Prefill(module, bands_fn_of([[INF, INF]] * hq)).sweep(SWEEP, q, k, v, SCALE, rows=rows)
    module.check_device_error()
    wanted = t if rows is None else min(t, rows)
    assert row0 % 256 == 0 and row0 <= t - wanted and t - wanted - row0 < 256
    assert out.shape == (len(SWEEP), batch, hq, t - row0, 128) and out.dtype == torch.bfloat16
    for c, (w8, w4) in enumerate(SWEEP):
        alone = Prefill(module, bands_fn_of([[w8, w4]] * hq))(0, q, k, v, SCALE)[:, :, row0:]
        module.check_device_error()
        if (w8, w4) == (1, 1):
            # no INT8 tile at all: a run of its own keeps V un-normalised (the reference's identity mode), the sweep
            # normalises V for every configuration; the outputs differ by the fp16 rounding of V' only
            assert_fp_close(out[c].float().cpu().numpy(), alone.float().cpu().numpy(), 2e-3, 0.9999)
        else:
            assert torch.equal(out[c], alone), (w8, w4, (out[c].float() - alone.float()).abs().max().item())


def test_sweep_fp16_outputs_and_argument_checks(module):
    hq, hk, t = 2, 1, 520
    q, k, v = (bf16_cuda(x) for x in make_inputs(hq, hk, t, seed=22))
    pre = Prefill(module, bands_fn_of([[INF, INF]] * hq))
    out, row0 = pre.sweep([(2, 4), (1, INF)], q, k, v, SCALE, rows=100, out_dtype=torch.float16)
    module.check_device_error()
    assert row0 == 256 and out.dtype == torch.float16
    alone = Prefill(module, bands_fn_of([[2, 4]] * hq))(0, q, k, v, SCALE, out_dtype=torch.float16)[:, :, row0:]
    assert torch.equal(out[0], alone)
    with pytest.raises(ValueError):
        pre.sweep([(0, 4)], q, k, v, SCALE)
    ops = pre.operands(1, hq, hk, t, True, False, frozenset({1, 2, 4}), q.device)
    bad = torch.empty((1, 1, hq, t, 128), dtype=torch.bfloat16, device=q.device)
    with pytest.raises(RuntimeError):     # row0 must be the first row of the group of four blocks that holds first_block
        module.attention_sweep(torch.ones((1, hq, 2), dtype=torch.int32, device=q.device), 5, ops["v16"], ops["v8h"],
                               ops["vstat"], ops["q8"], ops["k8"], ops["qa"], ops["ka"], ops["q4x"], ops["k4x"], ops["qa4"],
                               ops["ka4"], bad, 0, SCALE, hk, t)
