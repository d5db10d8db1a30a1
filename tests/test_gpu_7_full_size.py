"""Parity at the benchmark configurations' full sizes, one sequence at a time (the reference extension is
batch 1): prefill at 16,384 tokens (config 3) and at the 131,072-token cap (2,048 tiles, config 5's length),
decode over 8,192 (config 2) and 131,072 cached tokens, each against the reference's own kernels on the same
GPU, plus properties that do not depend on the size (an attention output is a convex combination of V rows;
the way the tile sequence is cut over CTAs does not change a decode result beyond summation order)."""
import numpy as np
import pytest
import torch

from ref_harness import RefRunner
from test_gpu_2_kv_write import assert_write_equals_reference, run_write
from triattention_b200.kernels.decode import DecodeCache
from triattention_b200.kernels.prefill import Prefill
from triattention_b200.maps import INF, from_bands
from util import assert_fp_close

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def synth_cuda(shape, seed, fraction=0.01, factor=20.0):
    """bf16 N(0,1) with `fraction` of the (head, channel) pairs scaled by `factor`, generated on the GPU."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, generator=g, device="cuda", dtype=torch.float32)
    heads, dims = shape[-3], shape[-1]
    pick = torch.randperm(heads * dims, generator=g, device="cuda")[:max(1, round(fraction * heads * dims))]
    scale = torch.ones(heads * dims, device="cuda")
    scale[pick] = factor
    return (x * scale.view(heads, 1, dims)).to(torch.bfloat16)


def bands_of(kinds, group):
    """kinds per KV head -> Q-head bands; BF16 heads are quantised as INT8 on the reference side."""
    rows = [[1, INF] if kind == "int4" else [INF, INF] for kind in kinds for _ in range(group)]
    return np.asarray(rows, np.int64), tuple(i for i, kind in enumerate(kinds) if kind == "bf16")


def quantised_q_heads(kinds, group):
    return [h for kh, kind in enumerate(kinds) if kind != "bf16" for h in range(kh * group, (kh + 1) * group)]


def check_convex(out, v, group):
    """Every output channel lies between the smallest and the largest value of that V channel (plus one
    quantisation step of the channel)."""
    vmin, vmax = v.float().amin(dim=2), v.float().amax(dim=2)
    margin = (vmax - vmin) / 127.0 + 0.05
    lo = (vmin - margin).repeat_interleave(group, dim=1)[:, :, None]
    hi = (vmax + margin).repeat_interleave(group, dim=1)[:, :, None]
    o = out.float()
    assert bool(((o >= lo) & (o <= hi)).all())


def assert_close_to_reference(got, ref, v, group, what):
    """The FP tolerance of the parity contract on every element (computed on the GPU: 58.7 M elements at 16,384 tokens):
    cosine >= 0.9999, mean-abs <= 5e-4, and max-abs 2e-3 plus one ulp of the output type at the reference value (both
    sides are rounded to it) —
      * as stated, unscaled, in every V channel of ordinary range (<= 16, i.e. twice that of a unit-variance channel);
      * scaled by range / 8 in wider channels (the benchmark's x20 outlier channels span > 150).  There the reference
        kernel itself is not reproducible to 2e-3: it adds every tile's integer P.V sums, biased by 12582912, into a
        float32 accumulator (prefill_sm80.cu:416-449), and that accumulator's own rounding noise, measured by evaluating
        the same codes and scales in float64 (tests/test_cpu_oracle.py::test_reference_accumulator_noise_floor), reaches
        4e-3 in such a channel within 64 rows.  This kernel sums the same products without the bias and lands between
        the two; what is left against the reference is the reference's noise;
      * and the unscaled bound still holds for all but 1e-5 of the elements (measured: about 1e-6).
    Prints the counts for the record."""
    digits = 7 if got.dtype == torch.bfloat16 else 10
    got, ref = got.float(), ref.float()
    ulp = torch.exp2(torch.floor(torch.log2(ref.abs().clamp_min(2.0 ** -120))) - digits)
    err = (got - ref).abs()
    rng = (v.float().amax(2) - v.float().amin(2)).repeat_interleave(group, 1)[:, :, None, :].expand_as(err)
    scale = (rng / 8.0).clamp_min(1.0)
    excess = float((err - (2e-3 * scale + ulp)).max())
    narrow = rng <= 16.0
    excess_narrow = float((err - (2e-3 + ulp))[narrow].max())
    over = int((err > 2e-3 + ulp).sum())
    cos = float((got.double() * ref.double()).sum() / (got.double().norm() * ref.double().norm()))
    print(f"{what}: elements over the unscaled 2e-3 + 1 ulp: {over} of {err.numel()} (all in channels of range > 16: "
          f"{bool(excess_narrow <= 0)}), worst excess over the unscaled bound {float((err - (2e-3 + ulp)).max()):.5f}, "
          f"mean {float(err.mean()):.2e}, cosine {cos:.7f}")
    assert excess <= 0 and excess_narrow <= 0 and cos >= 0.9999 and float(err.mean()) <= 5e-4, (what, excess, excess_narrow, cos)
    assert over <= 1e-5 * err.numel(), (what, over)


def check_codes(module, o, q, k, v):
    """Bit-exactness of the KV-cache write at this size, with the x20 outlier channels: INT8 and INT4 codes of Q, K and V,
    the fp16 V bits, and the bit patterns of every scale and statistic, against the operand buffers the reference
    extension filled for the same sequence.  The statistics blocks add 128 to 2,048 rows each at these lengths, so
    the summation order is exercised far beyond the small cases."""
    compared = assert_write_equals_reference(run_write(module, q, k, v), 0, o)
    assert {"q8", "q4", "k8", "k4", "v8", "v4", "qa", "qa4", "ka", "ka4"} <= set(compared), compared


def test_prefill_config3_size_vs_reference(module, ref_ext):
    hq, hk, t = 28, 4, 16384
    kinds = ["int8", "int8", "int4", "int8"]
    bands, _ = bands_of(kinds, hq // hk)
    q, k, v = synth_cuda((1, hq, t, 128), 1), synth_cuda((1, hk, t, 128), 2), synth_cuda((1, hk, t, 128), 3)
    got = Prefill(module, from_bands({"0": bands.tolist()}, None))(0, q, k, v, SCALE)
    module.check_device_error()
    o = RefRunner(ref_ext).prefill(q, k, v, bands, SCALE)
    check_codes(module, o, q, k, v)
    ref = o["out"]
    assert_close_to_reference(got, ref, v, hq // hk, "prefill at 16384 tokens")
    check_convex(got, v, hq // hk)
    # once more with fp16 outputs on both sides: the allowance for the final rounding shrinks from 2^-8 to 2^-11 of the value
    got16 = Prefill(module, from_bands({"0": bands.tolist()}, None))(0, q, k, v, SCALE, out_dtype=torch.float16)
    module.check_device_error()
    ref16 = RefRunner(ref_ext).prefill(q, k, v, bands, SCALE, with_decode=False, out_dtype=torch.float16)["out"]
    assert_close_to_reference(got16, ref16, v, hq // hk, "prefill at 16384 tokens, fp16 outputs")


def run_decode(module, q, k, v, bands, bf16, qd, kd, vd, ctas=None):
    cache = DecodeCache(module, max_tail=4, ctas=ctas)
    pre = Prefill(module, from_bands({"0": bands.tolist()}, None, {"0": list(bf16)} if bf16 else None), cache)
    table, ops = pre.write(0, q, k, v)
    cache.store(0, q.shape[2], ops, table.host, k, v, table.bf16_kv)
    out = cache(0, qd, kd, vd, SCALE)
    module.check_device_error()
    return out


def test_decode_config2_size_vs_reference(module, ref_ext):
    hq, hk, t = 24, 8, 8192
    kinds = ["int8", "bf16", "int4", "int8", "int8", "int4", "bf16", "int8"]
    bands, bf16 = bands_of(kinds, hq // hk)
    q, k, v = synth_cuda((1, hq, t, 128), 11), synth_cuda((1, hk, t, 128), 12), synth_cuda((1, hk, t, 128), 13)
    qd, kd, vd = synth_cuda((1, hq, 1, 128), 14), synth_cuda((1, hk, 1, 128), 15), synth_cuda((1, hk, 1, 128), 16)
    got = run_decode(module, q, k, v, bands, bf16, qd, kd, vd)
    run = RefRunner(ref_ext)
    o = run.prefill(q, k, v, bands, SCALE)
    check_codes(module, o, q, k, v)
    st = run.decode_setup(o, bands, max_tail=4, per=8)
    ref = run.decode(st, qd, kd, vd, SCALE)
    heads = quantised_q_heads(kinds, hq // hk)
    assert_fp_close(got.float().cpu().numpy()[0, heads], ref.float().cpu().numpy()[0, heads], "decode over 8192 tokens")
    # un-quantised heads: exact attention over prompt + current token
    for kh in bf16:
        kk, vv = torch.cat([k[0, kh], kd[0, kh]]).float(), torch.cat([v[0, kh], vd[0, kh]]).float()
        for h in range(kh * 3, kh * 3 + 3):
            w = torch.softmax(qd[0, h].float() @ kk.T * SCALE, dim=-1)
            want = (w @ vv).to(torch.bfloat16).float().cpu().numpy()
            assert_fp_close(got[0, h].float().cpu().numpy(), want, f"bf16 head {h}")
    # the cut of the tile sequence over CTAs only changes the summation order
    few = run_decode(module, q, k, v, bands, bf16, qd, kd, vd, ctas=7)
    assert_fp_close(few.float().cpu().numpy(), got.float().cpu().numpy(), "7 CTAs vs one per SM")


def test_max_length_prefill_and_decode_vs_reference(module, ref_ext):
    """131,072 tokens = 2,048 tiles, the cap of both implementations (prefill_sm80.cu:23,518)."""
    hq, hk, t = 8, 2, 131072
    kinds = ["int4", "int8"]
    bands, _ = bands_of(kinds, hq // hk)
    q, k, v = synth_cuda((1, hq, t, 128), 21), synth_cuda((1, hk, t, 128), 22), synth_cuda((1, hk, t, 128), 23)
    qd, kd, vd = synth_cuda((1, hq, 1, 128), 24), synth_cuda((1, hk, 1, 128), 25), synth_cuda((1, hk, 1, 128), 26)
    run = RefRunner(ref_ext)
    o = run.prefill(q, k, v, bands, SCALE)
    check_codes(module, o, q, k, v)
    got = Prefill(module, from_bands({"0": bands.tolist()}, None))(0, q, k, v, SCALE)
    module.check_device_error()
    assert_close_to_reference(got, o["out"], v, hq // hk, "prefill at 131072 tokens")
    st = run.decode_setup(o, bands, max_tail=4, per=64)
    ref = run.decode(st, qd, kd, vd, SCALE)
    dec = run_decode(module, q, k, v, bands, (), qd, kd, vd)
    assert_fp_close(dec.float().cpu().numpy(), ref.float().cpu().numpy(), "decode over 131072 tokens")
    with pytest.raises(RuntimeError):   # one token more than the cap is refused, not truncated
        Prefill(module, from_bands({"0": bands.tolist()}, None))(0, synth_cuda((1, hq, t + 1, 128), 27),
                                                                  synth_cuda((1, hk, t + 1, 128), 28), synth_cuda((1, hk, t + 1, 128), 29), SCALE)
